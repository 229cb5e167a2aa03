"""The session's host logic over a stand-in engine (no card): states, feed / mark / rewind / crop bookkeeping and refusals."""

import pytest
import torch

from btb_b200.session import Mark, Session, State


class FakeEngine:
    """logits of a pass's row t = one-hot of (sum of all tokens up to and including t) mod V: any wrong cache length shows"""

    V, cap = 50, 64

    def __init__(self):
        self.n0 = torch.zeros(1, dtype=torch.int32)
        self.rows: list[int] = []
        self.fail_next = False

    def reset(self):
        self.n0.zero_()

    def forward(self, ids):
        if self.fail_next:
            self.fail_next = False
            raise RuntimeError("the pass failed")
        n = int(self.n0)
        del self.rows[n:]
        out = torch.zeros(len(ids), self.V)
        for t, tok in enumerate(ids.tolist()):
            self.rows.append(int(tok))
            out[t, sum(self.rows) % self.V] = 1.0
        self.n0 += len(ids)
        return out

    def continue_from(self, logits, max_new, sampling=None):
        toks = [int(logits.argmax())]
        while len(toks) < max_new:
            toks.append(int(self.forward(torch.tensor([toks[-1]]))[0].argmax()))
        return toks


def test_states_feed_and_generate():
    s = Session(FakeEngine())
    assert s.state is State.EMPTY and s.fresh and len(s) == 0
    with pytest.raises(ValueError):
        s.feed([])
    with pytest.raises(ValueError):
        s.generate(3)
    st = s.feed([1, 2, 3])
    assert st.logits.shape == (3, 50) and st.logits.argmax(-1).tolist() == [1, 3, 6]
    assert s.state is State.READY and s.tokens == [1, 2, 3] and s.n_prompt == 3
    new = s.generate(4)
    assert new == [6, 12, 24, 48] and s.state is State.PENDING and len(s) == 7
    assert s.ids == [1, 2, 3, 6, 12, 24] and s.tokens[-1] == 48
    # a pending token is fed ahead of the next feed; its logits are not part of the step
    st = s.feed([5], last_only=False)
    assert st.logits.shape == (1, 50) and s.ids[-2:] == [48, 5] and s.state is State.READY
    assert int(st.logits.argmax()) == sum(s.ids) % 50
    assert s.feed([7, 7], last_only=True).logits.shape == (1, 50)


def test_mark_rewind_and_crop():
    eng = FakeEngine()
    s = Session(eng)
    s.feed([4, 5, 6])
    m = s.mark()
    assert m == Mark(3, None, m.logits, (4, 5, 6)) and int(m.logits.argmax()) == 15
    draft = s.feed([9, 9, 9]).logits.argmax(-1).tolist()
    assert draft == [24, 33, 42]
    s.rewind(m)
    assert s.tokens == [4, 5, 6] and int(eng.n0) == 3 and s.state is State.READY
    assert int(s.next_logits().argmax()) == 15
    # a decode from the mark is a fresh session's
    a = s.generate(3)
    f = Session(FakeEngine())
    f.feed([4, 5, 6])
    assert a == f.generate(3)
    # a mark taken while Pending brings the pending token back
    mp = s.mark()
    assert mp.pending == a[-1] and mp.logits is None
    s.feed([1])
    s.rewind(mp)
    assert s.state is State.PENDING and s.tokens[-1] == a[-1]
    with pytest.raises(ValueError):
        s.rewind(Mark(99))
    s.rewind(m)
    s.feed([8])
    with pytest.raises(ValueError):  # the session went another way since the later mark was taken
        s.rewind(mp)
    s.crop(2)
    assert s.ids == [4] and s.tokens == [4, 5] and s.state is State.PENDING and int(eng.n0) == 1
    assert int(s.next_logits().argmax()) == 9
    with pytest.raises(ValueError):
        s.crop(0)


def test_a_failed_pass_leaves_the_session_as_it_was():
    eng = FakeEngine()
    s = Session(eng)
    s.feed([1, 2])
    eng.fail_next = True
    with pytest.raises(RuntimeError):
        s.feed([3, 4])
    assert s.tokens == [1, 2] and int(eng.n0) == 2 and s.state is State.READY
    assert s.feed([3]).logits.argmax(-1).tolist() == [6]
    with pytest.raises(ValueError):
        s.feed(list(range(100)))  # past the cache
    assert s.tokens == [1, 2, 3]
