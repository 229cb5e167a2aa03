"""The paged cache on the card: the kernels read and write through the row map, so a conversation whose pages lie
anywhere in the pool decodes the contiguous engine's tokens; a second conversation with the same start takes over the
first one's pages and prefills only its own tail; pages go back to the pool with their last holder."""

import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from btb_b200 import capi  # noqa: E402
from btb_b200 import engine as E  # noqa: E402
from btb_b200.paged import PAGE, PagedEngine, PoolError  # noqa: E402

from .util import LAYER_STD, lively  # noqa: E402

CFG = E.DenseConfig("paged", hidden=256, layers=3, q_heads=8, kv_heads=2, head_dim=128, inter=512, vocab=1000)


def test_paged_conversations_decode_the_contiguous_engines_tokens_and_share_their_prefix():
    mw = E.synth_weights(CFG, seed=0, on_cpu=True, layer_std=LAYER_STD)
    flat = E.CardEngine(mw, cap=1024)
    eng = PagedEngine(mw, n_pages=12)
    # scatter the pool: the first pages handed out are not the first pages of the arena
    held = [eng.pool.alloc() for _ in range(3)]
    eng.pool.unref(held[1])
    g = torch.Generator().manual_seed(3)
    start = torch.randint(0, CFG.vocab, (150,), generator=g)
    pa = torch.cat([start, torch.randint(0, CFG.vocab, (23,), generator=g)])
    pb = torch.cat([start, torch.randint(0, CFG.vocab, (40,), generator=g)])
    want_a, want_b = flat.generate_greedy(pa, 20), flat.generate_greedy(pb, 20)
    lively(want_a)
    ca, la = eng.attach(pa)
    assert ca.shared == 0 and ca.pages[0].id == 1  # the page freed above, not page 0
    got_a = eng.decode(ca, int(la.float().argmax()), 20)
    assert got_a == want_a
    launches = []
    eng._k_orig, n = eng._k, [0]

    def counting(name, *a):
        n[0] += name == "btb_b200_embed"
        eng._k_orig(name, *a)

    eng._k = counting
    cb, lb = eng.attach(pb)
    eng._k = eng._k_orig
    # the first two pages of the common start are the first conversation's; only the rest was computed
    assert cb.shared == 2 * PAGE and [p.id for p in cb.pages[:2]] == [p.id for p in ca.pages[:2]]
    assert n[0] == -(-(len(pb) - 2 * PAGE) // 32), launches
    assert all(p.refs == 3 for p in cb.pages[:2])  # two conversations and the tree
    got_b = eng.decode(cb, int(lb.float().argmax()), 20)
    assert got_b == want_b
    # the first conversation goes on where it stood, its rows untouched by the second's
    more = eng.decode(ca, got_a[-1], 6)
    assert more == flat.generate_greedy(pa, 25)[19:]
    torch.cuda.synchronize()
    assert capi.status() == 0
    ca.release(), cb.release()
    assert eng.pool.check() == []
    assert all(n_.page.refs == 1 for n_ in eng.tree._nodes())  # the tree alone keeps the computed pages
    # a third conversation finds the whole common start (and the first one's third page) without anyone holding it
    cc, _ = eng.attach(pa)
    assert cc.shared == 2 * PAGE
    cc.release()
    # the pool runs short: unheld pages leave the tree, held ones refuse
    keep = []
    with pytest.raises(PoolError):
        while True:
            keep.append(eng._page())
    assert len(eng.tree) == 0
    for p in keep + [held[0], held[2]]:
        eng.pool.unref(p)
    assert len(eng.pool) == 0
