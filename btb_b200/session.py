"""A session over the card engine: the tokens the cache holds, the cache's length, and the calls a loop of one's own is
built from - `feed`, `mark`, `rewind`, `crop`, `generate`.

Mirrors btb's `Session` (btb/session.py:247-560: `State` :41-48, `Step` :51-59, `Mark` :73-85, `feed` :360-381, `mark`
:442-453, `rewind` :455-470, `crop`, `generate` :548-552) for what the card path holds: a dense attention cache, which is cut
back by moving its length (no recurrent states to restore). A session is `Empty`, `Ready` (every token in the cache and the
next token's logits in hand) or `Pending` (the last token drawn by a decode and not fed yet); a call that fails part way
leaves the session as it was.
"""

from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Any, Sequence

import torch


class State(enum.Enum):
    EMPTY = "empty"
    READY = "ready"
    PENDING = "pending"


@dataclass(frozen=True, eq=False)
class Step:
    """what a feed gives back: the logits after each fed token, float32 [T, V] ([1, V] with `last_only`)"""

    logits: torch.Tensor
    hidden: dict = field(default_factory=dict)


@dataclass(frozen=True)
class Mark:
    """a point of a session to rewind to: the rows its cache held, the token drawn but not yet fed or the next token's
    logits, and the tokens it was taken on (a rewind from a session that has since gone another way is refused)"""

    n: int
    pending: int | None = None
    logits: torch.Tensor | None = None
    path: tuple[int, ...] | None = None


class Session:
    """bound to one engine (`CardEngine` or a subclass with `forward`, `n0`, `cap`, `generate`); one session at a time owns
    the engine's cache"""

    CHUNK = 32  # rows a pass carries at most (btb/engine/cuda.py CARD_T_MAX)

    def __init__(self, engine: Any) -> None:
        self.engine = engine
        self.ids: list[int] = []  # the tokens whose rows stand in the cache
        self.n_prompt = 0
        self._pending: int | None = None
        self.logits: torch.Tensor | None = None  # the next token's logits [V] f32 when Ready
        self._held = False  # whether the engine's cache is this session's

    # -- what it holds ---------------------------------------------------------------------------------------------------
    @property
    def tokens(self) -> list[int]:
        """the sequence: the cache's tokens and, when Pending, the token drawn after them"""
        return self.ids if self._pending is None else [*self.ids, self._pending]

    def __len__(self) -> int:
        return len(self.ids) + (self._pending is not None)

    @property
    def state(self) -> State:
        if not self.ids and self._pending is None:
            return State.EMPTY
        return State.PENDING if self._pending is not None else State.READY

    @property
    def fresh(self) -> bool:
        return self.state is State.EMPTY

    # -- the cache under the session ---------------------------------------------------------------------------------------
    def _take(self) -> None:
        """the engine's cache stands at this session's rows (it is the session's from its first feed on)"""
        eng = self.engine
        if not self._held:
            eng.reset()
            self._held = True
        eng.n0.fill_(len(self.ids))

    def _run(self, new: list[int], last_only: bool) -> torch.Tensor:
        """`new` after the cache's rows, in passes of up to CHUNK rows; the logits after each, f32 [len(new), V]"""
        eng = self.engine
        if len(self.ids) + len(new) > int(eng.cap):
            raise ValueError(f"{len(self.ids) + len(new)} rows in a cache of {int(eng.cap)}")
        self._take()
        out = []
        for a in range(0, len(new), self.CHUNK):
            lg = eng.forward(torch.tensor(new[a : a + self.CHUNK], dtype=torch.int64))
            out.append(lg[-1:].float() if last_only else lg.float())  # (a copy: the pass's buffer is the next pass's)
        return out[-1] if last_only else torch.cat(out)

    # -- the public surface ---------------------------------------------------------------------------------------------------
    def feed(self, ids: Sequence[int], last_only: bool = False) -> Step:
        """Append `ids`: a `Step` of the logits after each of them ([1, V] with `last_only`). A pending token is fed ahead
        of them; its logits are not part of the step."""
        new = [int(t) for t in ids]
        if not new:
            raise ValueError("feed needs at least one token")
        lead = 0 if self._pending is None else 1
        run = new if not lead else [self._pending, *new]
        n_before = len(self.ids)
        try:
            out = self._run(run, last_only)
        except Exception:
            if self._held:
                self.engine.n0.fill_(n_before)  # the rows a failed pass wrote are past the length again
            raise
        self.ids.extend(run)
        self._pending, self.logits = None, out[-1].clone()
        if not self.n_prompt:
            self.n_prompt = len(self.ids)
        return Step(out if last_only else out[lead:])

    def next_logits(self) -> torch.Tensor:
        """the next token's logits [V]: a pending token is fed first"""
        if self.state is State.EMPTY:
            raise ValueError("an empty session has nothing to go on from: feed it a prompt first")
        if self._pending is not None:
            tok, self._pending = self._pending, None
            try:
                out = self._run([tok], True)
            except Exception:
                self._pending = tok
                raise
            self.ids.append(tok)
            self.logits = out[-1].clone()
        assert self.logits is not None
        return self.logits

    def mark(self) -> Mark:
        """this point of the sequence, to `rewind` to later"""
        return Mark(len(self.ids), self._pending, self.logits, tuple(self.tokens))

    def rewind(self, mark: Mark) -> None:
        """Back to `mark`: everything after it is dropped from the tokens and the cache. A decode from here is the one a
        fresh session at that point gives."""
        if mark.n + (mark.pending is not None) > len(self):
            raise ValueError(f"a mark at {mark.n} is past the session's {len(self)} tokens")
        if mark.path is not None and tuple(self.tokens[: len(mark.path)]) != mark.path:
            raise ValueError("this mark is not on the session's path: the tokens before it have changed since it was taken")
        del self.ids[mark.n :]
        self._pending, self.logits = mark.pending, mark.logits
        self.n_prompt = min(self.n_prompt, mark.n)
        if self._held:
            self.engine.n0.fill_(len(self.ids))

    def crop(self, n: int) -> None:
        """keep the first `n` tokens: the rows past them are dropped and the n-th token becomes the pending one (the logits
        that followed it went with the rows), so the next feed or decode runs it again"""
        n = int(n)
        if not 0 < n <= len(self):
            raise ValueError(f"crop to {n} of {len(self)} tokens")
        toks = self.tokens[:n]
        self.ids, self._pending, self.logits = toks[:-1], toks[-1], None
        self.n_prompt = min(self.n_prompt, n)
        if self._held:
            self.engine.n0.fill_(len(self.ids))

    def generate(self, max_new: int, sampling: Any = None) -> list[int]:
        """decode on from where the sequence stands: `max_new` new tokens (the engine's captured step loop); the session
        ends Pending on the last of them"""
        if self.state is State.EMPTY:
            raise ValueError("an empty session has nothing to go on from: feed it a prompt first")
        if max_new <= 0:
            return []
        eng = self.engine
        lg = self.next_logits()
        self._take()
        new = eng.continue_from(lg, int(max_new), sampling)
        self.ids.extend(new[:-1])
        self._pending, self.logits = new[-1], None
        return new
