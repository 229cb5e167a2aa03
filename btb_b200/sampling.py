"""How a token is picked: greedy, or temperature / top-k / top-p with a Gumbel-max draw keyed by (seed, cache row).

Mirrors btb's `Sampling` (btb/sampling.py:34-61: the fields, `greedy`, `masked`, `key_for`) and the card sampler's
device-side configuration (btb/engine/cuda.py:2131-2143: ``fp = [1/T, top_p]`` and the seed live in device buffers
filled before a replay, so one captured graph serves every temperature, top-p and seed; top-k is a launch parameter).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from .capi import call, ptr

_M64 = 0xFFFFFFFFFFFFFFFF


def _mix(*parts: int) -> int:
    """splitmix64 folded over the parts, 63 bits (btb/sampling.py:22-31)"""
    x = 0
    for p in parts:
        x = ((x ^ (int(p) & _M64)) + 0x9E3779B97F4A7C15) & _M64
        x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
        x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
        x ^= x >> 31
    return x & 0x7FFFFFFFFFFFFFFF


@dataclass(frozen=True)
class Sampling:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    seed: int | None = None

    def __post_init__(self) -> None:
        if not (self.temperature >= 0.0) or not (0.0 <= self.top_p <= 1.0) or self.top_k < 0:
            raise ValueError(f"sampling out of range: {self}")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def masked(self) -> bool:
        return self.top_k > 0 or self.top_p < 1.0

    def key_for(self, pos: int, salt: int = 0) -> int:
        """the noise key of the pick decided at cache row `pos`"""
        return _mix(self.seed or 0, pos, salt) if salt else _mix(self.seed or 0, pos)


class CardSampler:
    """a `Sampling` on the card: its parameters in device buffers and the one-launch pick over a pass's logits"""

    def __init__(self, device: Any):
        self.dev = torch.device(device)
        self.fp = torch.ones(2, dtype=torch.float32, device=self.dev)
        self.seed = torch.zeros(1, dtype=torch.int64, device=self.dev)
        self.top_k = 0
        self.sampling = Sampling()

    def set(self, s: Sampling) -> None:
        """new parameters; temperature, top-p and seed reach a captured graph as data, top-k needs a new capture"""
        self.sampling = s
        if not s.greedy:
            self.fp.copy_(torch.tensor([1.0 / s.temperature, s.top_p], dtype=torch.float32))
            self.seed.copy_(torch.tensor([(s.seed or 0) & 0x7FFFFFFFFFFFFFFF], dtype=torch.int64))
            self.top_k = int(s.top_k)

    def pick(self, logits: torch.Tensor, T: int, n0: torch.Tensor, depth: torch.Tensor | None, out: torch.Tensor,
             stream: int, keys: torch.Tensor | None = None, floors: torch.Tensor | None = None) -> None:  # fmt: skip
        """out[:T] = the draw of each of the T rows of `logits` (bf16 or f32, row-major); row r keyed by
        key_for(n0 + depth[r]) unless `keys` (int64 [T]) gives them"""
        V = int(logits.shape[-1])
        call("btb_b200_sample_pick", ptr(logits), int(logits.dtype == torch.float32), T, V, int(logits.stride(0)),
             ptr(self.fp), self.top_k, ptr(keys), ptr(self.seed), ptr(n0), ptr(depth), 0, ptr(out), ptr(floors), 0, stream)


class Verify:
    """The pick of a verify pass whose rows are tree nodes with drafted children (btb/sampling.py:272-372): at a node the
    children are tried in draw order, child i accepted with probability min(1, p_i(c) / q_i(c)), p_i the target after the
    earlier rejections' residuals and q_i the drafter's distribution with the earlier children removed; none accepted, a
    draw from the residual - so the emitted token is a draw from the target at every node. A row without a distribution
    (its drafts are point masses) draws from the target and accepts the child equal to the draw. `pick` returns packed
    outcomes (slot + 1) << 24 | token, slot -1 for none; one launch on the card, no host fallback."""

    greedy = False
    MAX_KIDS = 32

    def __init__(self, sampling: Sampling, q: torch.Tensor, kids: Any, hasq: Any) -> None:
        self.sampling = sampling
        self.q = q  # [T, Vd] the rows' distributions, zeros where hasq is False
        self.kids = [list(k) for k in kids]
        self.hasq = [bool(h) for h in hasq]
        self.width = max((len(k) for k in self.kids), default=0)
        if self.width > self.MAX_KIDS:
            raise ValueError(f"verify: {self.width} children a node; the kernel's table holds {self.MAX_KIDS}")

    @property
    def temperature(self) -> float:
        return self.sampling.temperature

    def key_for(self, pos: int) -> int:
        return self.sampling.key_for(pos)

    @staticmethod
    def unpack(v: int) -> tuple[int, int]:
        """(the accepted child's slot, -1 for none; the token)"""
        v = int(v)
        return (v >> 24) - 1, v & 0xFFFFFF

    def pick(self, logits: torch.Tensor, keys: Any, stream: int | None = None) -> torch.Tensor:
        """`logits` [T, V] on the card (bf16 or f32), `keys` one a row; [T] int64 packed outcomes"""
        if logits.device.type != "cuda":
            raise RuntimeError("Verify.pick runs on the card only")
        s, dev = self.sampling, logits.device
        T, V = int(logits.shape[0]), int(logits.shape[1])
        w = max(1, self.width)  # a pass without drafts still carries one (empty) slot a row
        kids = torch.tensor([[*k, *([-1] * (w - len(k)))] for k in self.kids], dtype=torch.int32, device=dev).reshape(T, w)
        hasq = torch.tensor([int(h) for h in self.hasq], dtype=torch.int32, device=dev)
        q = self.q.to(dev, torch.float32).contiguous()
        kk = torch.tensor([int(k) & 0x7FFFFFFFFFFFFFFF for k in keys], dtype=torch.int64, device=dev)
        fp = torch.tensor([1.0 / s.temperature, float(s.top_p)], dtype=torch.float32, device=dev)
        out = torch.empty(T, dtype=torch.int32, device=dev)
        if logits.dtype not in (torch.float32, torch.bfloat16) or logits.stride(1) != 1:
            logits = logits.float().contiguous()
        st = torch.cuda.current_stream().cuda_stream if stream is None else stream
        call("btb_b200_sample_verify", ptr(logits), int(logits.dtype == torch.float32), T, V, int(logits.stride(0)), ptr(q),
             int(q.shape[1]), ptr(kids), w, ptr(hasq), ptr(kk), int(s.top_k), ptr(fp), ptr(out), st)  # fmt: skip
        return out.to(torch.int64) & 0xFFFFFFFF
