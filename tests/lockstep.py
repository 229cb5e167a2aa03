"""TEST INFRASTRUCTURE. N tensor-parallel ranks as N engines of ONE process on ONE GPU, taking turns.

The exchange kernels wait for arrivals from every rank, so ranks must never be separate launches that wait on each other
on one GPU. Here they do not: the engines' passes advance piece by piece (`TPEngine.ops` yields after every piece that
ends in an exchange), every engine launching a piece before any engine launches the next, all on one stream - so each
consumer's arrivals are complete before it starts, and the N-rank data path (slices, offsets, strides, arrival counts,
the merged pick) runs for real on a single card."""

from __future__ import annotations

import torch

from btb_b200 import capi
from btb_b200 import engine as E
from btb_b200 import parallel as P
from btb_b200.capi import call, ptr
from btb_b200.exchange import PeerHeap


def make(cfg: E.DenseConfig, weights_of, world: int, cap: int = 512) -> list[P.TPEngine]:
    """`world` engines over shards of the model `weights_of()` draws (called once a rank: a shard keeps views)"""
    heaps = [PeerHeap(P.TPEngine.heap_bytes(cfg), r, world) for r in range(world)]
    PeerHeap.connect_engines(heaps)
    return [P.TPEngine(cfg, P.shard_dense(weights_of(), r, world), r, world, cap=cap, heap=heaps[r]) for r in range(world)]


def forward(engs: list[P.TPEngine], ids: torch.Tensor, advance: bool = True) -> list[torch.Tensor]:
    """one chain pass on every rank; returns each rank's logits slice"""
    T = int(ids.numel())
    M = E.pad_rows(T)
    s = capi.stream_ptr()
    for e in engs:
        g = e.bufs(M)
        g["ids"][:T].copy_(ids.to(e.dev, torch.int64))
        g["depth"][:M].copy_(torch.arange(M, dtype=torch.int32))
        g["par"][:M].copy_(torch.arange(-1, M - 1, dtype=torch.int32))
        e._embed(g, T, s)
    for _ in zip(*[e.ops(T) for e in engs], strict=True):
        pass
    for e in engs:
        if advance:
            call("btb_b200_publish", ptr(e.n0), 0, 0, 0, 0, T, s)
        e.tick(M, s)
    return [e.tp_bufs(M)["lg_l"][:T] for e in engs]


def greedy(engs: list[P.TPEngine], prompt, max_new: int) -> list[list[int]]:
    """every rank's greedy tokens (they must agree)"""
    prompt = torch.as_tensor(prompt, dtype=torch.int64)
    s = capi.stream_ptr()
    for e in engs:
        e.reset()
    last = None
    for a in range(0, int(prompt.numel()), 32):
        last = forward(engs, prompt[a : a + 32])
    keep = [lg[-1:].contiguous() for lg in last]

    def pick(logits_of) -> None:
        for phase in (1, 2):  # every rank's key is sent before any rank merges
            for e, lg in zip(engs, logits_of):
                e._pick({} if lg is None else {"logits_l": lg}, 1, s, e.bufs(1)["ids"], phase=phase, body_pass=lg is None)

    pick(keep)
    toks = [[int(e.bufs(1)["ids"][0].item())] for e in engs]
    while len(toks[0]) < max_new:
        for e in engs:
            e._embed(e.bufs(1), 1, s)
        for _ in zip(*[e.ops(1) for e in engs], strict=True):
            pass
        pick([None] * len(engs))
        for e, tk in zip(engs, toks):
            call("btb_b200_publish", ptr(e.n0), 0, 0, 0, 0, 1, s)
            tk.append(int(e.bufs(1)["ids"][0].item()))
    return toks


# ---- expert parallelism -------------------------------------------------------------------------------------------------


def make_moe(cfg, world: int, seed: int, layer_std: float, cap: int = 512):
    """`world` MoE engines, rank r holding expert e iff e % world == r, over one seeded model"""
    from btb_b200 import moe as MO

    heaps = [PeerHeap(MO.MoEEngine.heap_bytes(cfg), r, world) for r in range(world)]
    PeerHeap.connect_engines(heaps)
    return [MO.MoEEngine(MO.synth_moe_weights(cfg, seed=seed, on_cpu=True, ep_rank=r, ep_size=world, layer_std=layer_std),
                         cap=cap, heap=heaps[r]) for r in range(world)]  # fmt: skip


def moe_forward(engs, ids: torch.Tensor) -> list[torch.Tensor]:
    """one chain pass on every rank (every rank holds the whole logits row)"""
    T = int(ids.numel())
    M = E.pad_rows(T)
    s = capi.stream_ptr()
    for e in engs:
        g = e.bufs(M)
        g["ids"][:T].copy_(ids.to(e.dev, torch.int64))
        g["depth"][:M].copy_(torch.arange(M, dtype=torch.int32))
        g["par"][:M].copy_(torch.arange(-1, M - 1, dtype=torch.int32))
        e._embed(g, T, s)
    for _ in zip(*[e.ops(T) for e in engs], strict=True):
        pass
    for e in engs:
        call("btb_b200_publish", ptr(e.n0), 0, 0, 0, 0, T, s)
    return [e.bufs(M)["logits"][:T] for e in engs]


def moe_greedy(engs, prompt, max_new: int) -> list[list[int]]:
    prompt = torch.as_tensor(prompt, dtype=torch.int64)
    for e in engs:
        e.reset()
    last = None
    for a in range(0, int(prompt.numel()), 32):
        last = moe_forward(engs, prompt[a : a + 32])
    toks = [[int(lg[-1].float().argmax())] for lg in last]
    while len(toks[0]) < max_new:
        lgs = moe_forward(engs, torch.tensor([toks[0][-1]]))
        for tk, lg in zip(toks, lgs):
            tk.append(int(lg[-1].float().argmax()))
    return toks
