"""The multi-GPU cut on CPU ranks (gloo, world size 2): who owns which rows, heads and experts, how gathered slices are
laid out and how picks merge - with the oracle standing in for the card's arithmetic. The sharded result must be the
one-process result to the bit."""

import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from btb_b200 import parallel as P
from btb_b200.engine import DenseConfig
from oracle import oracle as O

CFG = DenseConfig("tp", hidden=128, layers=1, q_heads=4, kv_heads=2, head_dim=32, inter=192, vocab=96)


def _bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def _bf(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        c = CFG
        D = c.head_dim
        rnd = lambda r, k: (torch.randn(r, k, generator=g) * 0.05).to(torch.bfloat16)  # noqa: E731
        qkv, o, gu, down = rnd(c.qkv_rows, c.hidden), rnd(c.hidden, c.q_heads * D), rnd(2 * c.inter, c.hidden), rnd(c.hidden, c.inter)
        head = rnd(c.vocab, c.hidden)
        x = rnd(3, c.hidden)
        gemv = lambda w, v: _bf(O.gemv_card_bf16(_bits(w), _bits(v)))  # noqa: E731

        def gather(local):
            parts = torch.zeros(world, *local.shape, dtype=torch.float32)
            dist.all_gather_into_tensor(parts.view(-1, local.shape[-1]), local.float())
            return P.gathered_rows(parts).to(torch.bfloat16)

        ok = True
        # q|k|v by kv-head group: the gathered q, k, v slices are the full projection's
        full = gemv(qkv, x)
        loc = gemv(P.shard_qkv(qkv, c, rank, world), x)
        nq, nk = c.q_heads * D // world, c.kv_heads * D // world
        q, k, v = gather(loc[:, :nq].contiguous()), gather(loc[:, nq : nq + nk].contiguous()), gather(loc[:, nq + nk :].contiguous())
        ok &= torch.equal(torch.cat([q, k, v], 1).view(torch.int16), full.view(torch.int16))
        # o / down by output rows
        att = rnd(3, c.q_heads * D)
        lo, hi = P.row_shard(c.hidden, rank, world)
        ok &= torch.equal(gather(gemv(o[lo:hi].contiguous(), att)).view(torch.int16), gemv(o, att).view(torch.int16))
        # gate | up paired, the activation local, then the down projection over the gathered product
        gul = gemv(P.shard_gate_up(gu, c.inter, rank, world), x)
        m_full = _bf(O.silu_mul(_bits(gemv(gu, x))))
        m = gather(_bf(O.silu_mul(_bits(gul))))
        ok &= torch.equal(m.view(torch.int16), m_full.view(torch.int16))
        ok &= torch.equal(gather(gemv(down[lo:hi].contiguous(), m)).view(torch.int16), gemv(down, m_full).view(torch.int16))
        # the pick over a vocabulary cut by rows, with a tie across the cut
        lg = gemv(head, x).float()
        lg[0, 5] = lg[0, 70] = 99.0
        lg[1, 60] = 98.0
        vl, vh = P.row_shard(c.vocab, rank, world)
        val, idx = lg[:, vl:vh].max(dim=-1)
        pv, pi = torch.zeros(world, 3), torch.zeros(world, 3, dtype=torch.int64)
        dist.all_gather_into_tensor(pv.view(-1), val)
        dist.all_gather_into_tensor(pi.view(-1), idx)
        pick = P.merge_picks(pv, pi, c.vocab // world)
        ok &= pick.tolist() == lg.argmax(-1).tolist() and int(pick[0]) == 5
        # expert parallelism: a rank's own picks, zeros elsewhere, one all-reduce
        idx_e = torch.tensor([[3, 0, 6], [1, 2, 5]])
        prod = torch.randn(2, 3, 16, generator=g)
        mine = (idx_e % world == rank)[..., None]
        part = torch.where(mine, prod, torch.zeros_like(prod))
        dist.all_reduce(part)
        ok &= torch.equal(part, prod)
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_cpu_ranks_reproduce_one_process():
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, 29500 + os.getpid() % 1000, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}


def test_shards_refuse_uneven_cuts():
    with pytest.raises(ValueError):
        P.row_shard(10, 0, 4)
    with pytest.raises(ValueError):
        P.shard_qkv(torch.zeros(CFG.qkv_rows, 8), CFG, 0, 3)
