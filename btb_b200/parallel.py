"""One 8-GPU box, one process a GPU: how the decode path is cut across ranks, and the dense tensor-parallel engine.

btb has no multi-GPU path, so the contract here is bit-identity with the one-GPU arithmetic:

* dense layers (tensor parallel): every linear is cut by OUTPUT rows - q/k/v by kv-head group, o and down by rows of
  the hidden size, gate and up by the same rows of the intermediate size (paired), the head by vocabulary rows - so
  each output element's whole K-sum stays on one GPU in the one-GPU order. What a rank lacks of an activation vector it
  gets by all-gather (16-57 KB a hop at batch 1). Attention is cut by kv head; a rank holds only its heads' cache.
* MoE layers (expert parallel): expert e lives on rank e % N (`btb_b200.moe`); products are exchanged by one all-reduce
  of zeros-elsewhere f32 rows and every rank runs the same ordered sum.
* the greedy pick over a vocabulary cut by rows: each rank's (value, index) best, gathered, the largest value and on
  ties the lowest index - the one-GPU rule.

The host-side pieces (who owns what, how gathered slices are laid out, how picks merge) are plain functions so the
CPU tests can run them over gloo; `TPEngine` is the card engine over them.
"""

from __future__ import annotations

from typing import Any

import torch

from . import capi
from .capi import ptr
from .engine import CardEngine, DenseConfig, LayerWeights, ModelWeights, pad_rows


def row_shard(rows: int, rank: int, world: int) -> tuple[int, int]:
    """rank's contiguous share [lo, hi) of `rows` output rows; `rows` must divide evenly"""
    if rows % world:
        raise ValueError(f"{rows} rows do not cut into {world} equal shards")
    n = rows // world
    return rank * n, (rank + 1) * n


def shard_qkv(qkv: torch.Tensor, cfg: DenseConfig, rank: int, world: int) -> torch.Tensor:
    """the merged q|k|v block cut by kv-head group: rank r keeps its q heads, its k heads, its v heads, merged again"""
    D, Hq, Hk = cfg.head_dim, cfg.q_heads, cfg.kv_heads
    if Hk % world or Hq % world:
        raise ValueError(f"{Hq} q / {Hk} kv heads do not cut into {world} ranks")
    q, k, v = qkv[: Hq * D], qkv[Hq * D : (Hq + Hk) * D], qkv[(Hq + Hk) * D :]
    ql, qh = row_shard(Hq * D, rank, world)
    kl, kh = row_shard(Hk * D, rank, world)
    return torch.cat([q[ql:qh], k[kl:kh], v[kl:kh]]).contiguous()


def shard_gate_up(gu: torch.Tensor, inter: int, rank: int, world: int) -> torch.Tensor:
    """gate | up cut by the same intermediate rows on every rank (the SwiGLU pairs stay together)"""
    lo, hi = row_shard(inter, rank, world)
    return torch.cat([gu[lo:hi], gu[inter + lo : inter + hi]]).contiguous()


def shard_dense(mw: ModelWeights, rank: int, world: int) -> ModelWeights:
    """a rank's share of a dense model: every linear by output rows, norms and rope replicated"""
    c = mw.cfg
    out = ModelWeights(c, mw.embed[slice(*row_shard(c.vocab, rank, world))].contiguous(), mw.norm)
    for L in mw.layers:
        out.layers.append(LayerWeights(
            L.ln1, L.ln2, shard_qkv(L.qkv, c, rank, world), L.o[slice(*row_shard(c.hidden, rank, world))].contiguous(),
            shard_gate_up(L.gu, c.inter, rank, world), L.down[slice(*row_shard(c.hidden, rank, world))].contiguous(),
            L.wq, L.wk))  # fmt: skip
    return out


def gathered_rows(parts: torch.Tensor) -> torch.Tensor:
    """all-gather output [world, M, n] -> the full activation [M, world * n] (rank-major along the features)"""
    w, M, n = parts.shape
    return parts.permute(1, 0, 2).reshape(M, w * n)


def merge_picks(values: torch.Tensor, indices: torch.Tensor, shard: int) -> torch.Tensor:
    """every rank's best (value [world, T], local index [world, T]) of a vocabulary cut into `shard`-row pieces -> the
    global pick [T]: the largest value, the lowest global index on ties"""
    world = values.shape[0]
    gidx = indices + torch.arange(world, device=indices.device, dtype=indices.dtype)[:, None] * shard
    best = values.max(dim=0).values
    cand = torch.where(values == best[None, :], gidx, torch.full_like(gidx, 2**62))
    return cand.min(dim=0).values


class TPEngine(CardEngine):
    """a dense model tensor-parallel over a process group: this rank's row shards, its kv heads' cache"""

    def __init__(self, full_cfg: DenseConfig, shard: ModelWeights, rank: int, world: int, group: Any = None,
                 cap: int = 4096, device: Any = "cuda"):  # fmt: skip
        import dataclasses

        if world < 1 or full_cfg.q_heads % world or full_cfg.kv_heads % world or full_cfg.hidden % (8 * world) \
                or full_cfg.inter % (8 * world) or full_cfg.vocab % world:
            raise ValueError(f"{full_cfg.name} does not cut into {world} ranks")
        self.full, self.rank, self.world, self.group = full_cfg, rank, world, group
        # the local view: this rank's heads; hidden and intermediate stay whole as GEMV input widths
        local = dataclasses.replace(full_cfg, q_heads=full_cfg.q_heads // world, kv_heads=full_cfg.kv_heads // world)
        shard.cfg = local
        super().__init__(shard, cap=cap, step_kernel=False, device=device)
        self._tp: dict[int, dict[str, torch.Tensor]] = {}

    def tp_bufs(self, M: int) -> dict[str, torch.Tensor]:
        if M not in self._tp:
            c, w, dev = self.full, self.world, self.dev
            bf = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)  # noqa: E731
            self._tp[M] = {
                "att_l": bf(M, c.q_heads * c.head_dim // w), "att_g": bf(w, M, c.q_heads * c.head_dim // w),
                "y_l": bf(M, c.hidden // w), "y_g": bf(w, M, c.hidden // w), "att": bf(M, c.q_heads * c.head_dim),
                "y": bf(M, c.hidden), "gu_l": bf(M, 2 * c.inter // w), "m_l": bf(M, c.inter // w),
                "m_g": bf(w, M, c.inter // w), "m": bf(M, c.inter), "lg_l": bf(M, c.vocab // w),
                "pv": torch.zeros(w, M, dtype=torch.float32, device=dev),
                "pi": torch.zeros(w, M, dtype=torch.int64, device=dev),
            }  # fmt: skip
        return self._tp[M]

    def _gather(self, local: torch.Tensor, parts: torch.Tensor, full: torch.Tensor) -> None:
        if self.world == 1:
            full.copy_(local)
            return
        import torch.distributed as dist

        dist.all_gather_into_tensor(parts.view(-1, local.shape[-1]), local, group=self.group)
        full.copy_(gathered_rows(parts))

    def body(self, T: int, tail: bool = True, stream_ptr: int | None = None) -> None:
        c, lc, w = self.full, self.cfg, self.world
        M = pad_rows(T)
        g, t = self.bufs(M), self.tp_bufs(M)
        s = capi.stream_ptr() if stream_ptr is None else stream_ptr
        H, D, I = c.hidden, c.head_dim, c.inter
        K_ = self._k
        y_prev = None
        for i, L in enumerate(self.w.layers):
            K_("btb_b200_add_rmsnorm", ptr(g["h"]), ptr(y_prev), ptr(L.ln1), c.eps, ptr(g["x"]), T, H, 0, s)
            self._matvec(L.qkv, g["x"], g["qkv"], M, lc.qkv_rows, H, s)
            self._attention(g, i, L.wq, L.wk, T, s, out=t["att_l"])  # this rank's heads
            self._gather(t["att_l"], t["att_g"], t["att"])
            self._matvec(L.o, t["att"], t["y_l"], M, H // w, c.q_heads * D, s)
            self._gather(t["y_l"], t["y_g"], t["y"])
            K_("btb_b200_add_rmsnorm", ptr(g["h"]), ptr(t["y"]), ptr(L.ln2), c.eps, ptr(g["x"]), T, H, 0, s)
            self._matvec(L.gu, g["x"], t["gu_l"], M, 2 * I // w, H, s)
            K_("btb_b200_silu_mul", ptr(t["gu_l"]), ptr(t["m_l"]), M, I // w, s)
            self._gather(t["m_l"], t["m_g"], t["m"])
            self._matvec(L.down, t["m"], t["y_l"], M, H // w, I, s)
            self._gather(t["y_l"], t["y_g"], t["y"])
            y_prev = t["y"]
        if tail:
            K_("btb_b200_add_rmsnorm", ptr(g["h"]), ptr(y_prev), ptr(self.w.norm), c.eps, ptr(g["x"]), T, H, 0, s)
            self._matvec(self.w.embed, g["x"], t["lg_l"], M, c.vocab // w, H, s)

    def _embed(self, g: dict, T: int, s: int) -> None:
        """the embedding table is the head, cut by vocabulary rows: the owner of a token's row supplies it, the
        others zeros, and an all-reduce (x + 0, exact) gives every rank the row"""
        V = self.full.vocab // self.world
        ids = g["ids"][:T]
        local = ids - self.rank * V
        mine = (local >= 0) & (local < V)
        rows = self.w.embed[local.clamp(0, V - 1)] * mine[:, None].to(torch.bfloat16)
        if self.world > 1:
            import torch.distributed as dist

            rows = rows.float()
            dist.all_reduce(rows, group=self.group)
        g["h"][:T].copy_(rows.to(torch.bfloat16))
        self._n += 1

    def _pick(self, g: dict, T: int, s: int, out: torch.Tensor) -> None:
        M = pad_rows(T)
        t = self.tp_bufs(M)
        lg = t["lg_l"][:T].float()
        val, idx = lg.max(dim=-1)  # torch's max/argmax return the first of equal maxima: the lowest local index
        if self.world > 1:
            import torch.distributed as dist

            vp = torch.full((M,), float("-inf"), dtype=torch.float32, device=self.dev)
            ip = torch.zeros(M, dtype=torch.int64, device=self.dev)
            vp[:T], ip[:T] = val, idx
            dist.all_gather_into_tensor(t["pv"].view(-1), vp, group=self.group)
            dist.all_gather_into_tensor(t["pi"].view(-1), ip, group=self.group)
            out[:T].copy_(merge_picks(t["pv"][:, :T], t["pi"][:, :T], self.full.vocab // self.world))
        else:
            out[:T].copy_(idx)
        self._n += 1

    def forward(self, ids: torch.Tensor, depth: Any = None, parents: Any = None, advance: bool = True) -> torch.Tensor:
        """a pass; returns THIS RANK'S logits slice [T, V / world]"""
        super().forward(ids, depth, parents, advance)
        return self.tp_bufs(pad_rows(int(ids.numel())))["lg_l"][: int(ids.numel())]

    def prefill(self, prompt: torch.Tensor) -> torch.Tensor:
        lg = None
        for a in range(0, int(prompt.numel()), 32):
            lg = self.forward(prompt[a : a + 32])
        assert lg is not None
        return lg[-1:]

    def generate_greedy(self, prompt: Any, max_new: int, graph_steps: int = 1) -> list[int]:
        prompt = torch.as_tensor(prompt, dtype=torch.int64)
        self.reset()
        self.prefill(prompt)
        g = self.bufs(1)
        s = capi.stream_ptr()
        n = int(prompt.numel())
        last_M = pad_rows(n - (n - 1) // 32 * 32)
        # the last prompt row's slice sits in the last pass's buffer
        t = self.tp_bufs(last_M)
        keep = t["lg_l"][(n - 1) % 32 : (n - 1) % 32 + 1].clone()
        self.tp_bufs(1)["lg_l"][:1].copy_(keep)
        self._pick(g, 1, s, g["ids"])
        toks = [int(g["ids"][0].item())]
        while len(toks) < max_new:
            self._step_body_launches(s, publish=False)
            torch.cuda.current_stream().synchronize()
            toks.append(int(g["ids"][0].item()))
        return toks
