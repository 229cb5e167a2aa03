"""One 8-GPU box, one process a GPU: how the decode path is cut across ranks, and the dense tensor-parallel engine.

btb has no multi-GPU path, so the contract here is bit-identity with the one-GPU arithmetic:

* dense layers (tensor parallel): every linear is cut by OUTPUT rows - q/k/v by kv-head group, o and down by rows of
  the hidden size, gate and up by the same rows of the intermediate size (paired), the head by vocabulary rows - so
  each output element's whole K-sum stays on one GPU in the one-GPU order. Attention is cut by kv head; a rank holds
  only its heads' cache. What a rank lacks of an activation vector its peers write into its memory: the producing
  kernel's epilogue stores every finished element into every rank's copy and counts its CTAs' arrivals, the consuming
  kernel's prologue waits on its local counter (csrc/tp.cuh) - four such hops a layer, no collective call, no reduction
  (hence no change of summation order), and the whole step stays one captured CUDA graph.
* the greedy pick over a vocabulary cut by rows: each rank's (value, index) best goes to every rank, which takes the
  largest value and on ties the lowest index - the one-GPU rule.
* MoE layers (expert parallel): expert e lives on rank e % N (`btb_b200.moe`).

The host-side pieces (who owns what, how gathered slices are laid out, how picks merge) are plain functions so the
CPU tests can run them over gloo; `TPEngine` is the card engine over them.
"""

from __future__ import annotations

from typing import Any

import torch

import ctypes as C

from . import capi
from .capi import ptr
from .engine import CARD_ROWS, CardEngine, DenseConfig, LayerWeights, ModelWeights, pad_rows
from .exchange import FLAG_BYTES, PeerHeap


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
    # the embedding table stays whole on every rank (a step reads one row of it); the head is this rank's rows of it
    out = ModelWeights(c, mw.embed, mw.norm, head=mw.embed[slice(*row_shard(c.vocab, rank, world))])
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
    """a dense model tensor-parallel over the ranks of one box: this rank's row shards, its kv heads' cache, and the
    peer-store exchange (module docstring). `heap`: a `PeerHeap` already connected to the other ranks' (the lockstep
    emulation hands engines of one process each other's); None: one is made and connected through `group`."""

    XCHG = ("att", "yo", "m", "yd")  # the four vectors a layer exchanges, in order

    def __init__(self, full_cfg: DenseConfig, shard: ModelWeights, rank: int, world: int, group: Any = None,
                 cap: int = 4096, device: Any = "cuda", heap: PeerHeap | None = None):  # fmt: skip
        import dataclasses

        if world < 1 or world > 8 or full_cfg.q_heads % world or full_cfg.kv_heads % world \
                or full_cfg.hidden % (8 * world) or full_cfg.inter % (8 * world) or full_cfg.vocab % world:
            raise ValueError(f"{full_cfg.name} does not cut into {world} ranks")
        self.full, self.rank, self.world, self.group = full_cfg, rank, world, group
        # the local view: this rank's heads; hidden and intermediate stay whole as GEMV input widths
        local = dataclasses.replace(full_cfg, q_heads=full_cfg.q_heads // world, kv_heads=full_cfg.kv_heads // world)
        shard.cfg = local
        if shard.head is None:
            shard.head = shard.embed[slice(*row_shard(full_cfg.vocab, rank, world))]
        super().__init__(shard, cap=cap, step_kernel=False, device=device)
        c = full_cfg
        self.widths = {"att": c.q_heads * c.head_dim, "yo": c.hidden, "m": c.inter, "yd": c.hidden}
        self.heap = heap if heap is not None else PeerHeap(self.heap_bytes(c), rank, world)
        self._layout()
        if heap is None:
            self.heap.connect_processes(group)
        self._tp: dict[int, dict[str, Any]] = {}
        # passes made so far at each width, on the card: the layers' exchanges and the picks count their own
        self.passes = torch.zeros(len(CARD_ROWS), 2, dtype=torch.int32, device=self.dev)

    # -- the heap: the same layout on every rank -------------------------------------------------------------------------
    @classmethod
    def heap_bytes(cls, c: DenseConfig) -> int:
        per_row = 2 * (c.q_heads * c.head_dim + 2 * c.hidden + c.inter)
        flags = (4 * c.layers + 1) * FLAG_BYTES
        return sum(M * per_row + 4 * 256 + flags + 8 * 32 * 8 + 512 for M in CARD_ROWS) + 4096

    def _layout(self) -> None:
        self.off: dict[int, dict[str, int]] = {}
        for M in CARD_ROWS:
            o = {k: self.heap.carve(M * w * 2) for k, w in self.widths.items()}
            o["flags"] = self.heap.carve((4 * self.full.layers + 1) * FLAG_BYTES)
            o["picks"] = self.heap.carve(8 * 32 * 8)
            self.off[M] = o

    def flag_off(self, M: int, layer: int, which: str) -> int:
        return self.off[M]["flags"] + (4 * layer + self.XCHG.index(which)) * FLAG_BYTES

    def tp_bufs(self, M: int) -> dict[str, Any]:
        """width M's local buffers and its exchange descriptors"""
        if M not in self._tp:
            c, w, dev, hp = self.full, self.world, self.dev, self.heap
            bf = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)  # noqa: E731
            wi = CARD_ROWS.index(M)
            t: dict[str, Any] = {
                "att_l": bf(M, c.q_heads * c.head_dim // w), "gu_l": bf(M, 2 * c.inter // w), "m_l": bf(M, c.inter // w),
                "lg_l": bf(M, c.vocab // w), "tok_l": torch.zeros(M, dtype=torch.int64, device=dev),
                "pass": int(self.passes[wi, 0:1].data_ptr()), "pick_pass": int(self.passes[wi, 1:2].data_ptr()),
            }  # fmt: skip
            for k, width in self.widths.items():
                t[k] = hp.local + self.off[M][k]  # this rank's copy of the full vector
                t[k + "_t"] = hp.tensor(self.off[M][k], (M, width), torch.bfloat16)
                t["send_" + k] = [hp.send_desc(self.off[M][k], self.flag_off(M, i, k), width, self.rank * (width // w))
                                  for i in range(c.layers)]  # fmt: skip
            pick_flag = self.off[M]["flags"] + 4 * c.layers * FLAG_BYTES
            t["send_pick"] = hp.send_desc(self.off[M]["picks"], pick_flag, 8 * 32, 0)
            t["wait_pick"] = hp.wait_desc(pick_flag, t["pick_pass"], w)
            self._tp[M] = t
        return self._tp[M]

    def _wait(self, M: int, layer: int, which: str, ctas: int) -> Any:
        return self.heap.wait_desc(self.flag_off(M, layer, which), self.tp_bufs(M)["pass"], ctas * self.world)

    # -- the pass, one exchange-delimited piece at a time ---------------------------------------------------------------
    def ops(self, T: int, tail: bool = True, stream_ptr: int | None = None):
        """the pass's launches; yields after each piece that ends in an exchange, so that engines standing in for the
        ranks on ONE GPU can take turns (every producer launched before any consumer of its vector)"""
        c, lc, w = self.full, self.cfg, self.world
        M = pad_rows(T)
        g, t = self.bufs(M), self.tp_bufs(M)
        s = capi.stream_ptr() if stream_ptr is None else stream_ptr
        H, D, I = c.hidden, c.head_dim, c.inter
        A = c.q_heads * D
        K_ = self._k
        n = C.c_int(0)
        fuse = self.fuse_norm and M <= 8 and M * H * 2 <= 64 * 1024
        hcur, halt = g["h"], g["h2"]
        y_prev, wait_prev = 0, None  # the previous layer's output (every rank's slices, in this rank's copy)

        def normed(W: torch.Tensor, norm_w: torch.Tensor, R: int, out: Any, swiglu: bool, send: Any) -> int:
            """x = rmsnorm(h + y_prev) folded into the GEMV over W where the row fits, else the separate kernels"""
            nonlocal hcur, halt
            if fuse:
                K_("btb_b200_gemv_norm_x", ptr(W), ptr(hcur), y_prev, ptr(norm_w), c.eps, 0, ptr(halt) if y_prev else 0,
                   ptr(out) if send is None else 0, T, M, R, H, int(swiglu), wait_prev, send, C.byref(n), s)  # fmt: skip
                if y_prev:
                    hcur, halt = halt, hcur
                return n.value
            if wait_prev is not None:
                K_("btb_b200_xchg_wait", wait_prev, s)
            K_("btb_b200_add_rmsnorm", ptr(hcur), y_prev, ptr(norm_w), c.eps, ptr(g["x"]), T, H, 0, s)
            if not swiglu:
                K_("btb_b200_gemv_bf16_x", ptr(W), ptr(g["x"]), ptr(out) if send is None else 0, M, R, H, None, send,
                   C.byref(n), s)  # fmt: skip
                return n.value
            K_("btb_b200_gemv_bf16", ptr(W), ptr(g["x"]), ptr(t["gu_l"]), M, R, H, s)
            K_("btb_b200_silu_mul", ptr(t["gu_l"]), ptr(t["m_l"]), M, I // w, s)
            K_("btb_b200_xchg_send", ptr(t["m_l"]), M, I // w, 2, None, send, C.byref(n), s)
            return n.value

        for i, L in enumerate(self.w.layers):
            normed(L.qkv, L.ln1, lc.qkv_rows, g["qkv"], False, None)
            self._attention(g, i, L.wq, L.wk, T, s, out=t["att_l"])  # this rank's heads
            K_("btb_b200_xchg_send", ptr(t["att_l"]), M, A // w, 2, None, t["send_att"][i], C.byref(n), s)
            wait_prev = self._wait(M, i, "att", n.value)
            yield
            K_("btb_b200_gemv_bf16_x", ptr(L.o), t["att"], 0, M, H // w, A, wait_prev, t["send_yo"][i], C.byref(n), s)
            y_prev, wait_prev = t["yo"], self._wait(M, i, "yo", n.value)
            yield
            ctas = normed(L.gu, L.ln2, 2 * I // w, None, True, t["send_m"][i])
            wait_prev = self._wait(M, i, "m", ctas)
            yield
            K_("btb_b200_gemv_bf16_x", ptr(L.down), t["m"], 0, M, H // w, I, wait_prev, t["send_yd"][i], C.byref(n), s)
            y_prev, wait_prev = t["yd"], self._wait(M, i, "yd", n.value)
            yield
        if tail:
            normed(self.w.head, self.w.norm, c.vocab // w, t["lg_l"], False, None)
        elif wait_prev is not None:  # the last layer's output must have landed before the pass count moves on
            K_("btb_b200_xchg_wait", wait_prev, s)
        if hcur is not g["h"]:
            g["h"].copy_(hcur)

    def body(self, T: int, tail: bool = True, stream_ptr: int | None = None) -> None:
        for _ in self.ops(T, tail, stream_ptr):
            pass

    def tick(self, M: int, s: int) -> None:
        """a pass that ends without a pick advances the layers' pass count by a launch of its own"""
        self._k("btb_b200_xchg_tick", self.tp_bufs(M)["pass"], s)

    def _pick(self, g: dict, T: int, s: int, out: torch.Tensor, phase: int = 0, body_pass: bool = True) -> None:
        """the step's pick: this rank's lowest-index argmax of its vocabulary rows, then the merge over the ranks (which
        also closes the pass: the layers' pass count advances there)"""
        M = pad_rows(T)
        t = self.tp_bufs(M)
        lg = g.get("logits_l", t["lg_l"])
        Vl = self.full.vocab // self.world
        if phase != 2:
            self._k("btb_b200_argmax_bf16", ptr(lg), T, Vl, ptr(self.bufs(M)["pick"]), ptr(t["tok_l"]), s)
        self._k("btb_b200_xchg_pick", ptr(lg), T, Vl, self.rank * Vl, ptr(t["tok_l"]), self.rank, t["wait_pick"],
                t["send_pick"], ptr(out), t["pass"] if body_pass else 0, phase, s)  # fmt: skip

    def forward(self, ids: torch.Tensor, depth: Any = None, parents: Any = None, advance: bool = True) -> torch.Tensor:
        """a pass; returns THIS RANK'S logits slice [T, V / world]"""
        super().forward(ids, depth, parents, advance)
        M = pad_rows(int(ids.numel()))
        self.tick(M, capi.stream_ptr())
        return self.tp_bufs(M)["lg_l"][: int(ids.numel())]

    def generate_greedy(self, prompt: Any, max_new: int, graph_steps: int = 1) -> list[int]:
        """prefill, the first token from the prompt's last row, then the captured step graph replayed"""
        prompt = torch.as_tensor(prompt, dtype=torch.int64)
        self.reset()
        last = self.prefill(prompt)
        g = self.bufs(1)
        s = capi.stream_ptr()
        self._pick({"logits_l": last.contiguous()}, 1, s, g["ids"], body_pass=False)
        toks = [int(g["ids"][0].item())]
        graph = self.step_graph(1, publish=True)
        while len(toks) < max_new:
            graph.replay()
            torch.cuda.current_stream().synchronize()
            toks.append(int(self.pin_tok[0]))
        return toks
