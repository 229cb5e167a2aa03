"""One 8-GPU box, one process a GPU: how the decode path is cut across ranks, and the dense tensor-parallel engine.

btb has no multi-GPU path, so the contract here is bit-identity with the one-GPU arithmetic:

* dense layers (tensor parallel): every linear is cut by OUTPUT rows - q/k/v by kv-head group, o and down by rows of
  the hidden size, gate and up by the same rows of the intermediate size (paired), the head by vocabulary rows - so
  each output element's whole K-sum stays on one GPU in the one-GPU order. Attention is cut by kv head; a rank holds
  only its heads' cache. What a rank lacks of an activation vector its peers write into its memory: the producing
  kernel's epilogue stores every finished element, marked with the hop's sequence number, into every rank's copy, and
  the consuming kernel's prologue takes each word of its local copy once it carries the mark (csrc/tp.cuh) - four such
  hops a layer, no collective call, no fence or flag, no reduction (hence no change of summation order), and the whole
  step stays one captured CUDA graph.
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
from .exchange import PeerHeap


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
        self.x_stage_max = 96 * 1024  # an exchanged x is decoded on its way into shared memory up to this size

    # -- the heap: the same layout on every rank -------------------------------------------------------------------------
    PICK_TABLE = 8 * 32 * 2 * 8

    @classmethod
    def heap_bytes(cls, c: DenseConfig) -> int:
        per_row = 4 * (c.q_heads * c.head_dim + 2 * c.hidden + c.inter)  # a word an element
        return sum(M * per_row + 5 * 256 + cls.PICK_TABLE for M in CARD_ROWS) + 4096

    def _layout(self) -> None:
        self.off: dict[int, dict[str, int]] = {}
        for M in CARD_ROWS:
            o = {k: self.heap.carve(M * w * 4) for k, w in self.widths.items()}
            o["picks"] = self.heap.carve(self.PICK_TABLE)
            self.off[M] = o

    def tp_bufs(self, M: int) -> dict[str, Any]:
        """width M's local buffers and its exchange descriptors: hop 4 i + j + 1 of a pass carries layer i's vector j"""
        if M not in self._tp:
            c, w, dev, hp = self.full, self.world, self.dev, self.heap
            bf = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)  # noqa: E731
            wi = CARD_ROWS.index(M)
            t: dict[str, Any] = {
                "att_l": bf(M, c.q_heads * c.head_dim // w), "gu_l": bf(M, 2 * c.inter // w), "m_l": bf(M, c.inter // w),
                "lg_l": bf(M, c.vocab // w), "tok_l": torch.zeros(M, dtype=torch.int64, device=dev),
                "plain": bf(M, max(self.widths.values())),  # an exchanged vector decoded for a kernel that reads plain bf16
                "pass": int(self.passes[wi, 0:1].data_ptr()), "pick_pass": int(self.passes[wi, 1:2].data_ptr()),
            }  # fmt: skip
            per_pass = 4 * c.layers
            for j, (k, width) in enumerate(self.widths.items()):
                t[k] = hp.local + self.off[M][k]  # this rank's copy of the full vector (words)
                t[k + "_t"] = hp.tensor(self.off[M][k], (M, width), torch.int32)
                t["send_" + k] = [hp.send_desc(self.off[M][k], width, self.rank * (width // w), t["pass"], per_pass, 4 * i + j + 1)
                                  for i in range(c.layers)]  # fmt: skip
                t["recv_" + k] = [capi.Recv(t["pass"], per_pass, 4 * i + j + 1) for i in range(c.layers)]
            t["tables"] = (C.c_void_p * w)(*[hp.base[r] + self.off[M]["picks"] for r in range(w)])
            self._tp[M] = t
        return self._tp[M]

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
        fuse = self.fuse_norm and M <= 8 and M * H * 2 <= 64 * 1024
        hcur, halt = g["h"], g["h2"]
        y_prev, recv_prev = 0, None  # the previous block's output: every rank's slices, in this rank's copy

        def normed(W: torch.Tensor, norm_w: torch.Tensor, R: int, out: Any, swiglu: bool, send: Any) -> None:
            """x = rmsnorm(h + y_prev) folded into the GEMV over W where the row fits, else the separate kernels"""
            nonlocal hcur, halt
            if fuse:
                K_("btb_b200_gemv_norm_x", ptr(W), ptr(hcur), y_prev, ptr(norm_w), c.eps, 0, ptr(halt) if y_prev else 0,
                   ptr(out) if send is None else 0, T, M, R, H, int(swiglu), recv_prev, send, s)  # fmt: skip
                if y_prev:
                    hcur, halt = halt, hcur
                return
            y_plain = 0
            if y_prev:
                K_("btb_b200_xchg_unpack", y_prev, ptr(t["plain"]), T, H, recv_prev, s)
                y_plain = ptr(t["plain"])
            K_("btb_b200_add_rmsnorm", ptr(hcur), y_plain, ptr(norm_w), c.eps, ptr(g["x"]), T, H, 0, s)
            if not swiglu:
                K_("btb_b200_gemv_bf16_x", ptr(W), ptr(g["x"]), ptr(out) if send is None else 0, T, M, R, H, None, send, s)
                return
            K_("btb_b200_gemv_bf16", ptr(W), ptr(g["x"]), ptr(t["gu_l"]), M, R, H, s)
            K_("btb_b200_silu_mul", ptr(t["gu_l"]), ptr(t["m_l"]), M, I // w, s)
            K_("btb_b200_xchg_send", ptr(t["m_l"]), M, I // w, send, s)

        def over_exchanged(W: torch.Tensor, which: str, i: int, R: int, C_: int, send: Any) -> None:
            """a GEMV whose x is an exchanged vector: decoded inside the GEMV where x is staged, else beforehand"""
            if M <= 8 and M * C_ * 2 <= self.x_stage_max:
                K_("btb_b200_gemv_bf16_x", ptr(W), t[which], 0, T, M, R, C_, t["recv_" + which][i], send, s)
                return
            K_("btb_b200_xchg_unpack", t[which], ptr(t["plain"]), T, C_, t["recv_" + which][i], s)
            K_("btb_b200_gemv_bf16_x", ptr(W), ptr(t["plain"]), 0, T, M, R, C_, None, send, s)

        for i, L in enumerate(self.w.layers):
            normed(L.qkv, L.ln1, lc.qkv_rows, g["qkv"], False, None)
            self._attention_send(g, i, L.wq, L.wk, T, s, t["send_att"][i], (L.o, L.gu))  # this rank's heads, to every rank
            yield
            over_exchanged(L.o, "att", i, H // w, A, t["send_yo"][i])
            y_prev, recv_prev = t["yo"], t["recv_yo"][i]
            yield
            normed(L.gu, L.ln2, 2 * I // w, None, True, t["send_m"][i])
            yield
            over_exchanged(L.down, "m", i, H // w, I, t["send_yd"][i])
            y_prev, recv_prev = t["yd"], t["recv_yd"][i]
            yield
        if tail:
            normed(self.w.head, self.w.norm, c.vocab // w, t["lg_l"], False, None)
        elif y_prev:  # a pass without its head: the last block's output decoded into y, as the plain engine leaves it
            K_("btb_b200_xchg_unpack", y_prev, ptr(g["y"]), T, H, recv_prev, s)
        if hcur is not g["h"]:
            g["h"].copy_(hcur)

    def _attention_send(self, g: dict, i: int, wq: Any, wk: Any, T: int, s: int, send: Any, warm: tuple = ()) -> None:
        """`CardEngine._attention` over this rank's heads, its output rows stored into every rank's copy by the
        attention kernel itself"""
        c = self.cfg
        Hq, Hk, D = c.q_heads, c.kv_heads, c.head_dim
        if T == 1 and self.fuse_attn and D in (64, 128):
            (wa, na), (wb, nb) = self._warm(warm[0]) if warm else (0, 0), self._warm(warm[1]) if len(warm) > 1 else (0, 0)
            self._k("btb_b200_attn_step_w", ptr(g["qkv"]), ptr(wq), ptr(wk), c.eps, ptr(self.cos), ptr(self.sin),
                    ptr(self.n0), ptr(g["depth"]), ptr(self.K[i]), ptr(self.V[i]), ptr(g["q"]), 0, Hq, Hk, D, self.hs,
                    self.rs, 0, float(D**-0.5), ptr(g["part_m"]), ptr(g["part_l"]), ptr(g["part_acc"]), ptr(g["cnt"]), 0, 0,
                    0, self.cap, send, wa, na, wb, nb, s)  # fmt: skip
            return
        self._k("btb_b200_norm_rope_kv", ptr(g["qkv"]), ptr(wq), ptr(wk), c.eps, ptr(self.cos), ptr(self.sin),
                ptr(self.n0), ptr(g["depth"]), ptr(self.K[i]), ptr(self.V[i]), ptr(g["q"]), T, Hq, Hk, D, self.hs,
                self.rs, 0, 0, self.cap, s)  # fmt: skip
        self._k("btb_b200_attn_decode_x", ptr(g["q"]), ptr(self.K[i]), ptr(self.V[i]), ptr(self.n0), ptr(g["par"]), T, Hq,
                Hk, D, self.hs, self.rs, float(D**-0.5), ptr(g["part_m"]), ptr(g["part_l"]), ptr(g["part_acc"]),
                ptr(g["cnt"]), 0, 0, 0, self.cap, send, s)  # fmt: skip

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
        self._k("btb_b200_xchg_pick", ptr(lg), T, Vl, self.rank * Vl, ptr(t["tok_l"]), self.rank, self.world, t["tables"],
                ptr(out), t["pick_pass"], t["pass"] if body_pass else 0, phase, s)  # fmt: skip

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
