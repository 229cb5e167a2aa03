"""The MoE decoder on the card: attention as the dense engine's, the MLP a router and the picked experts' matvecs.

What this mirrors: btb serves MoE layers through `_Router` / `Qwen4Router` (btb/engine/host.py:175-191,
btb/engine/families/qwen4/router.py:24-50) and `_Experts._one_row` (host.py:508-569): the normed row widened to f32,
the router's logits by the host GEMV, top-k, each picked expert's gate_up and down by the grouped host GEMV over the
weights as stored (MXFP4 / FP8), the row dtype's gated activation between them, and the weighted sum in ascending
expert id. btb runs those matvecs on the CPU with two bus hops a layer; here they run on the card, the picks never
leaving it, with the same arithmetic (the 16-lane order of native/src/gemv.rs).

Expert parallelism (one process a GPU): expert e lives on rank e % ep; a rank multiplies only its own picks, and its
down matvecs' epilogue stores each product - rounded to bf16, which is the first thing the ordered sum does to it -
as a marked word into every rank's copy of the layer's [T, k, H] products (`btb_b200.exchange`, csrc/tp.cuh: plain peer
stores, no collective call); every rank then runs the same ordered bf16 sum over its own copy, taking each word as it
arrives - bit-identical to one GPU, and the whole step stays one captured graph. Attention, router and head are
computed by every rank.
"""

from __future__ import annotations

import os

from dataclasses import dataclass, field
from typing import Any

import torch

from . import capi
from .capi import ptr
from .engine import CARD_ROWS, CardEngine, DenseConfig, FP8Matrix, pad_rows
from .exchange import PeerHeap

FMT = {"bf16": 0, "mx4": 1, "fp8": 2}


@dataclass
class MoEConfig(DenseConfig):
    experts: int = 8
    top_k: int = 2
    router_mode: int = 0  # 0: softmax -> top-k -> renormalise (Qwen); 1: top-k -> softmax (gpt-oss)
    glu_kind: int = 0  # 0: silu(gate) * up over halves; 1: gpt-oss clamped GLU over interleaved lanes
    expert_fmt: str = "mx4"
    alpha: float = 1.702
    limit: float = 7.0
    dense_fmt: str = "bf16"  # the attention linears: bf16, or FP8 e4m3 with 128 x 128 block scales ("fp8")

    def expert_bytes(self) -> int:
        """one expert's stored bytes (gate_up + down)"""
        n = 3 * self.inter * self.hidden
        if self.expert_fmt == "mx4":
            return n // 2 + n // 32
        if self.expert_fmt == "fp8":
            return n + 4 * (n // (128 * 128))
        return 2 * n

    def weight_bytes_per_token(self, storage: str = "bf16") -> int:
        att = (2 if self.dense_fmt == "bf16" else 1) * self.hidden * (self.qkv_rows + self.q_heads * self.head_dim)
        att += 2 * self.experts * self.hidden
        return self.layers * (att + self.top_k * self.expert_bytes()) + self.vocab * self.hidden * 2


GPT_OSS_20B = MoEConfig("gpt-oss-20b", 2880, 24, 64, 8, 64, 2880, 201088, theta=150000.0, eps=1e-5, qk_norm=False,
                        experts=32, top_k=4, router_mode=1, glu_kind=1, expert_fmt="mx4")  # fmt: skip
QWEN3_30B_A3B = MoEConfig("qwen3-30b-a3b", 2048, 48, 32, 4, 128, 768, 151936, experts=128, top_k=8, router_mode=0,
                          glu_kind=0, expert_fmt="fp8", dense_fmt="fp8")  # fmt: skip


@dataclass
class ExpertStack:
    """a layer's experts as stored, the locally held ones stacked: w [n_local, R, ...] bytes, scales beside them"""

    fmt: str
    w: torch.Tensor
    scales: torch.Tensor | None
    R: int
    C: int
    sr: int = 1
    sc: int = 1

    @property
    def w_stride(self) -> int:
        return int(self.w[0].numel() * self.w.element_size())

    @property
    def s_stride(self) -> int:
        return 0 if self.scales is None else int(self.scales[0].numel() * self.scales.element_size())


@dataclass
class MoELayer:
    ln1: torch.Tensor
    ln2: torch.Tensor
    qkv: Any  # bf16 [rows, H] or FP8Matrix
    o: Any
    router: torch.Tensor  # [E, H] bf16
    gu: ExpertStack
    dn: ExpertStack
    wq: torch.Tensor | None = None
    wk: torch.Tensor | None = None


@dataclass
class MoEWeights:
    cfg: MoEConfig
    embed: torch.Tensor
    norm: torch.Tensor
    layers: list[MoELayer] = field(default_factory=list)
    ep_rank: int = 0
    ep_size: int = 1


def synth_expert_stack(cfg: MoEConfig, g: torch.Generator, n: int, R: int, C_: int, device: Any) -> ExpertStack:
    """seeded stored experts: MXFP4 nibbles uniform over the 16 codes with scales uniform in exponent [-8, 0]; FP8 bytes
    uniform over the finite codes with bf16 N(0, 0.02) scales per 128 x 128 block; bf16 N(0, 0.02)"""
    gdev = g.device
    if cfg.expert_fmt == "mx4":
        blocks = torch.randint(0, 256, (n, R, C_ // 32, 16), generator=g, device=gdev, dtype=torch.uint8)
        scales = torch.randint(119, 128, (n, R, C_ // 32), generator=g, device=gdev, dtype=torch.uint8)
        return ExpertStack("mx4", blocks.to(device), scales.to(device), R, C_)
    if cfg.expert_fmt == "fp8":
        w = torch.randint(0, 256, (n, R, C_), generator=g, device=gdev, dtype=torch.uint8)
        w = torch.where((w & 0x7F) == 0x7F, w & 0xF0, w)  # no NaN codes
        sr, sc = R // 128, C_ // 128
        s = (torch.randn(n, sr, sc, generator=g, device=gdev) * 0.02).to(torch.bfloat16).float()
        return ExpertStack("fp8", w.to(device), s.to(device).contiguous(), R, C_, sr, sc)
    w = (torch.randn(n, R, C_, generator=g, device=gdev) * 0.02).to(torch.bfloat16)
    return ExpertStack("bf16", w.to(device), None, R, C_)


def synth_moe_weights(cfg: MoEConfig, seed: int = 0, device: Any = "cuda", on_cpu: bool = False, ep_rank: int = 0,
                      ep_size: int = 1, layer_std: float = 0.02) -> MoEWeights:  # fmt: skip
    """random-init weights: attention, router, embedding bf16 N(0, 0.02); norm weights 1; experts as
    `synth_expert_stack`. Under expert parallelism every rank draws the same stream and keeps expert e iff
    e % ep_size == ep_rank, so the model is the same model at every N. `layer_std`: the deviation of the
    layers' bf16 linears (attention, router), as in `engine.synth_weights`."""
    gdev = "cpu" if on_cpu else device
    g = torch.Generator(device=gdev).manual_seed(seed)
    std = [0.02]

    def lin(r: int, c: int) -> torch.Tensor:
        return (torch.randn(r, c, generator=g, device=gdev, dtype=torch.float32) * std[0]).to(torch.bfloat16).to(device)

    def ones(n: int) -> torch.Tensor:
        return torch.ones(n, dtype=torch.bfloat16, device=device)

    def keep(st: ExpertStack) -> ExpertStack:
        if ep_size == 1:
            return st
        sel = torch.arange(ep_rank, cfg.experts, ep_size, device=st.w.device)
        st.w = st.w.index_select(0, sel).contiguous()
        if st.scales is not None:
            st.scales = st.scales.index_select(0, sel).contiguous()
        return st

    def dense(r: int, c: int) -> Any:
        if cfg.dense_fmt == "bf16":
            return lin(r, c)
        w = torch.randint(0, 256, (r, c), generator=g, device=gdev, dtype=torch.uint8)
        w = torch.where((w & 0x7F) == 0x7F, w & 0xF0, w)
        sc = (torch.randn(r // 128, c // 128, generator=g, device=gdev) * 0.02).to(torch.bfloat16).float()
        return FP8Matrix(w.to(device), sc.to(device))

    H, D, I, E = cfg.hidden, cfg.head_dim, cfg.inter, cfg.experts
    mw = MoEWeights(cfg, lin(cfg.vocab, H), ones(H), ep_rank=ep_rank, ep_size=ep_size)
    std[0] = layer_std
    for _ in range(cfg.layers):
        if cfg.dense_fmt == "bf16":
            qkv = torch.cat([lin(cfg.q_heads * D, H), lin(cfg.kv_heads * D, H), lin(cfg.kv_heads * D, H)])
        else:
            qkv = dense(cfg.qkv_rows, H)
        o = dense(H, cfg.q_heads * D)
        router = lin(E, H)
        gu = keep(synth_expert_stack(cfg, g, E, 2 * I, H, device))
        dn = keep(synth_expert_stack(cfg, g, E, H, I, device))
        mw.layers.append(MoELayer(ones(H), ones(H), qkv, o, router, gu, dn,
                                  ones(D) if cfg.qk_norm else None, ones(D) if cfg.qk_norm else None))  # fmt: skip
    return mw


class MoEEngine(CardEngine):
    """the MoE model on one card (or one rank of an expert-parallel group)"""

    def __init__(self, weights: MoEWeights, cap: int = 4096, device: Any = "cuda", group: Any = None,
                 heap: PeerHeap | None = None):
        super().__init__(weights, cap=cap, step_kernel=False, device=device)  # type: ignore[arg-type]
        self.group = group
        self.ep_rank, self.ep_size = weights.ep_rank, weights.ep_size
        self.heap: PeerHeap | None = None
        if self.ep_size > 1:
            # every rank's copy of a layer's products: words [M * k, H], three buffers taken in turn so that a rank
            # writing layer i + 1's never meets a slower rank still reading layer i's (see `_edn_buffer`)
            c = self.cfg
            self.heap = heap if heap is not None else PeerHeap(self.heap_bytes(c), self.ep_rank, self.ep_size)
            self.edn_off = {M: [self.heap.carve(M * c.top_k * c.hidden * 4) for _ in range(3)] for M in CARD_ROWS}
            if heap is None:
                self.heap.connect_processes(group)
            self.passes = torch.zeros(len(CARD_ROWS), dtype=torch.int32, device=self.dev)
            self._ep: dict[int, Any] = {}
        self.fuse_router = True  # the router's matvec and the picks in one cluster launch
        self.router_fuse_max = int(os.environ.get("BTB_B200_ROUTER_FUSE_MAX", "131072"))  # ... up to this many weights
        # the activation inside the down matvecs' launch, the picks' sum inside the next norm's: fewer launches, the
        # same bits, but measured slower than the separate kernels (one block a token sums the picks; every CTA of the
        # down matvecs repeats the activation) - off unless asked for
        self.fold = os.environ.get("BTB_B200_MOE_FOLD", "0") != "0"
        self.glu_epilogue = os.environ.get("BTB_B200_MOE_GLU", "1") != "0"  # the gated activation in the gate/up launch

    @staticmethod
    def heap_bytes(c: MoEConfig) -> int:
        return sum(3 * (M * c.top_k * c.hidden * 4 + 256) for M in CARD_ROWS) + 4096

    def _edn_buffer(self, i: int) -> int:
        """which of the three buffers layer i's products take: consecutive layers differ, and so do a pass's last layer
        and the next pass's first, so a buffer is rewritten only after every rank has read it (a rank sends layer i + 2's
        products only after its own sum over layer i + 1's, which needed every rank's, each sent after that rank's sum
        over layer i's)"""
        L = self.cfg.layers
        return 2 if (i == L - 1 and L % 2 == 1) else i % 2

    def ep_descs(self, M: int) -> Any:
        """width M's exchange descriptors: hop i + 1 of a pass carries layer i's products"""
        if M not in self._ep:
            c, hp = self.cfg, self.heap
            pas = int(self.passes[CARD_ROWS.index(M) : CARD_ROWS.index(M) + 1].data_ptr())
            sends = [hp.send_desc(self.edn_off[M][self._edn_buffer(i)], c.hidden, 0, pas, c.layers, i + 1) for i in range(c.layers)]
            recvs = [capi.Recv(pas, c.layers, i + 1) for i in range(c.layers)]
            local = [hp.local + self.edn_off[M][self._edn_buffer(i)] for i in range(c.layers)]
            self._ep[M] = (sends, recvs, local, pas)
        return self._ep[M]

    def bufs(self, M: int) -> dict[str, torch.Tensor]:
        g = super().bufs(M)
        if "xf" not in g:
            c, dev = self.cfg, self.dev
            f32 = lambda *s: torch.zeros(*s, dtype=torch.float32, device=dev)  # noqa: E731
            k = c.top_k
            g.update({
                "xf": f32(M, c.hidden), "rl": f32(M, c.experts), "idx": torch.zeros(M, k, dtype=torch.int32, device=dev),
                "rw": torch.zeros(M, k, dtype=torch.bfloat16, device=dev), "egu": f32(M * k, 2 * c.inter),
                "eh": f32(M * k, c.inter), "edn": f32(M * k, c.hidden),
                "rcnt": torch.zeros(M, dtype=torch.int32, device=dev),
            })  # fmt: skip
        return g

    def _expert_gemv(self, st: ExpertStack, idx: torch.Tensor, n_tasks: int, x: torch.Tensor, x_div: int,
                     y: torch.Tensor, s: int) -> None:  # fmt: skip
        self._k("btb_b200_moe_gemv", FMT[st.fmt], ptr(st.w), ptr(st.scales), st.w_stride, st.s_stride, st.sr, st.sc,
                ptr(idx), n_tasks, self.cfg.experts, ptr(x), x_div, ptr(y), st.R, st.C, self.ep_rank, self.ep_size, s)

    def body(self, T: int, tail: bool = True, stream_ptr: int | None = None) -> None:
        for _ in self.ops(T, tail, stream_ptr):
            pass

    def ops(self, T: int, tail: bool = True, stream_ptr: int | None = None):
        """the pass's launches; under expert parallelism it yields after each layer's products are sent, so that engines
        standing in for the ranks on ONE GPU can take turns (every rank's products sent before any rank sums them)"""
        c = self.cfg
        M = pad_rows(T)
        g = self.bufs(M)
        s = capi.stream_ptr() if stream_ptr is None else stream_ptr
        H, Hq, Hk, D, I, E, k = c.hidden, c.q_heads, c.kv_heads, c.head_dim, c.inter, c.experts, c.top_k
        K_ = self._k
        fold = self.fold and self.ep_size == 1
        pending = False  # the previous layer's picks are summed by the norm that reads them
        y_prev = None
        # the residual ping-pongs between two buffers where the norm is folded into the matvec that reads it (a CTA must
        # not read a row another CTA is updating); the pass ends on g["h"]
        hcur, halt = g["h"], g["h2"]
        fuse = self.fuse_norm and M <= 8 and M * H * 2 <= 64 * 1024

        def norm_in(norm_w: torch.Tensor) -> None:
            nonlocal pending
            if pending:
                K_("btb_b200_moe_combine_norm", ptr(g["edn"]), ptr(g["idx"]), ptr(g["rw"]), k, ptr(hcur), ptr(norm_w),
                   c.eps, ptr(g["x"]), 0, 0, T, H, 0, s)
                pending = False
            else:
                K_("btb_b200_add_rmsnorm", ptr(hcur), ptr(y_prev), ptr(norm_w), c.eps, ptr(g["x"]), T, H, 0, s)

        def normed_matvec(W: Any, norm_w: torch.Tensor, out: torch.Tensor, R: int) -> None:
            """x = norm(h + y_prev) and the matvec over it: one launch where the matrix is bf16 and the pass narrow"""
            nonlocal hcur, halt
            if fuse and not pending and isinstance(W, (torch.Tensor, FP8Matrix)):
                # (the first layer: no add, the residual stays where it is)
                ya, ho = (0, 0) if y_prev is None else (ptr(y_prev), ptr(halt))
                if isinstance(W, FP8Matrix):
                    K_("btb_b200_gemv_norm_fp8", ptr(W.w), ptr(W.scales), W.sr, W.sc, ptr(hcur), ya, ptr(norm_w), c.eps, 0,
                       ho, ptr(out), T, M, R, H, s)  # fmt: skip
                else:
                    K_("btb_b200_gemv_norm", ptr(W), 0, 0, 0, 0, 0, ptr(hcur), ya, ptr(norm_w), c.eps, 0, ho, ptr(out), T, M,
                       R, H, s)  # fmt: skip
                if y_prev is not None:
                    hcur, halt = halt, hcur
                return
            norm_in(norm_w)
            self._matvec(W, g["x"], out, M, R, H, s)

        for i, L in enumerate(self.w.layers):
            normed_matvec(L.qkv, L.ln1, g["qkv"], c.qkv_rows)
            self._attention(g, i, L.wq, L.wk, T, s)
            self._matvec(L.o, g["att"], g["y"], M, H, Hq * D, s)
            # the MoE block: x.float() (made by the norm's own launch), the router's logits by the host-order GEMV,
            # the picks, the experts, the sum
            # one cluster launch for the norm, the router's matvec and the picks where the router is small enough for it
            # to win (measured: 32 experts x 2880 yes, 128 x 2048 no)
            if self.fuse_router and H % 8 == 0 and E * H <= self.router_fuse_max:
                K_("btb_b200_moe_router_norm", ptr(L.router), ptr(hcur), ptr(g["y"]), ptr(L.ln2), c.eps, 0, ptr(halt), 0,
                   ptr(g["xf"]), 0, E, H, k, c.router_mode, ptr(g["idx"]), ptr(g["rw"]), T, s)  # fmt: skip
                hcur, halt = halt, hcur
            elif self.fuse_router and H % 8 == 0 and E <= 8192:
                # a larger router: the same three steps as one launch over the whole card, the last CTA to finish picking
                K_("btb_b200_moe_router_grid", ptr(L.router), ptr(hcur), ptr(g["y"]), ptr(L.ln2), c.eps, 0, ptr(halt), 0,
                   ptr(g["xf"]), ptr(g["rl"]), ptr(g["rcnt"]), E, H, k, c.router_mode, ptr(g["idx"]), ptr(g["rw"]), T, s)  # fmt: skip
                hcur, halt = halt, hcur
            else:
                K_("btb_b200_add_rmsnorm_wide", ptr(hcur), ptr(g["y"]), ptr(L.ln2), c.eps, ptr(g["x"]), ptr(g["xf"]), T, H,
                   0, s)  # fmt: skip
                K_("btb_b200_moe_gemv", 0, ptr(L.router), 0, 0, 0, 1, 1, 0, T, 1, ptr(g["xf"]), 1, ptr(g["rl"]), E, H, 0, 1, s)
                K_("btb_b200_moe_route", ptr(g["rl"]), E, E, k, c.router_mode, 1, ptr(g["idx"]), ptr(g["rw"]), T, s)
            # the gate/up matvecs, the gated activation in their epilogue where the layout lets a warp hold a pair's rows
            sg = L.gu
            glu = self.glu_epilogue and not fold and I % 4 == 0 and sg.C % 32 == 0 and getattr(L, "gu_bias", None) is None
            if glu:
                K_("btb_b200_moe_gemv_glu", FMT[sg.fmt], ptr(sg.w), ptr(sg.scales), sg.w_stride, sg.s_stride, sg.sr, sg.sc,
                   ptr(g["idx"]), T * k, E, ptr(g["xf"]), k, ptr(g["eh"]), sg.R, sg.C, c.glu_kind, c.alpha, c.limit,
                   self.ep_rank, self.ep_size, s)  # fmt: skip
            else:
                self._expert_gemv(L.gu, g["idx"], T * k, g["xf"], k, g["egu"], s)
            st = L.dn
            if fold and I % 32 == 0:
                # the gated activation is made inside the down matvecs' launch
                K_("btb_b200_moe_gemv_act", FMT[st.fmt], ptr(st.w), ptr(st.scales), st.w_stride, st.s_stride, st.sr, st.sc,
                   ptr(g["idx"]), T * k, E, ptr(g["egu"]), c.glu_kind, c.alpha, c.limit, ptr(g["edn"]), st.R, st.C,
                   self.ep_rank, self.ep_size, s)  # fmt: skip
            elif self.ep_size > 1:
                # this rank's picks: the products go, rounded and marked, into every rank's copy; the sum takes them there
                sends, recvs, local, _ = self.ep_descs(M)
                if not glu:
                    K_("btb_b200_moe_act", ptr(g["egu"]), ptr(g["eh"]), 0, 0, T * k, I, c.glu_kind, c.alpha, c.limit, s)
                K_("btb_b200_moe_gemv_x", FMT[st.fmt], ptr(st.w), ptr(st.scales), st.w_stride, st.s_stride, st.sr, st.sc,
                   ptr(g["idx"]), T * k, E, ptr(g["eh"]), 1, st.R, st.C, self.ep_rank, self.ep_size, sends[i], s)  # fmt: skip
                yield  # (engines standing in for the ranks on one GPU take turns here)
                K_("btb_b200_moe_combine_x", local[i], ptr(g["idx"]), ptr(g["rw"]), 0, ptr(g["y"]), T, k, H, recvs[i], s)
                y_prev = g["y"]
                continue
            else:
                if not glu:
                    K_("btb_b200_moe_act", ptr(g["egu"]), ptr(g["eh"]), 0, 0, T * k, I, c.glu_kind, c.alpha, c.limit, s)
                self._expert_gemv(L.dn, g["idx"], T * k, g["eh"], 1, g["edn"], s)
            if fold:
                pending = True
            else:
                K_("btb_b200_moe_combine", ptr(g["edn"]), ptr(g["idx"]), ptr(g["rw"]), 0, ptr(g["y"]), T, k, H, s)
            y_prev = g["y"]
        if tail:
            normed_matvec(self.w.embed, self.w.norm, g["logits"], c.vocab)
        elif pending:  # a pass without its head leaves the last layer's sum in y, as the unfolded pass does
            K_("btb_b200_moe_combine", ptr(g["edn"]), ptr(g["idx"]), ptr(g["rw"]), 0, ptr(g["y"]), T, k, H, s)
        if hcur is not g["h"]:  # an odd number of folded adds: bring the residual home
            g["h"].copy_(hcur)
        if self.ep_size > 1:  # the pass is over: its hops' sequence numbers move on
            K_("btb_b200_xchg_tick", self.ep_descs(M)[3], s)

    def weight_bytes(self) -> int:
        return self.cfg.weight_bytes_per_token()
