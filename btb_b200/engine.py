"""The card decode engine: the per-layer kernel sequence of btb's card graph, on the B200 library.

What this mirrors (all under btb/engine/cuda.py of btb): the load-time layout ``_card_weights``/``_card_merged``
(q, k, v merged into one row block, gate and up merged, cuda.py:1044-1164), the rope tables ``_card_tables``
(cuda.py:1166-1182), the static pass buffers ``_card_buffers`` (cuda.py:1491-1562), the pass body ``_card_body``
(cuda.py:1601-1837), the self-advancing step graph ``_card_step_graph`` (cuda.py:2101-2251) and the greedy loop
``_card_generate_greedy`` (cuda.py:2253-2459). Prefill runs chain passes of up to 32 rows through the same kernels,
so a prompt's cache rows are the rows the steps would have written.

PyTorch is plumbing here: device memory, streams, graph capture. Every kernel is the library's; a missing library
raises at construction.
"""

from __future__ import annotations

import os

from dataclasses import dataclass, field
from typing import Any

import torch

from . import capi
from .capi import call, ptr

CARD_ROWS = (1, 2, 4, 8, 16, 32)  # a pass's padded widths (btb/kinds.py CARD_ROWS)
GROUP_KEYS = 512  # keys a split of the attention takes


@dataclass
class DenseConfig:
    name: str
    hidden: int
    layers: int
    q_heads: int
    kv_heads: int
    head_dim: int
    inter: int
    vocab: int
    theta: float = 1e6
    eps: float = 1e-6
    qk_norm: bool = True

    @property
    def qkv_rows(self) -> int:
        return (self.q_heads + 2 * self.kv_heads) * self.head_dim

    def weight_bytes_per_token(self, storage: str = "bf16") -> int:
        """algorithmic weight bytes one decoded token reads: every layer's four matrices and the head"""
        per = self.hidden * (self.qkv_rows + self.q_heads * self.head_dim + 3 * self.inter)
        head = self.vocab * self.hidden * 2
        if storage == "bf16":
            return self.layers * per * 2 + head
        if storage == "p12":
            return self.layers * per * 3 // 2 + head  # the head stays bf16 (btb/engine/pack.py:82,105)
        raise ValueError(storage)

    def kv_bytes_per_row(self) -> int:
        return self.layers * 2 * self.kv_heads * self.head_dim * 2


QWEN3_4B = DenseConfig("qwen3-4b", 2560, 36, 32, 8, 128, 9728, 151936)
LLAMA31_70B = DenseConfig("llama-3.1-70b", 8192, 80, 64, 8, 128, 28672, 128256, theta=5e5, eps=1e-5, qk_norm=False)


def rope_tables(cfg: DenseConfig, cap: int, device: Any) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin [cap, D] bf16 from the default rotary: f32 inv_freq, f32 angles, halves concatenated, rounded once"""
    D = cfg.head_dim
    inv = 1.0 / (torch.tensor(cfg.theta, dtype=torch.float32) ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = torch.arange(cap, dtype=torch.float32)[:, None] * inv[None, :]
    emb = torch.cat([ang, ang], dim=-1)
    return emb.cos().to(torch.bfloat16).to(device), emb.sin().to(torch.bfloat16).to(device)


class P12Matrix:
    """one pack12 matrix on the card, as stored (btb/pack12.py:48-68) plus the per-row escape cursor"""

    def __init__(self, parts: tuple, rows: int, cols: int, device: Any):
        lo, hi4, table, esc_idx, esc_val = parts
        self.rows, self.cols = rows, cols
        as_t = lambda a, dt: torch.as_tensor(a, dtype=dt).to(device).contiguous()  # noqa: E731
        self.lo, self.hi4 = as_t(lo, torch.uint8), as_t(hi4, torch.uint8)
        # 16 bytes, host: it travels in the launch's arguments
        self.table = bytes(table) if isinstance(table, (bytes, bytearray)) else bytes(bytearray(int(v) for v in table))
        self.n_esc = int(len(esc_idx))
        self.esc_idx = as_t(esc_idx, torch.int32) if self.n_esc else None
        self.esc_val = as_t(esc_val, torch.uint8) if self.n_esc else None
        self.esc_row = None
        if self.n_esc:
            self.esc_row = torch.empty(rows + 1, dtype=torch.int32, device=device)
            call("btb_b200_p12_rows", ptr(self.esc_idx), self.n_esc, rows, cols, ptr(self.esc_row), capi.stream_ptr())

    @property
    def nbytes(self) -> int:
        return self.lo.numel() + self.hi4.numel() + 5 * self.n_esc


class FP8Matrix:
    """one FP8 matrix on the card as stored (btb/fp8.py:65-94 `F8Weight`): e4m3 bytes [R, C] and an f32 [sr, sc] grid"""

    def __init__(self, w: torch.Tensor, scales: torch.Tensor):
        self.w = w.contiguous().view(torch.uint8)
        self.scales = scales.float().contiguous()
        self.rows, self.cols = int(w.shape[0]), int(w.shape[1])
        self.sr, self.sc = int(scales.shape[0]), int(scales.shape[1])

    @property
    def nbytes(self) -> int:
        return self.w.numel() + 4 * self.scales.numel()


@dataclass
class LayerWeights:
    ln1: torch.Tensor
    ln2: torch.Tensor
    qkv: Any  # torch bf16 [rows, H] or P12Matrix
    o: Any
    gu: Any
    down: Any
    wq: torch.Tensor | None = None
    wk: torch.Tensor | None = None


@dataclass
class ModelWeights:
    cfg: DenseConfig
    embed: torch.Tensor  # [V, H] bf16, the tied head
    norm: torch.Tensor
    layers: list[LayerWeights] = field(default_factory=list)
    head: torch.Tensor | None = None  # a rank's vocabulary rows of `embed` (a view) when the model is cut over ranks


def synth_weights(cfg: DenseConfig, seed: int = 0, device: Any = "cuda", storage: str = "bf16",
                  on_cpu: bool = False, layer_std: float = 0.02) -> ModelWeights:  # fmt: skip
    """random-init weights of the config's shapes: linears bf16 N(0, 0.02), norm weights 1.0, in a fixed tensor order
    (embed; per layer q, k, v, o, gate, up, down). `on_cpu` draws with the CPU generator (small configs whose weights
    the CPU oracle must share); otherwise on the device. storage "p12" encodes every layer linear with pack12.
    `layer_std` is the layers' linears' deviation (the embedding keeps 0.02): a few narrow layers drawn at 0.02 leave
    the residual stream the embedding plus noise and greedy decoding repeats one token, so small test models draw
    theirs wider."""
    from . import pack12

    gdev = "cpu" if on_cpu else device
    g = torch.Generator(device=gdev).manual_seed(seed)
    std = [0.02]

    def lin(r: int, c: int) -> torch.Tensor:
        return (torch.randn(r, c, generator=g, device=gdev, dtype=torch.float32) * std[0]).to(torch.bfloat16).to(device)

    def ones(n: int) -> torch.Tensor:
        return torch.ones(n, dtype=torch.bfloat16, device=device)

    def store(w: torch.Tensor) -> Any:
        if storage == "bf16":
            return w
        return P12Matrix(pack12.pack_bf16(w), w.shape[0], w.shape[1], device)

    H, D = cfg.hidden, cfg.head_dim
    mw = ModelWeights(cfg, lin(cfg.vocab, H), ones(H))
    std[0] = layer_std
    for _ in range(cfg.layers):
        q, k, v = lin(cfg.q_heads * D, H), lin(cfg.kv_heads * D, H), lin(cfg.kv_heads * D, H)
        o = lin(H, cfg.q_heads * D)
        gate, up, down = lin(cfg.inter, H), lin(cfg.inter, H), lin(H, cfg.inter)
        mw.layers.append(
            LayerWeights(
                ones(H), ones(H), store(torch.cat([q, k, v])), store(o), store(torch.cat([gate, up])), store(down),
                ones(D) if cfg.qk_norm else None, ones(D) if cfg.qk_norm else None,
            )
        )  # fmt: skip
        del q, k, v, gate, up
    return mw


def pad_rows(T: int) -> int:
    for m in CARD_ROWS:
        if T <= m:
            return m
    raise ValueError(f"a pass holds at most {CARD_ROWS[-1]} rows, got {T}")


class CardEngine:
    """one model on one card: its cache arena, pass buffers, step graph and greedy loop"""

    def __init__(self, weights: ModelWeights, cap: int = 4096, silu_fold: bool = True, fuse_norm: bool = True,
                 step_kernel: bool = False, device: Any = "cuda"):
        capi.lib()  # fail here, loudly, when the library is not built
        if not torch.cuda.is_available():
            raise RuntimeError("btb_b200 needs a CUDA device: there is no CPU path")
        self.w, self.cfg = weights, weights.cfg
        self.dev = torch.device(device)
        self.cap = int(cap)
        c = self.cfg
        self.cos, self.sin = rope_tables(c, self.cap, self.dev)
        # the arena: per layer K and V position-major [cap, Hk, D] (btb/engine/arena.py:1-5)
        self.K = torch.zeros(c.layers, self.cap, c.kv_heads, c.head_dim, dtype=torch.bfloat16, device=self.dev)
        self.V = torch.zeros_like(self.K)
        self.hs, self.rs = c.head_dim, c.kv_heads * c.head_dim
        self.S = (self.cap + GROUP_KEYS - 1) // GROUP_KEYS
        self.n0 = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.silu_fold = silu_fold
        self.fuse_norm = fuse_norm
        # passes of 4..32 rows over bf16 weights through the tensor cores (btb_b200_gemv_tc_bf16). Off: every pass runs
        # the fp32-chain kernels, whose row r equals the one-row step's row r to the bit - what a speculative verify
        # pass compares. On: prefill chunks and small batches run several times faster; their rows agree with the
        # step's to rounding.
        self.wide_tc = False
        self._tc_ws: Any = None
        self.swiglu_epilogue = True  # SwiGLU in the gate/up GEMV's epilogue (passes of up to 8 rows)
        # ... and the output projection in the same (cooperative) launch
        self.fuse_attn_o = os.environ.get("BTB_B200_FUSE_ATTN_O", "0") == "1"
        self._bar = torch.zeros(2, dtype=torch.int32, device=self.dev)
        self.fuse_attn = True  # the step's row: norm + RoPE + cache write + attention as one launch
        # the whole step as one persistent kernel (head dim 128 only); else one launch a kernel
        self.step_kernel = bool(step_kernel) and weights.cfg.head_dim == 128 and weights.cfg.q_heads // weights.cfg.kv_heads in (2, 4, 8)
        self._programs: dict[Any, Any] = {}
        self._bufs: dict[int, dict[str, torch.Tensor]] = {}
        self._graphs: dict[Any, Any] = {}
        self.pin_tok = torch.zeros(1, dtype=torch.int64).pin_memory()
        self.pin_n0 = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.pin_ts = torch.zeros(1, dtype=torch.int64).pin_memory()
        self.pin_in = torch.zeros(CARD_ROWS[-1], dtype=torch.int64).pin_memory()
        self.launches_per_step = 0
        self._n = 0
        from .sampling import CardSampler

        self.sampler = CardSampler(self.dev)
        self._before = torch.full((1,), -1, dtype=torch.int32, device=self.dev)  # "the row before n0" as a depth

    # -- buffers -------------------------------------------------------------------------------------------------
    def bufs(self, M: int) -> dict[str, torch.Tensor]:
        """the static buffers of a pass of padded width M (btb/engine/cuda.py:1491-1562)"""
        if M in self._bufs:
            return self._bufs[M]
        c, dev = self.cfg, self.dev
        bf = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)  # noqa: E731
        H, Hq, D = c.hidden, c.q_heads, c.head_dim
        g = {
            "h": bf(M, H), "h2": bf(M, H), "x": bf(M, H), "y": bf(M, H), "qkv": bf(M, c.qkv_rows), "q": bf(M, Hq, D),
            "att": bf(M, Hq * D), "gu": bf(M, 2 * c.inter), "m": bf(M, c.inter), "logits": bf(M, c.vocab),
            "ids": torch.zeros(M, dtype=torch.int64, device=dev),
            "tok": torch.zeros(M, dtype=torch.int64, device=dev),
            "depth": torch.arange(M, dtype=torch.int32, device=dev),
            "par": torch.arange(-1, M - 1, dtype=torch.int32, device=dev),
            "part_m": torch.zeros(self.S * M * Hq, dtype=torch.float32, device=dev),
            "part_l": torch.zeros(self.S * M * Hq, dtype=torch.float32, device=dev),
            "part_acc": torch.zeros(self.S * M * Hq * D, dtype=torch.float32, device=dev),
            "cnt": torch.zeros(M * c.q_heads, dtype=torch.int32, device=dev),
            "pick": torch.zeros((int(capi.lib().btb_b200_argmax_scratch_bytes(M)) + 7) // 8, dtype=torch.int64,
                                device=dev),
        }  # fmt: skip
        self._bufs[M] = g
        return g

    # -- the pass ------------------------------------------------------------------------------------------------
    def _k(self, name: str, *args: Any) -> None:
        """one kernel launch through the C-ABI, counted"""
        call(name, *args)
        self._n += 1

    def _matvec(self, W: Any, x: torch.Tensor, y: torch.Tensor, M: int, R: int, C_: int, s: int) -> None:
        if self.wide_tc and M >= 4 and (isinstance(W, torch.Tensor) or (isinstance(W, P12Matrix) and C_ % 64 == 0)):
            # a pass of several rows over bf16 or pack12 weights: the tensor-core matvec (its own summation order; the
            # packed store is widened tile by tile on its way into the MMA's operand - the same sums as over a bf16 copy)
            need = int(capi.lib().btb_b200_gemv_tc_workspace_bytes(R, C_))
            if self._tc_ws is None or self._tc_ws.numel() * 4 < need:
                self._tc_ws = torch.zeros(max(need // 4, 4), dtype=torch.float32, device=self.dev)
            if isinstance(W, P12Matrix):
                self._k("btb_b200_gemv_tc_p12", ptr(W.lo), ptr(W.hi4), W.table, ptr(W.esc_idx), ptr(W.esc_val),
                        ptr(W.esc_row), ptr(x), ptr(y), M, R, C_, ptr(self._tc_ws), s)  # fmt: skip
            else:
                self._k("btb_b200_gemv_tc_bf16", ptr(W), ptr(x), ptr(y), M, R, C_, ptr(self._tc_ws), s)
            if need:
                self._n += 1  # the ordered sum of the K ranges is a launch of its own
            return
        if isinstance(W, P12Matrix):
            self._k("btb_b200_gemv_p12", ptr(W.lo), ptr(W.hi4), W.table, ptr(W.esc_idx), ptr(W.esc_val),
                    ptr(W.esc_row), ptr(x), ptr(y), M, R, C_, s)  # fmt: skip
        elif isinstance(W, FP8Matrix):
            self._k("btb_b200_gemv_fp8", ptr(W.w), ptr(W.scales), W.sr, W.sc, ptr(x), ptr(y), M, R, C_, s)
        else:
            self._k("btb_b200_gemv_bf16", ptr(W), ptr(x), ptr(y), M, R, C_, s)

    def body(self, T: int, tail: bool = True, stream_ptr: int | None = None) -> None:
        """the pass's kernels over the width's buffers (btb/engine/cuda.py:1601-1837): T live rows, padded to M"""
        c = self.cfg
        M = pad_rows(T)
        g = self.bufs(M)
        s = capi.stream_ptr() if stream_ptr is None else stream_ptr
        H, Hq, Hk, D, I = c.hidden, c.q_heads, c.kv_heads, c.head_dim, c.inter
        k = self._k
        # the residual ping-pongs between two buffers when the norm is folded into the GEMV that reads it (a CTA must
        # not read a row another CTA is updating); the pass starts and ends on g["h"]
        tc = self.wide_tc and M >= 4 and isinstance(self.w.layers[0].qkv, (torch.Tensor, P12Matrix))
        fuse = self.fuse_norm and M <= 8 and M * max(H, 1) * 2 <= 64 * 1024 and not tc
        hcur, halt = g["h"], g["h2"]

        def normed_matvec(W: Any, norm_w: torch.Tensor, y_add: Any, out: torch.Tensor, R: int,
                          swiglu: bool = False) -> None:
            nonlocal hcur, halt
            if fuse:
                p12 = isinstance(W, P12Matrix)
                parts = ((ptr(W.lo), ptr(W.hi4), W.table, ptr(W.esc_idx), ptr(W.esc_val), ptr(W.esc_row)) if p12
                         else (ptr(W), 0, 0, 0, 0, 0))  # fmt: skip
                k("btb_b200_gemv_norm_swiglu" if swiglu else "btb_b200_gemv_norm", *parts, ptr(hcur), ptr(y_add),
                  ptr(norm_w), c.eps, 0, ptr(halt) if y_add is not None else 0, ptr(out), T, M, R, H, s)
                if y_add is not None:
                    hcur, halt = halt, hcur
            else:
                k("btb_b200_add_rmsnorm", ptr(hcur), ptr(y_add), ptr(norm_w), c.eps, ptr(g["x"]), T, H, 0, s)
                self._matvec(W, g["x"], out, M, R, H, s)

        y_prev = None
        for i, L in enumerate(self.w.layers):
            normed_matvec(L.qkv, L.ln1, y_prev, g["qkv"], c.qkv_rows)
            if T == 1 and self.fuse_attn_o and self.fuse_attn and D in (64, 128) and isinstance(L.o, torch.Tensor):
                # the step's attention row and its output projection in one cooperative launch
                k("btb_b200_attn_o_step", ptr(g["qkv"]), ptr(L.wq), ptr(L.wk), c.eps, ptr(self.cos), ptr(self.sin),
                  ptr(self.n0), ptr(g["depth"]), ptr(self.K[i]), ptr(self.V[i]), ptr(g["q"]), ptr(g["att"]), Hq, Hk, D,
                  self.hs, self.rs, 0, float(D**-0.5), ptr(g["part_m"]), ptr(g["part_l"]), ptr(g["part_acc"]),
                  ptr(g["cnt"]), 0, 0, self.cap, ptr(L.o), ptr(g["y"]), H, ptr(self._bar), s)  # fmt: skip
            else:
                self._attention(g, i, L.wq, L.wk, T, s, warm=(L.o, L.gu))
                self._matvec(L.o, g["att"], g["y"], M, H, Hq * D, s)
            if fuse and self.swiglu_epilogue and not isinstance(L.gu, FP8Matrix):
                # the gate/up GEMV activates each pair itself: g["gu"] is never written, the down GEMV reads g["m"]
                normed_matvec(L.gu, L.ln2, g["y"], g["m"], 2 * I, swiglu=True)
                self._matvec(L.down, g["m"], g["y"], M, H, I, s)
                y_prev = g["y"]
                continue
            if tc and isinstance(L.gu, torch.Tensor):
                # the tensor-core matvec's gate/up form: the activation in its epilogue (the matvec and silu_mul, to the bit)
                k("btb_b200_add_rmsnorm", ptr(hcur), ptr(g["y"]), ptr(L.ln2), c.eps, ptr(g["x"]), T, H, 0, s)
                need = int(capi.lib().btb_b200_gemv_tc_glu_workspace_bytes(I, H))
                if self._tc_ws is None or self._tc_ws.numel() * 4 < need:
                    self._tc_ws = torch.zeros(max(need // 4, 4), dtype=torch.float32, device=self.dev)
                k("btb_b200_gemv_tc_glu_bf16", ptr(L.gu), ptr(g["x"]), ptr(g["m"]), M, I, H, ptr(self._tc_ws), s)
                if need:
                    self._n += 1
                self._matvec(L.down, g["m"], g["y"], M, H, I, s)
                y_prev = g["y"]
                continue
            normed_matvec(L.gu, L.ln2, g["y"], g["gu"], 2 * I)
            if self.silu_fold and M <= 8 and M * I * 2 <= 160 * 1024 and not tc:
                if isinstance(L.down, P12Matrix):
                    W = L.down
                    k("btb_b200_gemv_silu_p12", ptr(W.lo), ptr(W.hi4), W.table, ptr(W.esc_idx), ptr(W.esc_val),
                      ptr(W.esc_row), ptr(g["gu"]), ptr(g["y"]), M, H, I, s)  # fmt: skip
                else:
                    k("btb_b200_gemv_silu_bf16", ptr(L.down), ptr(g["gu"]), ptr(g["y"]), M, H, I, s)
            else:
                k("btb_b200_silu_mul", ptr(g["gu"]), ptr(g["m"]), M, I, s)
                self._matvec(L.down, g["m"], g["y"], M, H, I, s)
            y_prev = g["y"]
        if tail:
            normed_matvec(self.w.embed, self.w.norm, y_prev, g["logits"], c.vocab)
        if hcur is not g["h"]:  # an odd number of folded adds (a pass without its tail): bring the residual home
            g["h"].copy_(hcur)

    @staticmethod
    def _warm(W: Any) -> tuple[int, int]:
        """(address, bytes) of a bf16 matrix for the attention launch's L2 warming, nothing for packed stores"""
        if isinstance(W, torch.Tensor):
            return ptr(W), (W.numel() * W.element_size()) & ~15
        return 0, 0

    def _attention(self, g: dict, i: int, wq: Any, wk: Any, T: int, s: int, win: int = 0, sinks: Any = None,
                   out: Any = None, warm: tuple = ()) -> None:
        """q/k-norm + RoPE + cache write, then the attention over the cache: one fused launch for the step's single
        row, the two kernels for a pass of several rows (the same bits either way). `warm`: the matrices the next
        kernels stream, pulled into L2 by the SMs the step's row leaves idle (the `l2_warm_kb` tunable bounds it)"""
        c = self.cfg
        Hq, Hk, D = c.q_heads, c.kv_heads, c.head_dim
        out = g["att"] if out is None else out
        if T == 1 and self.fuse_attn and D in (64, 128):
            (wa, na), (wb, nb) = (self._warm(warm[0]) if len(warm) > 0 else (0, 0)), (self._warm(warm[1]) if len(warm) > 1 else (0, 0))
            self._k("btb_b200_attn_step_w", ptr(g["qkv"]), ptr(wq), ptr(wk), c.eps, ptr(self.cos), ptr(self.sin),
                    ptr(self.n0), ptr(g["depth"]), ptr(self.K[i]), ptr(self.V[i]), ptr(g["q"]), ptr(out), Hq, Hk,
                    D, self.hs, self.rs, 0, float(D**-0.5), ptr(g["part_m"]), ptr(g["part_l"]), ptr(g["part_acc"]),
                    ptr(g["cnt"]), win, 0, ptr(sinks), self.cap, None, wa, na, wb, nb, s)  # fmt: skip
            return
        self._k("btb_b200_norm_rope_kv", ptr(g["qkv"]), ptr(wq), ptr(wk), c.eps, ptr(self.cos), ptr(self.sin),
                ptr(self.n0), ptr(g["depth"]), ptr(self.K[i]), ptr(self.V[i]), ptr(g["q"]), T, Hq, Hk, D, self.hs,
                self.rs, 0, 0, self.cap, s)  # fmt: skip
        self._k("btb_b200_attn_decode", ptr(g["q"]), ptr(self.K[i]), ptr(self.V[i]), ptr(out), ptr(self.n0),
                ptr(g["par"]), T, Hq, Hk, D, self.hs, self.rs, float(D**-0.5), ptr(g["part_m"]), ptr(g["part_l"]),
                ptr(g["part_acc"]), ptr(g["cnt"]), win, 0, ptr(sinks), self.cap, s)  # fmt: skip

    def _embed(self, g: dict, T: int, s: int) -> None:
        self._k("btb_b200_embed", ptr(self.w.embed), ptr(g["ids"]), ptr(g["h"]), T, self.cfg.hidden, self.cfg.vocab, s)

    def _pick(self, g: dict, T: int, s: int, out: torch.Tensor) -> None:
        """the pass's tokens: the lowest-index argmax, or the sampler's draw keyed by each row's cache position"""
        if self.sampler.sampling.greedy:
            self._k("btb_b200_argmax_bf16", ptr(g["logits"]), T, self.cfg.vocab, ptr(g["pick"]), ptr(out), s)
        else:
            self.sampler.pick(g["logits"], T, self.n0, g.get("depth"), out, s)
            self._n += 1

    def set_sampling(self, sampling: Any) -> None:
        """greedy or sampled picks from here on (btb/sampling.py:34-61); temperature, top-p and seed are data to a
        captured step graph, greedy/sampled and top-k are part of its shape"""
        self.sampler.set(sampling)

    # -- passes --------------------------------------------------------------------------------------------------
    def reset(self) -> None:
        self.n0.zero_()

    def forward(self, ids: torch.Tensor, depth: Any = None, parents: Any = None, advance: bool = True) -> torch.Tensor:
        """one eager pass of T rows after the cache's rows (a chain by default); returns bf16 logits [T, V]"""
        T = int(ids.numel())
        M = pad_rows(T)
        g = self.bufs(M)
        s = capi.stream_ptr()
        g["ids"][:T].copy_(ids.to(self.dev, torch.int64))
        if depth is not None:
            g["depth"][:T].copy_(torch.as_tensor(depth, dtype=torch.int32))
            g["par"][:T].copy_(torch.as_tensor(parents, dtype=torch.int32))
        else:
            g["depth"][:M].copy_(torch.arange(M, dtype=torch.int32))
            g["par"][:M].copy_(torch.arange(-1, M - 1, dtype=torch.int32))
        self._embed(g, T, s)
        self.body(T)
        if advance:
            call("btb_b200_publish", ptr(self.n0), 0, 0, 0, 0, T, s)
        return g["logits"][:T]

    # -- prefill on the tensor cores -------------------------------------------------------------------------------
    def prefill_gemm(self, prompt: torch.Tensor, chunk: int = 256) -> torch.Tensor:
        """the prompt in chunks of up to `chunk` rows with every linear a tensor-core GEMM (btb_b200_gemm_tc_bf16) - the
        reference's prefill (btb/engine/cuda.py:2817-3039 `_forward_card_prefill`: the step's own kernels over T rows, the
        matvecs replaced by the GEMM whose rows are the tensor-core matvec's). The attention runs the decode kernel over
        the chunk 32 rows at a time (each row against the cache rows before it and the chunk's rows up to itself, all
        written by the chunk's norm + RoPE pass beforehand). bf16 weights only. Returns the last row's logits [1, V];
        a row's values are the 32-row tensor-core pass's (`wide_tc`), to rounding the fp32-chain pass's."""
        c = self.cfg
        if not isinstance(self.w.layers[0].qkv, torch.Tensor):
            raise TypeError("prefill_gemm reads bf16 weights")
        H, Hq, Hk, D, I = c.hidden, c.q_heads, c.kv_heads, c.head_dim, c.inter
        P = int(chunk)
        if "wide" not in self._programs or self._programs["wide"]["h"].shape[0] < P:
            bf = lambda *s_: torch.zeros(*s_, dtype=torch.bfloat16, device=self.dev)  # noqa: E731
            self._programs["wide"] = {
                "h": bf(P, H), "x": bf(P, H), "y": bf(P, H), "qkv": bf(P, c.qkv_rows), "q": bf(P, Hq, D), "att": bf(P, Hq * D),
                "gu": bf(P, 2 * I), "m": bf(P, I), "ids": torch.zeros(P, dtype=torch.int64, device=self.dev),
                "depth": torch.arange(P, dtype=torch.int32, device=self.dev),
                "n0s": torch.zeros((P + 31) // 32, dtype=torch.int32, device=self.dev),
            }  # fmt: skip
        b, g32 = self._programs["wide"], self.bufs(32)
        s = capi.stream_ptr()
        k = self._k
        prompt = prompt.to(self.dev, torch.int64)
        n = int(prompt.numel())
        for a in range(0, n, P):
            T = min(P, n - a)
            b["ids"][:T].copy_(prompt[a : a + T])
            b["n0s"].copy_(self.n0 + torch.arange(0, b["n0s"].numel() * 32, 32, dtype=torch.int32, device=self.dev))
            k("btb_b200_embed", ptr(self.w.embed), ptr(b["ids"]), ptr(b["h"]), T, H, c.vocab, s)
            y_prev = None
            for i, L in enumerate(self.w.layers):
                k("btb_b200_add_rmsnorm", ptr(b["h"]), ptr(y_prev), ptr(L.ln1), c.eps, ptr(b["x"]), T, H, 0, s)
                k("btb_b200_gemm_tc_bf16", ptr(L.qkv), ptr(b["x"]), ptr(b["qkv"]), T, c.qkv_rows, H, s)
                k("btb_b200_norm_rope_kv", ptr(b["qkv"]), ptr(L.wq), ptr(L.wk), c.eps, ptr(self.cos), ptr(self.sin),
                  ptr(self.n0), ptr(b["depth"]), ptr(self.K[i]), ptr(self.V[i]), ptr(b["q"]), T, Hq, Hk, D, self.hs, self.rs,
                  0, 0, self.cap, s)  # fmt: skip
                for j, r0 in enumerate(range(0, T, 32)):  # rows r0 .. r0 + 31: a chain standing after n0 + r0 rows
                    rows = min(32, T - r0)
                    k("btb_b200_attn_decode", ptr(b["q"][r0]), ptr(self.K[i]), ptr(self.V[i]), ptr(b["att"][r0]),
                      ptr(b["n0s"][j : j + 1]), ptr(g32["par"]), rows, Hq, Hk, D, self.hs, self.rs, float(D**-0.5),
                      ptr(g32["part_m"]), ptr(g32["part_l"]), ptr(g32["part_acc"]), ptr(g32["cnt"]), 0, 0, 0, self.cap, s)  # fmt: skip
                k("btb_b200_gemm_tc_bf16", ptr(L.o), ptr(b["att"]), ptr(b["y"]), T, H, Hq * D, s)
                k("btb_b200_add_rmsnorm", ptr(b["h"]), ptr(b["y"]), ptr(L.ln2), c.eps, ptr(b["x"]), T, H, 0, s)
                k("btb_b200_gemm_tc_bf16", ptr(L.gu), ptr(b["x"]), ptr(b["gu"]), T, 2 * I, H, s)
                k("btb_b200_silu_mul", ptr(b["gu"]), ptr(b["m"]), T, I, s)
                k("btb_b200_gemm_tc_bf16", ptr(L.down), ptr(b["m"]), ptr(b["y"]), T, H, I, s)
                y_prev = b["y"]
            call("btb_b200_publish", ptr(self.n0), 0, 0, 0, 0, T, s)
            last = T - 1
        # the last row's logits: the final norm and the head over that one row
        g1 = self.bufs(1)
        g1["h"].copy_(b["h"][last : last + 1])
        g1["y"].copy_(b["y"][last : last + 1])
        k("btb_b200_add_rmsnorm", ptr(g1["h"]), ptr(g1["y"]), ptr(self.w.norm), c.eps, ptr(g1["x"]), 1, H, 0, s)
        self._matvec(self.w.embed, g1["x"], g1["logits"], 1, c.vocab, H, s)
        return g1["logits"][:1]

    def prefill(self, prompt: torch.Tensor) -> torch.Tensor:
        """the prompt through chain passes of up to 32 rows; returns the last row's logits"""
        lg = None
        for a in range(0, int(prompt.numel()), CARD_ROWS[-1]):
            lg = self.forward(prompt[a : a + CARD_ROWS[-1]])
        assert lg is not None
        return lg[-1:]

    # -- the step graph ------------------------------------------------------------------------------------------
    def program(self, M: int, steps: int = 1, pick: bool = True, publish: bool = True) -> Any:
        """the whole-step kernel's program for a pass width (built once, its records live on the card)"""
        from .step import StepProgram

        key = (M, steps, pick, publish)
        if key not in self._programs:
            self._programs[key] = StepProgram(self, M, steps, pick, publish)
        return self._programs[key]

    def _step_body(self, s: int, publish: bool, steps: int = 1) -> None:
        """embed(ids) -> layers -> head -> greedy pick into ids -> n0 += 1 (and the handoff to pinned memory)"""
        if self.step_kernel and self.sampler.sampling.greedy:
            self.program(1, steps, True, publish).launch(stream=torch.cuda.current_stream())
            self.launches_per_step = 1.0 / steps
            return
        for _ in range(steps):
            self._step_body_launches(s, publish)

    def _step_body_launches(self, s: int, publish: bool) -> None:
        g = self.bufs(1)
        self._n = 0
        self._embed(g, 1, s)
        self.body(1, stream_ptr=s)
        self._pick(g, 1, s, g["ids"])
        if publish:
            self._k("btb_b200_publish", ptr(self.n0), ptr(g["ids"]), ptr(self.pin_tok), ptr(self.pin_n0),
                    ptr(self.pin_ts), 1, s)  # fmt: skip
        else:
            self._k("btb_b200_publish", ptr(self.n0), 0, 0, 0, 0, 1, s)
        self.launches_per_step = self._n

    def step_graph(self, steps: int = 1, publish: bool = True) -> Any:
        """`steps` self-advancing decode steps as one CUDA graph (btb/engine/cuda.py:2101-2251)"""
        key = ("step", steps, publish, self.sampler.sampling.greedy, self.sampler.top_k)
        if key in self._graphs:
            return self._graphs[key]
        # run once eagerly on a side stream (allocations, shared-memory opt-ins), with the state put back after
        n_keep, ids_keep = self.n0.clone(), self.bufs(1)["ids"].clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._step_body(capi.stream_ptr(side), publish, steps)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.n0.copy_(n_keep)
        self.bufs(1)["ids"].copy_(ids_keep)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._step_body(capi.stream_ptr(), publish, steps)
        self.n0.copy_(n_keep)
        self.bufs(1)["ids"].copy_(ids_keep)
        self._graphs[key] = graph
        return graph

    def generate(self, prompt: Any, max_new: int, sampling: Any = None) -> list[int]:
        """`generate_greedy`'s loop under a sampling: every pick is keyed by (seed, the cache row that decides it)"""
        if sampling is not None:
            self.set_sampling(sampling)
        return self.generate_greedy(prompt, max_new)

    def generate_greedy(self, prompt: Any, max_new: int, graph_steps: int = 1) -> list[int]:
        """prefill, the first token from the prompt's last logits, then the step graph replayed; tokens come back
        through pinned host memory (btb/engine/cuda.py:2253-2459)"""
        prompt = torch.as_tensor(prompt, dtype=torch.int64)
        self.reset()
        last = self.prefill(prompt)
        g = self.bufs(1)
        s = capi.stream_ptr()
        self._pick({"logits": last.contiguous(), "pick": g["pick"], "depth": self._before}, 1, s, g["ids"])
        toks = [int(g["ids"][0].item())]
        graph = self.step_graph(1, publish=True)
        while len(toks) < max_new:
            graph.replay()
            torch.cuda.current_stream().synchronize()
            toks.append(int(self.pin_tok[0]))
        return toks

    def continue_from(self, logits: torch.Tensor, max_new: int, sampling: Any = None) -> list[int]:
        """`max_new` tokens after the cache's rows, given the logits that follow them ([V] or [1, V], any float dtype as
        long as the values are the pass's bf16 logits): the first picked from `logits`, the rest by the step graph - what
        `generate_greedy` does after its prefill. The last token is drawn but not fed (its row is not in the cache)."""
        if sampling is not None:
            self.set_sampling(sampling)
        g = self.bufs(1)
        s = capi.stream_ptr()
        last = logits.reshape(1, -1).to(self.dev, torch.bfloat16).contiguous()
        self._pick({"logits": last, "pick": g["pick"], "depth": self._before}, 1, s, g["ids"])
        toks = [int(g["ids"][0].item())]
        graph = self.step_graph(1, publish=True)
        while len(toks) < max_new:
            graph.replay()
            torch.cuda.current_stream().synchronize()
            toks.append(int(self.pin_tok[0]))
        return toks

    def session(self) -> Any:
        """a `Session` over this engine (btb's `model.session()`)"""
        from .session import Session

        return Session(self)

    def generate_speculative(self, prompt: Any, max_new: int, budget: int = 8, v_max: int = 8) -> tuple[list[int], dict]:
        """greedy decode with n-gram tree drafts verified a tree a pass (btb/engine/generate.py:682-795); the tokens
        are generate_greedy's"""
        from .draft import generate_speculative

        return generate_speculative(self, prompt, max_new, budget, v_max)

    def step(self, token: int) -> int:
        """the public one-token call: the token from pinned host memory to the card, one step, the next token back"""
        g = self.bufs(1)
        self.pin_in[0] = token
        g["ids"][:1].copy_(self.pin_in[:1], non_blocking=True)
        self.step_graph(1, publish=True).replay()
        torch.cuda.current_stream().synchronize()
        return int(self.pin_tok[0])

    def weight_bytes(self) -> int:
        tot = self.w.embed.numel() * 2
        for L in self.w.layers:
            for W in (L.qkv, L.o, L.gu, L.down):
                tot += W.nbytes if isinstance(W, P12Matrix) else W.numel() * 2
        return tot


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


__all__ = ["CardEngine", "DenseConfig", "ModelWeights", "LayerWeights", "P12Matrix", "QWEN3_4B", "LLAMA31_70B",
           "synth_weights", "rope_tables", "pad_rows"]  # fmt: skip
