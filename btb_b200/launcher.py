"""A ``Launcher`` for btb's card-kernel seam, served by the sm_100a library.

btb launches every card kernel through an object with one method (btb/engine/card_launch.py:428-440 of btb)::

    launch(name, grid, block, args, stream=None, shared=0)

``name`` is the kernel's symbol in native/cuda/btb_kernels.cu, ``args`` one ctypes value per kernel parameter in the
kernel's own order. ``B200Launcher`` accepts exactly those calls for the kernel families this library replaces and
routes each to its C-ABI function; ``grid``/``block``/``shared`` describe the reference kernels' launch shapes and are
only read where they carry information the parameters do not (the row count of ``btb_add_rmsnorm`` is its grid, the
capacity of ``btb_attn_flash`` its grid's second extent). A kernel outside the replaced families raises
``KeyError`` - there is no fallback.

The typed functions below (``btb_gemv_bf16(launcher, M, grid, block, w, x, y, R, C)`` ...) mirror the generated
launchers of card_launch.py so call sites written against the reference read the same here.
"""

from __future__ import annotations

import ctypes as C
import re
from collections.abc import Sequence
from typing import Any

from . import capi

Dim3 = tuple[int, int, int]
INT_MAX = 2**31 - 1


def _v(a: Any) -> Any:
    """a ctypes value's payload (None for a null c_void_p), a plain Python number as is"""
    return a.value if isinstance(a, C._SimpleCData) else a


def _p(a: Any) -> int:
    v = _v(a)
    return 0 if v is None else int(v)


class B200Launcher:
    """launch(name, ...) of the reference's kernels on the B200 library; holds no state but the loaded library"""

    #: the reference kernel families served (regex -> handler name)
    FAMILIES = (
        (r"btb_gemv_bf16_m(\d+)$", "_gemv_bf16"),
        (r"btb_gemv_silu_bf16_m(\d+)$", "_gemv_silu"),
        (r"btb_gemv_mma_bf16$", "_gemv_mma"),
        (r"btb_gemv_mma8_bf16$", "_gemv_mma"),  # the reference's 8-rows-a-warp launch shape of the same sums
        (r"btb_gemv_mma_glu_silu$", "_gemv_mma_glu"),
        (r"btb_add_rmsnorm$", "_add_rmsnorm"),
        (r"btb_silu_mul$", "_silu_mul"),
        (r"btb_norm_rope_kv_d(\d+)$", "_norm_rope_kv"),
        (r"btb_norm_rope_kv_tbl_d(\d+)$", "_norm_rope_kv"),
        (r"btb_attn_flash_d(\d+)$", "_attn_flash"),
        (r"btb_norm_rope_kv_rows_d(\d+)$", "_norm_rope_kv_rows"),
        (r"btb_attn_flash_rows_d(\d+)$", "_attn_flash_rows"),
        (r"btb_publish$", "_publish"),
        (r"btb_moe_route$", "_moe_route"),
        (r"btb_gemv_lane16_f32_m(\d+)$", "_gemv_lane16"),
        (r"btb_gemv_lane16_mx4_f32_m(\d+)$", "_gemv_lane16_mx4"),
        (r"btb_sample_keys$", "_sample_keys"),
        (r"btb_sample_max$", "_sample_max"),
        (r"btb_sample_hist$", "_sample_level"),
        (r"btb_sample_bin$", "_sample_bin"),
        (r"btb_sample_draw$", "_sample_draw"),
        (r"btb_sample_out$", "_sample_out"),
        (r"btb_sample_verify$", "_sample_verify"),
    )

    def __init__(self) -> None:
        self.lib = capi.lib()
        self._tc_ws: Any = None  # the tensor-core matvec's partial sums (matrices of few rows)
        self._top_k = 0  # the pick being assembled: the reference launches it as a pipeline of kernels
        self._families = [(re.compile(rx), getattr(self, h)) for rx, h in self.FAMILIES if hasattr(self, h)]

    def serves(self, name: str) -> bool:
        return any(rx.match(name) for rx, _ in self._families)

    def launch(
        self, name: str, grid: Dim3, block: Dim3, args: Sequence[Any], stream: Any = None, shared: int = 0
    ) -> None:
        for rx, handler in self._families:
            m = rx.match(name)
            if m:
                handler(name, m, grid, list(args), capi.stream_ptr(stream))
                return
        raise KeyError(f"{name}: not a kernel family of the B200 library")

    # -- handlers: the reference kernel's parameter list -> the C-ABI call ------------------------------------------
    def _gemv_bf16(self, name, m, grid, a, s):
        w, x, y, R, Cc = a
        capi.call("btb_b200_gemv_bf16", _p(w), _p(x), _p(y), int(m.group(1)), int(_v(R)), int(_v(Cc)), s)

    def _gemv_silu(self, name, m, grid, a, s):
        w, gu, y, R, Cc = a
        capi.call("btb_b200_gemv_silu_bf16", _p(w), _p(gu), _p(y), int(m.group(1)), int(_v(R)), int(_v(Cc)), s)

    def _gemv_mma(self, name, m, grid, a, s):
        # btb_gemv_mma_bf16(w [R, C], x [32, C], y [32, R], R, C, M): the tensor-core matvec, M live rows
        w, x, y, R, Cc, M = a
        R, Cc = int(_v(R)), int(_v(Cc))
        ws = self._workspace(int(self.lib.btb_b200_gemv_tc_workspace_bytes(R, Cc)))
        capi.call("btb_b200_gemv_tc_bf16", _p(w), _p(x), _p(y), int(_v(M)), R, Cc, ws, s)

    def _gemv_mma_glu(self, name, m, grid, a, s):
        # btb_gemv_mma_glu_silu(w [2I, C], x [32, C], m [32, I], I, C, M): gate/up and the activation in one launch
        w, x, mm, I, Cc, M = a
        I, Cc = int(_v(I)), int(_v(Cc))
        ws = self._workspace(int(self.lib.btb_b200_gemv_tc_glu_workspace_bytes(I, Cc)))
        capi.call("btb_b200_gemv_tc_glu_bf16", _p(w), _p(x), _p(mm), int(_v(M)), I, Cc, ws, s)

    def _workspace(self, need: int) -> int:
        """the tensor-core matvecs' partial sums (matrices of few rows): one buffer, grown as asked"""
        import torch

        if need and (self._tc_ws is None or self._tc_ws.numel() * 4 < need):
            self._tc_ws = torch.zeros(need // 4, dtype=torch.float32, device="cuda")
        return 0 if not need else int(self._tc_ws.data_ptr())

    def _add_rmsnorm(self, name, m, grid, a, s):
        h, y, w, eps, x, H, cen = a
        capi.call("btb_b200_add_rmsnorm", _p(h), _p(y), _p(w), float(_v(eps)), _p(x), int(grid[0]), int(_v(H)),
                  int(_v(cen)), s)  # fmt: skip

    def _silu_mul(self, name, m, grid, a, s):
        gu, mm, T, I = a
        capi.call("btb_b200_silu_mul", _p(gu), _p(mm), int(_v(T)), int(_v(I)), s)

    def _norm_rope_kv(self, name, m, grid, a, s):
        tbl = a[17] if len(a) > 17 else None
        qkv, wq, wk, eps, cos, sin, n0p, depth, K, V, qo, T, Hq, Hk, hs, rs, cen = a[:17]
        capi.call("btb_b200_norm_rope_kv", _p(qkv), _p(wq), _p(wk), float(_v(eps)), _p(cos), _p(sin), _p(n0p),
                  _p(depth), _p(K), _p(V), _p(qo), int(_v(T)), int(_v(Hq)), int(_v(Hk)), int(m.group(1)),
                  int(_v(hs)), int(_v(rs)), int(_v(cen)), _p(tbl), INT_MAX, s)  # fmt: skip

    def _attn_flash(self, name, m, grid, a, s):
        q, K, V, out, n0p, par, T, Hq, Hk, hs, rs, scale, pm, pl, pa, cnt, win, tbl = a
        capi.call("btb_b200_attn_decode", _p(q), _p(K), _p(V), _p(out), _p(n0p), _p(par), int(_v(T)), int(_v(Hq)),
                  int(_v(Hk)), int(m.group(1)), int(_v(hs)), int(_v(rs)), float(_v(scale)), _p(pm), _p(pl), _p(pa),
                  _p(cnt), int(_v(win)), _p(tbl), 0, int(grid[1]) * 512, s)  # fmt: skip

    def _norm_rope_kv_rows(self, name, m, grid, a, s):
        qkv, wq, wk, eps, cos, sin, rw, K, V, qo, T, Hq, Hk, hs, rs, cen = a
        capi.call("btb_b200_norm_rope_kv_rows", _p(qkv), _p(wq), _p(wk), float(_v(eps)), _p(cos), _p(sin), _p(rw), _p(K),
                  _p(V), _p(qo), int(_v(T)), int(_v(Hq)), int(_v(Hk)), int(m.group(1)), int(_v(hs)), int(_v(rs)),
                  int(_v(cen)), INT_MAX, s)  # fmt: skip

    def _attn_flash_rows(self, name, m, grid, a, s):
        q, K, V, out, rw, T, Hq, Hk, hs, rs, scale, pm, pl, pa, cnt, win = a
        capi.call("btb_b200_attn_decode_rows", _p(q), _p(K), _p(V), _p(out), _p(rw), int(_v(T)), int(_v(Hq)), int(_v(Hk)),
                  int(m.group(1)), int(_v(hs)), int(_v(rs)), float(_v(scale)), _p(pm), _p(pl), _p(pa), _p(cnt),
                  int(_v(win)), 0, int(grid[1]) * 512, s)  # fmt: skip

    def _publish(self, name, m, grid, a, s):
        n0, ids, out_tok, out_n0, out_ts = a
        capi.call("btb_b200_publish", _p(n0), _p(ids), _p(out_tok), _p(out_n0), _p(out_ts), 0, s)

    def _moe_route(self, name, m, grid, a, s):
        logits, ls, E, k, idx, w, hidx, hw, cnt, seq, hseq = a
        if _p(hidx) or _p(hseq):
            raise KeyError("btb_moe_route: the host publish is not served (the experts run on the card)")
        capi.call("btb_b200_moe_route", _p(logits), int(_v(ls)), int(_v(E)), int(_v(k)), 0, 0, _p(idx), _p(w),
                  int(grid[0]), s)  # fmt: skip

    def _gemv_lane16(self, name, m, grid, a, s):
        w, x, y, R, Cc = a
        capi.call("btb_b200_gemv_lane16_f32", _p(w), _p(x), _p(y), int(m.group(1)), int(_v(R)), int(_v(Cc)), s)

    def _gemv_lane16_mx4(self, name, m, grid, a, s):
        blocks, scales, x, y, R, Cc = a
        capi.call("btb_b200_gemv_lane16_mx4_f32", _p(blocks), _p(scales), _p(x), _p(y), int(m.group(1)), int(_v(R)),
                  int(_v(Cc)), s)  # fmt: skip


    # the sampled pick (native/cuda/btb_kernels.cu:1865-2124). The reference runs max -> three radix levels for top-k
    # -> three for top-p -> draw as separate launches sharing global scratch; the library does all of it inside the
    # draw's launch. The earlier stages only tell this launcher the pick's shape: max opens a pick, a count-mode bin
    # carries top_k; whether the nucleus applies is read from fp[1] on the card (top_p < 1), which is what decides
    # whether the reference's host launches the mass-mode levels at all.
    def _sample_keys(self, name, m, grid, a, s):
        seed, pos, salt, keys = a
        capi.call("btb_b200_sample_keys", _p(seed), _p(pos), int(_v(salt)), _p(keys), s)

    def _sample_max(self, name, m, grid, a, s):
        self._top_k = 0

    def _sample_level(self, name, m, grid, a, s):
        pass

    def _sample_bin(self, name, m, grid, a, s):
        level, mode, top_k = (int(_v(v)) for v in a[:3])
        if mode == 0:
            self._top_k = top_k

    def _sample_draw(self, name, m, grid, a, s):
        x, keys, V, fp, gM, gpreK, gpreP, gbest = a
        R = int(grid[1])
        capi.call("btb_b200_sample_pick", _p(x), 1, R, int(_v(V)), int(_v(V)), _p(fp), self._top_k, _p(keys), 0, 0, 0,
                  0, 0, 0, _p(gbest), s)  # fmt: skip
        self._top_k = 0

    def _sample_out(self, name, m, grid, a, s):
        gbest, out, R = a
        capi.call("btb_b200_sample_out", _p(gbest), _p(out), int(_v(R)), s)

    def _sample_verify(self, name, m, grid, a, s):
        x, q, kids, hasq, keys, V, Vd, Cw, top_k, fp, out = a
        capi.call("btb_b200_sample_verify", _p(x), 1, int(grid[0]), int(_v(V)), int(_v(V)), _p(q), int(_v(Vd)), _p(kids),
                  int(_v(Cw)), _p(hasq), _p(keys), int(_v(top_k)), _p(fp), _p(out), s)  # fmt: skip


# -- typed launchers, the reference's names and argument order (btb/engine/card_launch.py) --------------------------
_P, _I, _F = C.c_void_p, C.c_int, C.c_float


def btb_gemv_bf16(launcher, M, grid, block, w, x, y, R, C_, *, stream=None, shared=0):
    launcher.launch(f"btb_gemv_bf16_m{M}", grid, block, [_P(w), _P(x), _P(y), _I(R), _I(C_)], stream, shared)


def btb_gemv_silu_bf16(launcher, M, grid, block, w, gu, y, R, C_, *, stream=None, shared=0):
    launcher.launch(f"btb_gemv_silu_bf16_m{M}", grid, block, [_P(w), _P(gu), _P(y), _I(R), _I(C_)], stream, shared)


def btb_add_rmsnorm(launcher, grid, block, h, y, w, eps, x, H, centered, *, stream=None, shared=0):
    launcher.launch(
        "btb_add_rmsnorm", grid, block, [_P(h), _P(y), _P(w), _F(eps), _P(x), _I(H), _I(centered)], stream, shared
    )


def btb_silu_mul(launcher, grid, block, gu, m, T, I, *, stream=None, shared=0):
    launcher.launch("btb_silu_mul", grid, block, [_P(gu), _P(m), _I(T), _I(I)], stream, shared)


def btb_norm_rope_kv(launcher, D, grid, block, qkv, wq, wk, eps, cos_t, sin_t, n0p, depth, K, V, qo, T, Hq, Hk, hs,
                     rs, centered, *, stream=None, shared=0):  # fmt: skip
    launcher.launch(
        f"btb_norm_rope_kv_d{D}", grid, block,
        [_P(qkv), _P(wq), _P(wk), _F(eps), _P(cos_t), _P(sin_t), _P(n0p), _P(depth), _P(K), _P(V), _P(qo), _I(T),
         _I(Hq), _I(Hk), _I(hs), _I(rs), _I(centered)],
        stream, shared,
    )  # fmt: skip


def btb_norm_rope_kv_tbl(launcher, D, grid, block, qkv, wq, wk, eps, cos_t, sin_t, n0p, depth, K, V, qo, T, Hq, Hk,
                         hs, rs, centered, tbl, *, stream=None, shared=0):  # fmt: skip
    launcher.launch(
        f"btb_norm_rope_kv_tbl_d{D}", grid, block,
        [_P(qkv), _P(wq), _P(wk), _F(eps), _P(cos_t), _P(sin_t), _P(n0p), _P(depth), _P(K), _P(V), _P(qo), _I(T),
         _I(Hq), _I(Hk), _I(hs), _I(rs), _I(centered), _P(tbl)],
        stream, shared,
    )  # fmt: skip


def btb_attn_flash(launcher, D, grid, block, q, K, V, out, n0p, par, T, Hq, Hk, hs, rs, scale, part_m, part_l,
                   part_acc, cnt, win, tbl, *, stream=None, shared=0):  # fmt: skip
    launcher.launch(
        f"btb_attn_flash_d{D}", grid, block,
        [_P(q), _P(K), _P(V), _P(out), _P(n0p), _P(par), _I(T), _I(Hq), _I(Hk), _I(hs), _I(rs), _F(scale),
         _P(part_m), _P(part_l), _P(part_acc), _P(cnt), _I(win), _P(tbl)],
        stream, shared,
    )  # fmt: skip


def btb_norm_rope_kv_rows(launcher, D, grid, block, qkv, wq, wk, eps, cos_t, sin_t, rw, K, V, qo, T, Hq, Hk, hs, rs, centered, *,
                          stream=None, shared=0):  # fmt: skip
    launcher.launch(
        f"btb_norm_rope_kv_rows_d{D}", grid, block,
        [_P(qkv), _P(wq), _P(wk), _F(eps), _P(cos_t), _P(sin_t), _P(rw), _P(K), _P(V), _P(qo), _I(T), _I(Hq), _I(Hk), _I(hs),
         _I(rs), _I(centered)],
        stream, shared,
    )  # fmt: skip


def btb_attn_flash_rows(launcher, D, grid, block, q, K, V, out, rw, T, Hq, Hk, hs, rs, scale, part_m, part_l, part_acc, cnt,
                        win, *, stream=None, shared=0):  # fmt: skip
    launcher.launch(
        f"btb_attn_flash_rows_d{D}", grid, block,
        [_P(q), _P(K), _P(V), _P(out), _P(rw), _I(T), _I(Hq), _I(Hk), _I(hs), _I(rs), _F(scale), _P(part_m), _P(part_l),
         _P(part_acc), _P(cnt), _I(win)],
        stream, shared,
    )  # fmt: skip


def btb_publish(launcher, grid, block, n0, ids, out_tok, out_n0, out_ts, *, stream=None, shared=0):
    launcher.launch("btb_publish", grid, block, [_P(n0), _P(ids), _P(out_tok), _P(out_n0), _P(out_ts)], stream, shared)


def btb_sample_keys(launcher, grid, block, seed, pos, salt, keys, *, stream=None, shared=0):
    launcher.launch("btb_sample_keys", grid, block, [_P(seed), _P(pos), _I(salt), _P(keys)], stream, shared)


def btb_sample_max(launcher, grid, block, x, V, fp, gM, *, stream=None, shared=0):
    launcher.launch("btb_sample_max", grid, block, [_P(x), _I(V), _P(fp), _P(gM)], stream, shared)


def btb_sample_hist(launcher, grid, block, x, V, fp, level, mode, gM, gpre, gfloor, ghist, *, stream=None, shared=0):
    launcher.launch("btb_sample_hist", grid, block,
                    [_P(x), _I(V), _P(fp), _I(level), _I(mode), _P(gM), _P(gpre), _P(gfloor), _P(ghist)], stream, shared)  # fmt: skip


def btb_sample_bin(launcher, grid, block, level, mode, top_k, fp, ghist, gpre, gcarry, *, stream=None, shared=0):
    launcher.launch("btb_sample_bin", grid, block,
                    [_I(level), _I(mode), _I(top_k), _P(fp), _P(ghist), _P(gpre), _P(gcarry)], stream, shared)  # fmt: skip


def btb_sample_draw(launcher, grid, block, x, keys, V, fp, gM, gpreK, gpreP, gbest, *, stream=None, shared=0):
    launcher.launch("btb_sample_draw", grid, block,
                    [_P(x), _P(keys), _I(V), _P(fp), _P(gM), _P(gpreK), _P(gpreP), _P(gbest)], stream, shared)  # fmt: skip


def btb_sample_out(launcher, grid, block, gbest, out, R, *, stream=None, shared=0):
    launcher.launch("btb_sample_out", grid, block, [_P(gbest), _P(out), _I(R)], stream, shared)


def btb_sample_verify(launcher, grid, block, x, q, kids, hasq, keys, V, Vd, C_, top_k, fp, out, *, stream=None, shared=0):
    launcher.launch("btb_sample_verify", grid, block,
                    [_P(x), _P(q), _P(kids), _P(hasq), _P(keys), _I(V), _I(Vd), _I(C_), _I(top_k), _P(fp), _P(out)],
                    stream, shared)  # fmt: skip


def btb_gemv_mma_bf16(launcher, grid, block, w, x, y, R, C_, M, *, stream=None, shared=0):
    launcher.launch("btb_gemv_mma_bf16", grid, block, [_P(w), _P(x), _P(y), _I(R), _I(C_), _I(M)], stream, shared)


def btb_moe_route(launcher, grid, block, logits, ls, E, k, idx, w, hidx, hw, cnt, seq, hseq, *, stream=None, shared=0):
    launcher.launch("btb_moe_route", grid, block,
                    [_P(logits), _I(ls), _I(E), _I(k), _P(idx), _P(w), _P(hidx), _P(hw), _P(cnt), _P(seq), _P(hseq)],
                    stream, shared)  # fmt: skip


def btb_gemv_lane16_f32(launcher, M, grid, block, w, x, y, R, C_, *, stream=None, shared=0):
    launcher.launch(f"btb_gemv_lane16_f32_m{M}", grid, block, [_P(w), _P(x), _P(y), _I(R), _I(C_)], stream, shared)


def btb_gemv_lane16_mx4_f32(launcher, M, grid, block, blocks, scales, x, y, R, C_, *, stream=None, shared=0):
    launcher.launch(f"btb_gemv_lane16_mx4_f32_m{M}", grid, block,
                    [_P(blocks), _P(scales), _P(x), _P(y), _I(R), _I(C_)], stream, shared)  # fmt: skip


def btb_gemv_mma8_bf16(launcher, grid, block, w, x, y, R, C_, M, *, stream=None, shared=0):
    launcher.launch("btb_gemv_mma8_bf16", grid, block, [_P(w), _P(x), _P(y), _I(R), _I(C_), _I(M)], stream, shared)


def btb_gemv_mma_glu_silu(launcher, grid, block, w, x, m, I, C_, M, *, stream=None, shared=0):
    launcher.launch("btb_gemv_mma_glu_silu", grid, block, [_P(w), _P(x), _P(m), _I(I), _I(C_), _I(M)], stream, shared)
