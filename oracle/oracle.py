"""TEST INFRASTRUCTURE - not a product path.

ctypes face of the CPU oracle (``btb_oracle.c``): numpy in, numpy out. bf16 tensors travel as ``uint16`` bit
patterns. Only the tests, the smoke entry and the benchmark's CPU-baseline leg may import this module; the shipped
package never does.
"""

from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libbtb_oracle.so")

_lib = None


def build(force: bool = False) -> str:
    """compile the oracle with the Makefile beside it (gcc only); returns the library's path"""
    src = os.path.join(HERE, "btb_oracle.c")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "CC=gcc", "libbtb_oracle.so"], check=True, capture_output=True)
    return LIB


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.btb_isa.restype = C.c_char_p
    return _lib


class OracleError(RuntimeError):
    pass


def _p(a: np.ndarray | None) -> C.c_void_p:
    if a is None:
        return C.c_void_p(0)
    assert a.flags["C_CONTIGUOUS"], "the oracle reads contiguous arrays"
    return C.c_void_p(a.ctypes.data)


def _ck(rc: int, what: str) -> None:
    if rc != 0:
        raise OracleError(f"{what}: rc {rc}")


def _u16(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    assert a.dtype == np.uint16, a.dtype
    return a


def isa() -> str:
    return lib().btb_isa().decode()


def force_scalar(on: bool) -> None:
    lib().orc_force_scalar(C.c_int(1 if on else 0))


# ---- bf16 helpers -------------------------------------------------------------------------------------------


def bf16_bits(t) -> np.ndarray:
    """a torch bf16 tensor's bit patterns as uint16"""
    import torch

    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def bits_bf16(a: np.ndarray):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16).copy()).view(torch.bfloat16)


def bits_to_f32(a: np.ndarray) -> np.ndarray:
    return (a.astype(np.uint32) << 16).view(np.float32)


def f32_to_bits(f: np.ndarray) -> np.ndarray:
    """round to nearest even, NaN canonical (the card's __float2bfloat16_rn)"""
    b = np.ascontiguousarray(f, dtype=np.float32).view(np.uint32)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)
    nan = (b & 0x7FFFFFFF) > 0x7F800000
    r[nan] = 0x7FFF
    return r


# ---- widens -------------------------------------------------------------------------------------------------


def pack_p12(bits16) -> tuple[np.ndarray, np.ndarray, np.ndarray, np.ndarray, np.ndarray]:
    """the reference's encoder (btb/pack12.py:48-68 `pack_bf16`) restated over bf16 bit patterns: (lo, hi4, table,
    esc_idx, esc_val). What the card's encoder is checked against where no reference-made fixture exists."""
    bits = np.ascontiguousarray(bits16, np.uint16).reshape(-1)
    lo, hi = (bits & 0xFF).astype(np.uint8), (bits >> 8).astype(np.uint8)
    hist = np.bincount(hi, minlength=256)
    top = np.argsort(-hist, kind="stable")[:15]  # count descending, byte value ascending among equals
    top = top[hist[top] > 0]
    code_of = np.full(256, 15, np.uint8)
    code_of[top] = np.arange(top.size, dtype=np.uint8)
    codes = code_of[hi]
    where = np.flatnonzero(codes == 15)
    if codes.size & 1:
        codes = np.append(codes, np.uint8(0))
    table = np.zeros(16, np.uint8)
    table[: top.size] = top
    return lo, (codes[0::2] | (codes[1::2] << 4)).astype(np.uint8), table, where.astype(np.int32), hi[where]


def widen_p12(lo, hi4, table, esc_idx, esc_val, n: int) -> np.ndarray:
    out = np.empty(n, np.uint16)
    esc_idx = np.ascontiguousarray(esc_idx, np.int32)
    esc_val = np.ascontiguousarray(esc_val, np.uint8)
    _ck(
        lib().orc_widen_p12(_p(lo), _p(hi4), _p(table), _p(esc_idx), _p(esc_val), C.c_size_t(esc_idx.size),
                            C.c_size_t(n), _p(out)),
        "orc_widen_p12",
    )  # fmt: skip
    return out


def widen_mxfp4(blocks, scales, rows: int, cols: int) -> np.ndarray:
    out = np.empty((rows, cols), np.float32)
    _ck(lib().orc_widen_mxfp4(_p(blocks), _p(scales), C.c_size_t(rows), C.c_size_t(cols), _p(out)), "orc_widen_mxfp4")
    return out


def widen_fp8(w, scales, rows: int, cols: int) -> np.ndarray:
    scales = np.ascontiguousarray(scales, np.float32)
    sr, sc = scales.shape
    out = np.empty((rows, cols), np.uint16)
    _ck(
        lib().orc_widen_fp8(_p(w), _p(scales), C.c_size_t(rows), C.c_size_t(cols), C.c_size_t(sr), C.c_size_t(sc),
                            _p(out)),
        "orc_widen_fp8",
    )  # fmt: skip
    return out


# ---- card-path arithmetic -----------------------------------------------------------------------------------


def gemv_card_bf16(w, x) -> np.ndarray:
    w, x = _u16(w), _u16(x)
    (R, Cc), M = w.shape, x.shape[0]
    y = np.empty((M, R), np.uint16)
    _ck(lib().orc_gemv_card_bf16(_p(w), _p(x), _p(y), M, R, Cc), "orc_gemv_card_bf16")
    return y


def gemv_card_silu_bf16(w, gu) -> np.ndarray:
    w, gu = _u16(w), _u16(gu)
    (R, Cc), M = w.shape, gu.shape[0]
    assert gu.shape[1] == 2 * Cc
    y = np.empty((M, R), np.uint16)
    _ck(lib().orc_gemv_card_silu_bf16(_p(w), _p(gu), _p(y), M, R, Cc), "orc_gemv_card_silu_bf16")
    return y


def gemv_card_p12(lo, hi4, table, esc_idx, esc_val, x, R: int, Cc: int) -> np.ndarray:
    x = _u16(x)
    M = x.shape[0]
    esc_idx = np.ascontiguousarray(esc_idx, np.int32)
    esc_val = np.ascontiguousarray(esc_val, np.uint8)
    y = np.empty((M, R), np.uint16)
    _ck(
        lib().orc_gemv_card_p12(_p(lo), _p(hi4), _p(table), _p(esc_idx), _p(esc_val), C.c_size_t(esc_idx.size),
                                _p(x), _p(y), M, R, Cc),
        "orc_gemv_card_p12",
    )  # fmt: skip
    return y


def gemv_card_fp8(w, scales, x, R: int, Cc: int) -> np.ndarray:
    x = _u16(x)
    scales = np.ascontiguousarray(scales, np.float32)
    M = x.shape[0]
    y = np.empty((M, R), np.uint16)
    _ck(
        lib().orc_gemv_card_fp8(_p(w), _p(scales), scales.shape[0], scales.shape[1], _p(x), _p(y), M, R, Cc),
        "orc_gemv_card_fp8",
    )
    return y


def gemv_card_mxfp4(blocks, scales, x, R: int, Cc: int) -> np.ndarray:
    x = _u16(x)
    M = x.shape[0]
    y = np.empty((M, R), np.uint16)
    _ck(lib().orc_gemv_card_mxfp4(_p(blocks), _p(scales), _p(x), _p(y), M, R, Cc), "orc_gemv_card_mxfp4")
    return y


def silu_mul(gu) -> np.ndarray:
    gu = _u16(gu)
    T, I2 = gu.shape
    m = np.empty((T, I2 // 2), np.uint16)
    _ck(lib().orc_silu_mul(_p(gu), _p(m), T, I2 // 2), "orc_silu_mul")
    return m


def add_rmsnorm(h, y, w, eps: float, centered: bool = False):
    """returns (h after the add, x); h is not modified in place"""
    h = _u16(h).copy()
    T, H = h.shape
    x = np.empty((T, H), np.uint16)
    yy = None if y is None else _u16(y)
    _ck(lib().orc_add_rmsnorm(_p(h), _p(yy), _p(_u16(w)), C.c_float(eps), _p(x), T, H, int(centered)), "orc_add_rmsnorm")
    return h, x


def norm_rope_kv(qkv, wq, wk, eps, cos_t, sin_t, n0, depth, K, V, Hq, Hk, D, hs, rs, centered=False, tbl=None):
    """writes K and V in place (uint16 arrays), returns q [T, Hq, D]"""
    qkv = _u16(qkv)
    T = qkv.shape[0]
    depth = np.ascontiguousarray(depth, np.int32)
    qo = np.empty((T, Hq, D), np.uint16)
    tb = None if tbl is None else np.ascontiguousarray(tbl, np.int32)
    _ck(
        lib().orc_norm_rope_kv(_p(qkv), _p(None if wq is None else _u16(wq)), _p(None if wk is None else _u16(wk)),
                               C.c_float(eps), _p(_u16(cos_t)), _p(_u16(sin_t)), int(n0), _p(depth), _p(K), _p(V),
                               _p(qo), T, Hq, Hk, D, C.c_long(hs), C.c_long(rs), int(centered), _p(tb)),
        "orc_norm_rope_kv",
    )  # fmt: skip
    return qo


def attn_decode(q, K, V, n0, par, Hq, Hk, D, hs, rs, scale, win=0, tbl=None, sinks=None) -> np.ndarray:
    q = _u16(q)
    T = q.shape[0]
    par = np.ascontiguousarray(par, np.int32)
    out = np.empty((T, Hq * D), np.uint16)
    tb = None if tbl is None else np.ascontiguousarray(tbl, np.int32)
    sk = None if sinks is None else np.ascontiguousarray(sinks, np.float32)
    _ck(
        lib().orc_attn_decode(_p(q), _p(K), _p(V), _p(out), int(n0), _p(par), T, Hq, Hk, D, C.c_long(hs),
                              C.c_long(rs), C.c_float(scale), int(win), _p(tb), _p(sk)),
        "orc_attn_decode",
    )  # fmt: skip
    return out


# ---- the rows layout (native/cuda/btb_kernels.cu:228-248 of btb): row t a sequence of its own --------------------------------
# rw = [base, step, W, then (col, off, len) a row]; row t's logical key j lives at cache row off + j for j < len (its
# prefix), else base + (j - len) * W + col (its own steps). Each row is restated as the one-sequence functions above over a
# row map built from its place: the reference's own statement of the layout ("the sequence a one-row step of that sequence
# alone walks", btb_kernels.cu:236-239).
def rows_map(rw, t: int) -> np.ndarray | None:
    """row t's logical -> cache row map over its len + step + 1 keys (None: padding)"""
    base, step, W = (int(v) for v in rw[:3])
    col, off, ln = (int(v) for v in rw[3 + 3 * t : 6 + 3 * t])
    if ln < 0:
        return None
    j = np.arange(ln + step + 1)
    return np.where(j < ln, off + j, base + (j - ln) * W + col).astype(np.int32)


def norm_rope_kv_rows(qkv, wq, wk, eps, cos_t, sin_t, rw, K, V, Hq, Hk, D, hs, rs, centered=False):
    """writes each live row's K and V at its step's cache row, returns q [T, Hq, D] (zeros for padding rows)"""
    qkv = _u16(qkv)
    T = qkv.shape[0]
    qo = np.zeros((T, Hq, D), np.uint16)
    for t in range(T):
        m = rows_map(rw, t)
        if m is None:
            continue
        pos = len(m) - 1
        qo[t] = norm_rope_kv(qkv[t : t + 1], wq, wk, eps, cos_t, sin_t, pos, [0], K, V, Hq, Hk, D, hs, rs, centered, m)[0]
    return qo


def attn_decode_rows(q, K, V, rw, Hq, Hk, D, hs, rs, scale, win=0, sinks=None) -> np.ndarray:
    q = _u16(q)
    T = q.shape[0]
    out = np.zeros((T, Hq * D), np.uint16)
    for t in range(T):
        m = rows_map(rw, t)
        if m is None:
            continue
        out[t] = attn_decode(q[t : t + 1], K, V, len(m) - 1, [-1], Hq, Hk, D, hs, rs, scale, win, m, sinks)[0]
    return out


def moe_route(logits, E: int, k: int, mode: int):
    """logits [T, ls]: uint16 (bf16 bits) or float32"""
    logits = np.ascontiguousarray(logits)
    f32 = logits.dtype == np.float32
    assert f32 or logits.dtype == np.uint16
    T, ls = logits.shape
    idx = np.empty((T, k), np.int32)
    w = np.empty((T, k), np.uint16)
    _ck(lib().orc_moe_route(_p(logits), ls, E, k, mode, int(f32), _p(idx), _p(w), T), "orc_moe_route")
    return idx, w


def bfround(f: np.ndarray) -> np.ndarray:
    """f32 values rounded to the nearest bf16 (ties to even), still as f32"""
    return bits_to_f32(f32_to_bits(np.asarray(f, np.float32)))


def moe_act(gu: np.ndarray, kind: int, bias=None, alpha: float = 1.702, limit: float = 7.0) -> np.ndarray:
    """the experts' middle (btb/engine/host.py:414-450): gu f32 [n, 2I] to the row dtype, the gated activation with
    every torch op's bf16 rounding, back to f32 [n, I]. kind 0: silu(gate) * up over halves; kind 1: gpt-oss"""
    gu = bfround(gu)
    if bias is not None:
        gu = bfround(gu + bits_to_f32(bias))
    I = gu.shape[1] // 2
    if kind == 0:
        g, u = gu[:, :I], gu[:, I:]
        with np.errstate(over="ignore"):
            act = bfround((g / (np.float32(1) + np.exp(-g, dtype=np.float32))).astype(np.float32))
        return bfround(act * u)
    g, u = gu[:, 0::2], gu[:, 1::2]
    g = np.minimum(g, np.float32(limit))
    u = np.clip(u, np.float32(-limit), np.float32(limit))
    t1 = bfround(g * np.float32(alpha))
    with np.errstate(over="ignore"):
        t2 = bfround((np.float32(1) / (np.float32(1) + np.exp(-t1, dtype=np.float32))).astype(np.float32))
    glu = bfround(g * t2)
    return bfround(bfround(u + np.float32(1)) * glu)


def moe_combine(dn: np.ndarray, idx: np.ndarray, w_bits: np.ndarray, bias=None) -> np.ndarray:
    """host.py:426-431,565-569: dn f32 [T, k, H]; out_e = bf16(dn_e) (+ bias) * w_e; the sum one bf16 add at a time in
    ascending expert id from zero. Returns bf16 bits [T, H]."""
    T, k, H = dn.shape
    y = np.zeros((T, H), np.float32)
    for t in range(T):
        for s in np.argsort(idx[t], kind="stable"):
            o = bfround(dn[t, s])
            if bias is not None:
                o = bfround(o + bits_to_f32(bias[idx[t, s]]))
            o = bfround(o * bits_to_f32(w_bits[t, s : s + 1]))
            y[t] = bfround(y[t] + o)
    return f32_to_bits(y)


def argmax_bf16(logits) -> np.ndarray:
    logits = _u16(logits)
    T, V = logits.shape
    out = np.empty(T, np.int64)
    _ck(lib().orc_argmax_bf16(_p(logits), T, V, _p(out)), "orc_argmax_bf16")
    return out


def sample_pick(x, keys, temperature: float, top_k: int = 0, top_p: float = 1.0):
    """(tokens [R], floors [R, 2] ordered bits, margin [R]) of the sampled pick over f32 logits [R, V]"""
    x = np.ascontiguousarray(x, np.float32)
    keys = np.ascontiguousarray(keys, np.uint64)
    R, V = x.shape
    out, floors, margin = np.empty(R, np.uint32), np.empty((R, 2), np.uint32), np.empty(R, np.float32)
    L = lib()
    L.orc_sample_pick.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_float, C.c_uint32, C.c_float,
                                  C.c_void_p, C.c_void_p, C.c_void_p]  # fmt: skip
    _ck(L.orc_sample_pick(_p(x), R, V, _p(keys), np.float32(1.0) / np.float32(temperature), int(top_k), float(top_p),
                          _p(out), _p(floors), _p(margin)), "orc_sample_pick")  # fmt: skip
    return out, floors, margin


def sample_verify(x, q, kids, hasq, keys, temperature: float, top_k: int = 0, top_p: float = 1.0) -> np.ndarray:
    """packed outcomes [R] ((accepted slot + 1) << 24 | token) of the verify pass's pick: x [R, V] f32 logits, q [R, Vd]
    the drafter's masses, kids [R, C] int32 (-1 after the last), hasq [R], keys [R]"""
    x = np.ascontiguousarray(x, np.float32)
    q = np.ascontiguousarray(q, np.float32)
    kids = np.ascontiguousarray(kids, np.int32)
    hasq = np.ascontiguousarray(hasq, np.uint32)
    keys = np.ascontiguousarray(keys, np.uint64)
    R, V = x.shape
    out = np.empty(R, np.uint32)
    L = lib()
    L.orc_sample_verify.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p,
                                    C.c_void_p, C.c_float, C.c_uint32, C.c_float, C.c_void_p]  # fmt: skip
    _ck(L.orc_sample_verify(_p(x), R, V, _p(q), q.shape[1], _p(kids), kids.shape[1], _p(hasq), _p(keys),
                            np.float32(1.0) / np.float32(temperature), int(top_k), float(top_p), _p(out)),
        "orc_sample_verify")  # fmt: skip
    return out


def sample_key(seed: int, pos: int, salt: int = 0) -> int:
    L = lib()
    L.orc_sample_key.restype, L.orc_sample_key.argtypes = C.c_uint64, [C.c_uint64, C.c_uint64, C.c_uint32]
    return int(L.orc_sample_key(seed, pos, salt))


def sample_uniform(key: int, idx) -> np.ndarray:
    L = lib()
    L.orc_sample_uniform.restype, L.orc_sample_uniform.argtypes = C.c_float, [C.c_uint64, C.c_uint32]
    return np.asarray([L.orc_sample_uniform(key, int(i)) for i in idx], np.float32)


def sample_exp(t) -> np.ndarray:
    L = lib()
    L.orc_sample_exp.restype, L.orc_sample_exp.argtypes = C.c_float, [C.c_float]
    return np.asarray([L.orc_sample_exp(float(v)) for v in t], np.float32)


# ---- CPU tier C-ABI -----------------------------------------------------------------------------------------


def cpu_gemv_bf16(w, x, threads: int = 0) -> np.ndarray:
    w = _u16(w)
    x = np.ascontiguousarray(x, np.float32)
    R, Cc = w.shape
    b = x.shape[0]
    y = np.empty((b, R), np.float32)
    _ck(lib().btb_gemv_bf16_rows(_p(w), C.c_size_t(R), C.c_size_t(Cc), _p(x), C.c_size_t(b), _p(y), C.c_size_t(threads)),
        "btb_gemv_bf16_rows")  # fmt: skip
    return y


def cpu_gemv_p12(lo, hi4, table, esc_idx, esc_val, R, Cc, x, threads: int = 0) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    esc_idx = np.ascontiguousarray(esc_idx, np.int32)
    esc_val = np.ascontiguousarray(esc_val, np.uint8)
    b = x.shape[0]
    y = np.empty((b, R), np.float32)
    _ck(
        lib().btb_gemv_p12_rows(_p(lo), _p(hi4), _p(table), _p(esc_idx), _p(esc_val), C.c_size_t(esc_idx.size),
                                C.c_size_t(R), C.c_size_t(Cc), _p(x), C.c_size_t(b), _p(y), C.c_size_t(threads)),
        "btb_gemv_p12_rows",
    )  # fmt: skip
    return y


def cpu_gemv_mxfp4(blocks, scales, R, Cc, x, threads: int = 0) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    b = x.shape[0]
    y = np.empty((b, R), np.float32)
    _ck(
        lib().btb_gemv_mxfp4_rows(_p(blocks), _p(scales), C.c_size_t(R), C.c_size_t(Cc), _p(x), C.c_size_t(b), _p(y),
                                  C.c_size_t(threads)),
        "btb_gemv_mxfp4_rows",
    )  # fmt: skip
    return y


def cpu_gemv_fp8(w, scales, R, Cc, x, threads: int = 0) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    scales = np.ascontiguousarray(scales, np.float32)
    b = x.shape[0]
    y = np.empty((b, R), np.float32)
    _ck(
        lib().btb_gemv_fp8_rows(_p(w), _p(scales), C.c_size_t(R), C.c_size_t(Cc), C.c_size_t(scales.shape[0]),
                                C.c_size_t(scales.shape[1]), _p(x), C.c_size_t(b), _p(y), C.c_size_t(threads)),
        "btb_gemv_fp8_rows",
    )  # fmt: skip
    return y


def cpu_attn_decode(q, k, v, scale: float) -> np.ndarray:
    """q [hq, d] f32; k, v [hk, n, d] uint16 (bf16 bits); returns [hq, d] f32"""
    q = np.ascontiguousarray(q, np.float32)
    k, v = _u16(k), _u16(v)
    hq, d = q.shape
    hk, n, _ = k.shape
    out = np.empty((hq, d), np.float32)
    _ck(
        lib().btb_attn_decode_bf16(_p(q), _p(k), _p(v), C.c_size_t(n), C.c_size_t(hq), C.c_size_t(hk), C.c_size_t(d),
                                   C.c_size_t(n * d), C.c_size_t(n * d), C.c_float(scale), _p(out), C.c_size_t(1)),
        "btb_attn_decode_bf16",
    )  # fmt: skip
    return out
