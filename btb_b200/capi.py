"""ctypes binding of ``libbtb_b200.so`` - the host side of the C-ABI in ``include/btb_b200.h``.

Mirrors the reference's FFI shim (btb/engine/native.py of btb): a nonzero return code raises ``NativeError(call, rc)``
(native.py:253-260), a tensor of the wrong dtype raises ``NativeDtypeError`` before the call. There is no CPU
fallback: if the CUDA library is missing or does not load, importing the binding's ``lib()`` raises.
"""

from __future__ import annotations

import ctypes as C
import os
from typing import Any

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libbtb_b200.so")

OK = 0
ERR_NULL, ERR_DOMAIN, ERR_CUDA, ERR_TIMEOUT = -1, -6, -10, -11
_NAMES = {ERR_NULL: "ERR_NULL", ERR_DOMAIN: "ERR_DOMAIN", ERR_CUDA: "ERR_CUDA", ERR_TIMEOUT: "ERR_TIMEOUT"}


class NativeError(RuntimeError):
    """a C-ABI call returned a negative code"""

    def __init__(self, call: str, rc: int):
        super().__init__(f"{call}: {_NAMES.get(rc, 'error')} ({rc})")
        self.call, self.rc = call, rc


class NativeDtypeError(TypeError):
    """a tensor handed to a kernel is not of the dtype the kernel reads"""


_P, _I, _F, _LL, _SZ = C.c_void_p, C.c_int, C.c_float, C.c_longlong, C.c_size_t

# every symbol include/btb_b200.h declares, with its argument types (the header is the contract; tests/test_capi.py
# checks the two agree)
SIGNATURES: dict[str, tuple[Any, list[Any]]] = {
    "btb_b200_version": (_I, []),
    "btb_b200_sm_count": (_I, []),
    "btb_b200_set_tuning": (_I, [C.c_char_p, _I]),
    "btb_b200_status": (_I, [C.POINTER(C.c_int)]),
    "btb_b200_gemv_bf16": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "btb_b200_gemv_tc_bf16": (_I, [_P, _P, _P, _I, _I, _I, _P, _P]),
    "btb_b200_gemv_tc_p12": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P, _P]),
    "btb_b200_gemv_tc_workspace_bytes": (_SZ, [_I, _I]),
    "btb_b200_gemm_tc_bf16": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "btb_b200_gemv_tc_glu_bf16": (_I, [_P, _P, _P, _I, _I, _I, _P, _P]),
    "btb_b200_gemv_tc_glu_workspace_bytes": (_SZ, [_I, _I]),
    "btb_b200_gemv_silu_bf16": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "btb_b200_gemv_p12": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P]),
    "btb_b200_gemv_fp8": (_I, [_P, _P, _I, _I, _P, _P, _I, _I, _I, _P]),
    "btb_b200_gemv_silu_p12": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P]),
    "btb_b200_gemv_norm": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _F, _I, _P, _P, _I, _I, _I, _I, _P]),
    "btb_b200_gemv_norm_fp8": (_I, [_P, _P, _I, _I, _P, _P, _P, _F, _I, _P, _P, _I, _I, _I, _I, _P]),
    "btb_b200_gemv_norm_swiglu": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _F, _I, _P, _P, _I, _I, _I, _I, _P]),
    "btb_b200_p12_rows": (_I, [_P, _I, _I, _I, _P, _P]),
    "btb_b200_p12_tiles": (_SZ, [_LL]),
    "btb_b200_p12_hist": (_I, [_P, _LL, _P, _P]),
    "btb_b200_p12_table": (_I, [C.POINTER(C.c_uint), C.POINTER(C.c_ubyte), C.POINTER(C.c_int)]),
    "btb_b200_p12_encode": (_I, [_P, _LL, C.POINTER(C.c_ubyte), _I, _P, _P, _P, _P]),
    "btb_b200_p12_escapes": (_I, [_P, _LL, C.POINTER(C.c_ubyte), _I, _P, _P, _P, _P]),
    "btb_b200_embed": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "btb_b200_add_rmsnorm": (_I, [_P, _P, _P, _F, _P, _I, _I, _I, _P]),
    "btb_b200_add_rmsnorm_wide": (_I, [_P, _P, _P, _F, _P, _P, _I, _I, _I, _P]),
    "btb_b200_silu_mul": (_I, [_P, _P, _I, _I, _P]),
    "btb_b200_norm_rope_kv": (_I, [_P, _P, _P, _F, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _LL, _LL, _I, _P, _I, _P]),
    "btb_b200_norm_rope_kv_rows": (_I, [_P, _P, _P, _F, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _LL, _LL, _I, _I, _P]),
    "btb_b200_attn_decode_rows": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _LL, _LL, _F, _P, _P, _P, _P, _I, _P, _I, _P]),
    "btb_b200_attn_decode": (
        _I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _LL, _LL, _F, _P, _P, _P, _P, _I, _P, _P, _I, _P],
    ),
    "btb_b200_attn_step": (
        _I, [_P, _P, _P, _F, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _LL, _LL, _I, _F, _P, _P, _P, _P, _I, _P, _P,
             _I, _P],
    ),
    "btb_b200_attn_step_batch": (
        _I, [_P, _P, _P, _F, _P, _P, _P, _P, _P, _P, _P, _P, _I, _LL, _I, _I, _I, _LL, _LL, _I, _F, _P, _P, _P, _P, _I,
             _P, _I, _P],
    ),
    "btb_b200_attn_o_step": (
        _I, [_P, _P, _P, _F, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _LL, _LL, _I, _F, _P, _P, _P, _P, _I, _P, _I,
             _P, _P, _I, _P, _P],
    ),
    "btb_b200_attn_scratch_floats": (_SZ, [_I, _I, _I, _I]),
    "btb_b200_argmax_bf16": (_I, [_P, _I, _I, _P, _P, _P]),
    "btb_b200_argmax_scratch_bytes": (_SZ, [_I]),
    "btb_b200_argmax_bf16_static": (_I, [_P, _I, _I, _P, _P]),
    "btb_b200_sample_pick": (_I, [_P, _I, _I, _I, _LL, _P, _I, _P, _P, _P, _P, C.c_uint, _P, _P, _P, _P]),
    "btb_b200_sample_out": (_I, [_P, _P, _I, _P]),
    "btb_b200_sample_verify": (_I, [_P, _I, _I, _I, _LL, _P, _I, _P, _I, _P, _P, _I, _P, _P, _P]),
    "btb_b200_sample_keys": (_I, [_P, _P, C.c_uint, _P, _P]),
    "btb_b200_kv_commit": (_I, [_P, _P, _LL, _I, _P, _P, _I, _I, _LL, _P, _I, _P]),
    "btb_b200_publish": (_I, [_P, _P, _P, _P, _P, _I, _P]),
    "btb_b200_moe_route": (_I, [_P, _I, _I, _I, _I, _I, _P, _P, _I, _P]),
    "btb_b200_moe_router": (_I, [_P, _P, _P, _I, _I, _I, _I, _P, _P, _I, _P]),
    "btb_b200_moe_router_grid": (_I, [_P, _P, _P, _P, _F, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P, _I, _P]),
    "btb_b200_moe_router_norm": (_I, [_P, _P, _P, _P, _F, _I, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P, _I, _P]),
    "btb_b200_gemv_lane16_f32": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "btb_b200_gemv_lane16_mx4_f32": (_I, [_P, _P, _P, _P, _I, _I, _I, _P]),
    "btb_b200_gemv_lane16_fp8_f32": (_I, [_P, _P, _I, _I, _P, _P, _I, _I, _I, _P]),
    "btb_b200_moe_gemv": (_I, [_I, _P, _P, _LL, _LL, _I, _I, _P, _I, _I, _P, _I, _P, _I, _I, _I, _I, _P]),
    "btb_b200_moe_gemv_act": (
        _I, [_I, _P, _P, _LL, _LL, _I, _I, _P, _I, _I, _P, _I, _F, _F, _P, _I, _I, _I, _I, _P],
    ),
    "btb_b200_moe_gemv_glu": (_I, [_I, _P, _P, _LL, _LL, _I, _I, _P, _I, _I, _P, _I, _P, _I, _I, _I, _F, _F, _I, _I, _P]),
    "btb_b200_moe_combine_norm": (_I, [_P, _P, _P, _I, _P, _P, _F, _P, _P, _P, _I, _I, _I, _P]),
    "btb_b200_moe_act": (_I, [_P, _P, _P, _P, _I, _I, _I, _F, _F, _P]),
    "btb_b200_moe_combine": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _P]),
    "btb_b200_widen_f32": (_I, [_P, _P, _I, _P]),
    "btb_b200_ngram_new": (_P, [_I, _I, _I]),
    "btb_b200_ngram_free": (None, [_P]),
    "btb_b200_ngram_extend": (_I, [_P, C.POINTER(C.c_longlong), _I]),
    "btb_b200_ngram_length": (_I, [_P]),
    "btb_b200_ngram_chains": (_I, [_P, _I, _I, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int),
                                   C.POINTER(C.c_int)]),
    "btb_b200_chains_tree": (_I, [C.POINTER(C.c_int), C.POINTER(C.c_int), _I, _I, C.POINTER(C.c_int), C.POINTER(C.c_int),
                                  C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "btb_b200_ngram_tree": (_I, [_P, _I, _I, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int),
                                 C.POINTER(C.c_int)]),
    "btb_b200_tree_walk": (_I, [C.POINTER(C.c_longlong), C.POINTER(C.c_int), C.POINTER(C.c_int), _I, C.POINTER(C.c_int),
                                C.POINTER(C.c_int)]),
    "btb_b200_step": (_I, [_P, _I, _I, _I, _P]),
    "btb_b200_step_op_bytes": (_SZ, []),
    "btb_b200_step_args_bytes": (_SZ, []),
}  # fmt: skip



class Recv(C.Structure):
    """`btb_b200_recv` of the header: how a consumer knows a word of its hop"""

    _fields_ = [("pass_", C.c_void_p), ("per_pass", C.c_uint), ("base", C.c_uint)]


class Send(C.Structure):
    """`btb_b200_send` of the header: every rank's copy of a vector and the hop's number"""

    _fields_ = [("out", C.c_void_p * 8), ("n", C.c_int), ("stride", C.c_int), ("offset", C.c_int), ("pass_", C.c_void_p),
                ("per_pass", C.c_uint), ("base", C.c_uint)]  # fmt: skip


_RP, _SP = C.POINTER(Recv), C.POINTER(Send)
SIGNATURES.update({
    "btb_b200_peer_alloc": (_I, [_SZ, C.POINTER(C.c_void_p)]),
    "btb_b200_peer_free": (_I, [_P]),
    "btb_b200_peer_handle": (_I, [_P, C.POINTER(C.c_ubyte)]),
    "btb_b200_peer_open": (_I, [C.POINTER(C.c_ubyte), C.POINTER(C.c_void_p)]),
    "btb_b200_peer_close": (_I, [_P]),
    "btb_b200_gemv_bf16_x": (_I, [_P, _P, _P, _I, _I, _I, _I, _RP, _SP, _P]),
    "btb_b200_gemv_norm_x": (_I, [_P, _P, _P, _P, _F, _I, _P, _P, _I, _I, _I, _I, _I, _RP, _SP, _P]),
    "btb_b200_attn_step_x": (
        _I, [_P, _P, _P, _F, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _LL, _LL, _I, _F, _P, _P, _P, _P, _I, _P, _P, _I, _SP,
             _P],
    ),
    "btb_b200_attn_step_w": (
        _I, [_P, _P, _P, _F, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _LL, _LL, _I, _F, _P, _P, _P, _P, _I, _P, _P, _I, _SP,
             _P, _LL, _P, _LL, _P],
    ),
    "btb_b200_attn_decode_x": (
        _I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _LL, _LL, _F, _P, _P, _P, _P, _I, _P, _P, _I, _SP, _P],
    ),
    "btb_b200_xchg_send": (_I, [_P, _I, _I, _SP, _P]),
    "btb_b200_xchg_unpack": (_I, [_P, _P, _I, _I, _RP, _P]),
    "btb_b200_xchg_pick": (_I, [_P, _I, _I, _I, _P, _I, _I, C.POINTER(C.c_void_p), _P, _P, _P, _I, _P]),
    "btb_b200_xchg_tick": (_I, [_P, _P]),
    "btb_b200_moe_gemv_x": (_I, [_I, _P, _P, _LL, _LL, _I, _I, _P, _I, _I, _P, _I, _I, _I, _I, _I, _SP, _P]),
    "btb_b200_moe_combine_x": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _RP, _P]),
})  # fmt: skip

_lib: C.CDLL | None = None


def lib() -> C.CDLL:
    """the loaded library, its functions typed; raises if it is not built (``python -m btb_b200.build``)"""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is not built: run `python -m btb_b200.build` (needs nvcc); no fallback exists")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name, None)
            if fn is None:
                continue  # declared here, not yet in this build: calling it raises AttributeError at the call site
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def ptr(t: Any) -> int:
    """a torch tensor's device address, None the null pointer (btb/engine/card_launch.py:443-446 `ptr`)"""
    return 0 if t is None else int(t.data_ptr())


def stream_ptr(stream: Any = None) -> int:
    """the cudaStream_t to enqueue on: the given torch stream, else torch's current stream"""
    import torch

    s = torch.cuda.current_stream() if stream is None else stream
    return int(s.cuda_stream)


def call(name: str, *args: Any) -> None:
    rc = getattr(lib(), name)(*args)
    if rc != 0:
        raise NativeError(name, int(rc))


def need(t: Any, dtype: Any, what: str) -> None:
    if t is not None and t.dtype != dtype:
        raise NativeDtypeError(f"{what}: {t.dtype}, the kernel reads {dtype}")


def status() -> int:
    """the device status word (0 = nothing refused); clears it"""
    v = C.c_int(0)
    call("btb_b200_status", C.byref(v))
    return int(v.value)


def set_tuning(**kw: int) -> None:
    for k, v in kw.items():
        call("btb_b200_set_tuning", k.encode(), int(v))
