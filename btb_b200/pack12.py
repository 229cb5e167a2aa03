"""pack12 (btb's 12-bit lossless bf16 store, btb/pack12.py:1-14 of btb) encoded ON THE CARD.

The kernels of this library read a pack12 tensor as its five parts (low bytes, packed 4-bit codes, the table of the 15
most frequent high bytes, the escapes' ascending indices and their high bytes) and widen it inside the GEMV. A caller
that holds the parts already - btb's loader reads them from a packed checkpoint, btb's own encoder writes them - hands
them to `engine.P12Matrix` as they are. `pack_bf16` is for a model that sits on the card as bf16 (the synthetic
configs): histogram, table, codes and the ordered escape list are made by the library's kernels
(`btb_b200_p12_hist/_table/_encode/_escapes`), byte-identical to the reference encoder's output, and nothing is
copied to the host but 256 counts and the escape total.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import capi
from .capi import call, ptr

MAX_ELEMENTS = 2**31 - 1  # escape indices are int32


def pack_bf16(t: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, bytes, torch.Tensor, torch.Tensor]:
    """(lo u8 [n], hi4 u8 [ceil(n / 2)], table 16 bytes, esc_idx i32 [n_esc], esc_val u8 [n_esc]) of a bf16 tensor, the
    tensors on the card; a tensor on the host is copied to the current device first"""
    if t.dtype != torch.bfloat16:
        raise capi.NativeDtypeError(f"pack12 packs bf16, got {t.dtype}")
    n = int(t.numel())
    if not 0 < n <= MAX_ELEMENTS:
        raise ValueError(f"{n} elements: a tensor packs 1 to {MAX_ELEMENTS}")
    if not t.is_cuda:
        t = t.cuda()
    src = t.contiguous()
    dev, s = src.device, capi.stream_ptr()
    hist = torch.empty(256, dtype=torch.int32, device=dev)
    call("btb_b200_p12_hist", ptr(src), n, ptr(hist), s)
    counts = (C.c_uint * 256)(*[int(v) & 0xFFFFFFFF for v in hist.tolist()])
    table = (C.c_ubyte * 16)()
    n_codes = C.c_int(0)
    call("btb_b200_p12_table", counts, table, C.byref(n_codes))
    tiles = int(capi.lib().btb_b200_p12_tiles(n))
    lo = torch.empty(n, dtype=torch.uint8, device=dev)
    hi4 = torch.empty((n + 1) // 2, dtype=torch.uint8, device=dev)
    off = torch.empty(tiles + 1, dtype=torch.int32, device=dev)
    call("btb_b200_p12_encode", ptr(src), n, table, n_codes.value, ptr(lo), ptr(hi4), ptr(off), s)
    n_esc = int(off[tiles].item())
    esc_idx = torch.empty(n_esc, dtype=torch.int32, device=dev)
    esc_val = torch.empty(n_esc, dtype=torch.uint8, device=dev)
    if n_esc:
        call("btb_b200_p12_escapes", ptr(src), n, table, n_codes.value, ptr(off), ptr(esc_idx), ptr(esc_val), s)
    return lo, hi4, bytes(table), esc_idx, esc_val
