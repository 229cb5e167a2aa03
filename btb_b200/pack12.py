"""pack12, version 1: the 12-bit lossless bf16 store (btb/pack12.py:1-14 of btb), host side.

A bf16 tensor is a low byte per element and a 4-bit code per element into a table of the 15 most frequent high
bytes; code 15 marks an escape, listed by ascending element index with its high byte. ``pack_bf16`` returns the five
parts in the order the reference's encoder does (lo, hi4, table, esc_idx, esc_val) and packs to the same bytes: the
table lists high bytes by count descending, ties by value ascending. The kernels read these parts as stored
(``btb_b200_gemv_p12``); ``unpack_bf16`` is the host-side inverse used by tests.
"""

from __future__ import annotations

import numpy as np
import torch

ESC = 15
MAX_ELEMENTS = 2**31 - 1  # escape indices are int32


def pack_bf16(t: torch.Tensor) -> tuple[np.ndarray, np.ndarray, np.ndarray, np.ndarray, np.ndarray]:
    if t.dtype != torch.bfloat16:
        raise TypeError(f"pack12 packs bf16, got {t.dtype}")
    if t.numel() > MAX_ELEMENTS:
        raise ValueError(f"{t.numel()} elements: a tensor packs up to {MAX_ELEMENTS}")
    bits = t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16).reshape(-1)
    lo = (bits & 0xFF).astype(np.uint8)
    hi = (bits >> 8).astype(np.uint8)
    hist = np.bincount(hi, minlength=256)
    # by count descending, ties by value ascending: a stable sort of the negated counts over ascending values
    order = np.argsort(-hist, kind="stable")
    top = order[:ESC]
    top = top[hist[top] > 0]
    code_of = np.full(256, ESC, np.uint8)
    code_of[top] = np.arange(top.size, dtype=np.uint8)
    codes = code_of[hi]
    where = np.flatnonzero(codes == ESC)
    esc_idx, esc_val = where.astype(np.int32), hi[where]
    if codes.size & 1:
        codes = np.append(codes, np.uint8(0))
    hi4 = (codes[0::2] | (codes[1::2] << 4)).astype(np.uint8)
    table = np.zeros(16, np.uint8)
    table[: top.size] = top
    return lo, hi4, table, esc_idx, esc_val


def unpack_bf16(lo, hi4, table, esc_idx, esc_val, shape) -> torch.Tensor:
    lo = np.asarray(lo, np.uint8)
    n = lo.size
    h = np.asarray(hi4, np.uint8)
    codes = np.empty(h.size * 2, np.uint8)
    codes[0::2], codes[1::2] = h & 15, h >> 4
    hi = np.asarray(table, np.uint8)[codes[:n]].astype(np.uint16)
    if len(esc_idx):
        hi[np.asarray(esc_idx, np.int64)] = np.asarray(esc_val, np.uint16)
    bits = (hi << 8) | lo
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).reshape(tuple(shape))
