// Stored expert weights to the f32 values btb multiplies with, one element at a time (the element-load kernel and the
// narrow instances of the streaming kernel; the wide instances widen several at once by byte permutes):
//   MXFP4 (btb/mxfp4.py:41, 113-124 of btb): an e2m1 code times 2^(s - 127), s the block's e8m0 byte;
//   FP8 (btb/fp8.py:36-46, 97-100): the e4m3fn value times the block's f32 scale, held as the nearest bf16.
#pragma once

#include <cuda_fp8.h>

#include "common.cuh"

// the sixteen e2m1 values, a lookup: 0, .5, 1, 1.5, 2, 3, 4, 6 and their negatives
__device__ __forceinline__ float fp4_to_f32(uint32_t code) {
    // the eight magnitudes as bf16 high halves, two a word; the sign is the code's top bit
    const uint32_t pair = (code & 6u) == 0u ? 0x3F000000u : (code & 6u) == 2u ? 0x3FC03F80u : (code & 6u) == 4u ? 0x40404000u : 0x40C04080u;
    const uint32_t half = (code & 1u) ? (pair >> 16) : (pair & 0xffffu);
    return __uint_as_float((half << 16) | ((code & 8u) << 28));
}
// an e8m0 scale byte as 2^(s - 127): the byte is the f32 exponent field; s = 0 is 2^-127, a subnormal f32 written out
__device__ __forceinline__ float e8m0_to_f32(uint32_t s) { return __uint_as_float(s != 0u ? s << 23 : 0x00400000u); }
// one e4m3fn byte through the conversion unit (e4m3 -> f16 and f16 -> f32 are exact), times the scale, to the nearest
// bf16 with ties to even
__device__ __forceinline__ float e4m3_held(uint32_t byte, float scale) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)byte, __NV_E4M3);
    return bfround(__fmul_rn(__half2float(__ushort_as_half(h.x)), scale));
}
