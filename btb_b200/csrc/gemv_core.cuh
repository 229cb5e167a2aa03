// The GEMV's arithmetic, shared by the standalone kernels (gemv.cu) and the whole-step kernel (step.cu): how x is
// built in shared memory (copy, SwiGLU, residual + RMSNorm) and how one ring stage of weights is multiplied into a
// warp's accumulators in the reference's chain order. Activations are read with L2-coherent loads (ld.global.cg):
// the whole-step kernel re-reads buffers that other SMs rewrote earlier in the same launch.
#pragma once

#include <cuda_fp8.h>

#include "common.cuh"
#include "tp.cuh"

enum Fmt { F_BF16 = 0, F_P12 = 1, F_FP8 = 2 };

// what a stage's widen needs beside the bytes: pack12's table and the row's escapes, FP8's scale row
struct WidenCtx {
    const int32_t* esc_idx;
    const uint8_t* esc_val;
    uint32_t table[4];
    int e0, e1;         // the row's escapes are [e0, e1) of the ascending list
    const float* srow;  // FP8: the row's scales, one per `bn` columns
    int bn;
};

__device__ __forceinline__ uint4 ldcg16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }

// a stage's bytes for `n` elements of a row
template <int FMT>
__host__ __device__ constexpr int stage_bytes(int n) {
    return FMT == F_BF16 ? n * 2 : (FMT == F_P12 ? n + n / 2 : n);
}

// e4m3fn byte -> f32 from its bits, times the block's scale, to the nearest bf16 (ties to even) by integer arithmetic:
// the value btb holds for an FP8 weight (native/src/gemv.rs:2996-3020, 3081; btb/fp8.py:97-100), as an f32
__device__ __forceinline__ float fp8_held(uint32_t b, float scale) {
    const uint32_t a = b & 0x7Fu;
    float mag;
    if (a == 0x7Fu) mag = __uint_as_float(0x7FC00000u);
    else if (a < 8u) mag = __fmul_rn((float)a, 1.0f / 512.0f);
    else mag = __uint_as_float((a << 20) + (120u << 23));
    const float v = __fmul_rn(__uint_as_float(__float_as_uint(mag) | ((b & 0x80u) << 24)), scale);
    const uint32_t u = __float_as_uint(v);
    return __uint_as_float((u + 0x7FFFu + ((u >> 16) & 1u)) & 0xFFFF0000u);
}

// two e4m3 bytes (the low 16 bits of `two`) the same way through the conversion unit: e4m3 -> f16 is exact, f16 -> f32 is
// exact, so the product and its rounding to bf16 (nearest, ties to even) are fp8_held's for every finite weight
__device__ __forceinline__ void fp8x2_held(uint32_t two, float scale, float& a, float& b) {
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(two & 0xffffu), __NV_E4M3);
    a = bfround(__fmul_rn(__half2float(__ushort_as_half(h.x)), scale));
    b = bfround(__fmul_rn(__half2float(__ushort_as_half(h.y)), scale));
}

// the activation of the SwiGLU fold, native/cuda/btb_kernels.cu:159 of the reference: silu in f32 as torch computes it
__device__ __forceinline__ float act_silu(float g) { return g / (1.f + expf(-g)); }

// the same, left as the packed bf16 pair (a in the low half): what the mixed-precision fma multiplies with
__device__ __forceinline__ uint32_t fp8x2_held_pair(uint32_t two, float scale) { return e4m3x2_held_pair(two, scale); }

// ---- pack12: eight weights of a chunk as four bf16 pairs ---------------------------------------------------------
// lo: the chunk's 8 low bytes (two words), codes: its 8 nibbles (one word, element e in nibble e). The table's 16
// high bytes sit in four registers; a code picks its byte with two byte-permutes (codes 0-7, 8-15) and a third that
// chooses between them by the code's top bit. Returns pairs p[k] = (elem 2k low half, elem 2k+1 high half).
__device__ __forceinline__ void p12_chunk(uint32_t lo0, uint32_t lo1, uint32_t codes, const uint32_t (&t)[4],
                                          uint32_t (&p)[4]) {
    // both halves' selectors at once (a byte permute reads only the low 16 bits of its selector: the second half's are
    // a shift away): the codes' low three bits pick within a table half, their top bits pick the half
    const uint32_t s7 = codes & 0x77777777u;
    const uint32_t pick = 0x32103210u | ((codes >> 1) & 0x44444444u);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t sel = h ? s7 >> 16 : s7, pk = h ? pick >> 16 : pick;
        const uint32_t a = __byte_perm(t[0], t[1], sel);
        const uint32_t b = __byte_perm(t[2], t[3], sel);
        const uint32_t hi = __byte_perm(a, b, pk);  // the four high bytes
        const uint32_t lo = h ? lo1 : lo0;
        p[2 * h] = __byte_perm(lo, hi, 0x5140u);      // lo0 hi0 lo1 hi1
        p[2 * h + 1] = __byte_perm(lo, hi, 0x7362u);  // lo2 hi2 lo3 hi3
    }
}

// an escaped element's high byte: the row's escapes are [e0, e1) of the ascending list; binary search for `gi`
static __device__ __noinline__ uint32_t p12_escape(const int32_t* __restrict__ esc_idx, const uint8_t* __restrict__ esc_val,
                                            int e0, int e1, int gi) {
    int a = e0, b = e1;
    while (a < b) {
        const int mid = (a + b) >> 1;
        if (__ldg(esc_idx + mid) < gi) a = mid + 1;
        else b = mid;
    }
    return a < e1 ? (uint32_t)__ldg(esc_val + a) : 0u;  // never past the row's run, whatever the list holds
}


// ---- x into shared memory ------------------------------------------------------------------------------------------

// x [M, C] bf16 as is; `marked`: x is this rank's copy of an exchanged vector (u32 words [M, C], tp.cuh), each element
// taken once it carries this hop's `mark`
// (only the pass's `live` rows are awaited - a producer may have none to send for the padding rows - the rest are zeros)
template <int M, int NT>
__device__ __forceinline__ void stage_x_copy(bf16* xs, const bf16* x, int C, bool marked = false, uint32_t mark = 0u,
                                             int live = M) {
    uint4* dst = reinterpret_cast<uint4*>(xs);
    const int nt = NT > 0 ? NT : (int)blockDim.x;  // NT 0: the block's width is a launch parameter
    if (marked) {
        const int n_live = live * (C / 8);
        for (int i = threadIdx.x; i < M * C / 8; i += nt)
            dst[i] = i < n_live ? b2_take8(reinterpret_cast<const uint32_t*>(x) + (size_t)i * 8, mark) : make_uint4(0u, 0u, 0u, 0u);
        return;
    }
    for (int i = threadIdx.x; i < M * C / 8; i += nt) dst[i] = ldcg16(reinterpret_cast<const uint4*>(x) + i);
}

// x[m][c] = bf16(bf16(silu(g)) * u), gu [M, 2C] gate then up: the values btb_silu_mul would have written
// (native/cuda/btb_kernels.cu:171-209 of the reference); eight elements a thread a trip, elementwise so the order is free
// U: trips whose loads are in flight together
template <int M, int NT, int U = 4>
__device__ __forceinline__ void stage_x_silu(bf16* xs, const bf16* gu, int C) {
    const int cv = C >> 3;
    const int nt = NT > 0 ? NT : (int)blockDim.x;
    for (int i0 = threadIdx.x; i0 < M * cv; i0 += U * nt) {
        uint4 gv[U], uv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * nt;
            if (i < M * cv) {
                const int m = i / cv, c8 = i - m * cv;
                gv[u] = ldcg16(reinterpret_cast<const uint4*>(gu + (size_t)m * 2 * C) + c8);
                uv[u] = ldcg16(reinterpret_cast<const uint4*>(gu + (size_t)m * 2 * C + C) + c8);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * nt;
            if (i < M * cv) {
                const int m = i / cv, c8 = i - m * cv;
                const uint32_t gw[4] = {gv[u].x, gv[u].y, gv[u].z, gv[u].w}, uw[4] = {uv[u].x, uv[u].y, uv[u].z, uv[u].w};
                uint32_t o[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float a = bfround(act_silu(bf_lo(gw[k]))) * bf_lo(uw[k]);
                    const float b = bfround(act_silu(bf_hi(gw[k]))) * bf_hi(uw[k]);
                    const __nv_bfloat162 pr = __floats2bfloat162_rn(a, b);
                    o[k] = *reinterpret_cast<const uint32_t*>(&pr);
                }
                reinterpret_cast<uint4*>(xs + (size_t)m * C)[c8] = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
    }
}

// residual + RMSNorm on the way in (the arithmetic of add_rmsnorm, native/cuda/btb_kernels.cu:365-393 of the
// reference): hv = bf16(h + y); thread i of 256 sums hv^2 over i, i + 256, .. in order; the fixed 256 -> 1 tree;
// x = bf16(hv * rsqrt(ss / H + eps) * w). Every CTA computes the same values; the one with `writer` set stores the
// new residual to h_out (never the buffer h_in points into). `rows`: when not null, row m of the input is
// h_in + rows[m] * C (an embedding table's row: the gather folded in). scratch: C + 256 floats.
template <int M, int NT, bool PRE = true>
__device__ __forceinline__ void stage_x_norm(bf16* xs, float* scratch, const bf16* h_in, const long long* rows,
                                             const bf16* y_add, const bf16* norm_w, bf16* h_out, float eps,
                                             int centered, int T, int C, bool writer, bool marked = false,
                                             uint32_t mark = 0u) {
    float* hsm = scratch;
    float* red = hsm + C;
    const int cv = C >> 3, tid = threadIdx.x;
    const int nt = NT > 0 ? NT : (int)blockDim.x;
    // the norm's weights are on their way before the first barrier (they do not depend on the row)
    // (PRE false: a caller short of registers reads them where they are used)
    constexpr int UW = PRE ? 4 : 1;
    uint4 wpre[UW];
#pragma unroll
    for (int u = 0; u < UW; ++u)
        if (PRE && tid + u * nt < cv) wpre[u] = __ldg(reinterpret_cast<const uint4*>(norm_w) + tid + u * nt);
    for (int m = 0; m < M; ++m) {
        if (m >= T) {  // a padding row: zeros
            for (int i = tid; i < cv; i += nt) reinterpret_cast<uint4*>(xs + (size_t)m * C)[i] = make_uint4(0u, 0u, 0u, 0u);
            continue;
        }
        const bf16* hrow = rows != nullptr ? h_in + (size_t)__ldcg(rows + m) * C : h_in + (size_t)m * C;
        for (int i = tid; i < cv; i += nt) {
            const uint4 hv = ldcg16(reinterpret_cast<const uint4*>(hrow) + i);
            uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w};
            if (y_add != nullptr) {
                // (in a model cut over ranks y_add is this rank's copy of an exchanged vector: words with marks)
                const uint4 yv = marked ? b2_take8(reinterpret_cast<const uint32_t*>(y_add) + (size_t)m * C + (size_t)i * 8, mark)
                                        : ldcg16(reinterpret_cast<const uint4*>(y_add + (size_t)m * C) + i);
                const uint32_t yw[4] = {yv.x, yv.y, yv.z, yv.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const __nv_bfloat162 pr =
                        __floats2bfloat162_rn(bf_lo(hw[k]) + bf_lo(yw[k]), bf_hi(hw[k]) + bf_hi(yw[k]));
                    hw[k] = *reinterpret_cast<const uint32_t*>(&pr);
                }
            }
            if (writer && h_out != nullptr)
                reinterpret_cast<uint4*>(h_out + (size_t)m * C)[i] = make_uint4(hw[0], hw[1], hw[2], hw[3]);
            reinterpret_cast<float4*>(hsm)[2 * i] = make_float4(bf_lo(hw[0]), bf_hi(hw[0]), bf_lo(hw[1]), bf_hi(hw[1]));
            reinterpret_cast<float4*>(hsm)[2 * i + 1] = make_float4(bf_lo(hw[2]), bf_hi(hw[2]), bf_lo(hw[3]), bf_hi(hw[3]));
        }
        __syncthreads();
        if (tid < 256) {  // the reference's 256 strided partial sums, whatever the block's width
            float ss = 0.f;
            for (int i = tid; i < C; i += 256) ss = fmaf(hsm[i], hsm[i], ss);
            red[tid] = ss;
        }
        __syncthreads();
        // the reference's tree red[t] += red[t + st], st = 128 .. 1, with the same pairs in the same order on one warp:
        // lane l holds red[l + 32 k]; st >= 32 pairs registers of one lane, st < 32 pairs lanes
        if (tid < 32) {
            float v[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = red[tid + 32 * k];
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] += v[k + 4];
            v[0] += v[2];
            v[1] += v[3];
            v[0] += v[1];
#pragma unroll
            for (int st = 16; st > 0; st >>= 1) v[0] += __shfl_down_sync(0xffffffffu, v[0], st);
            if (tid == 0) red[0] = v[0];
        }
        __syncthreads();
        const float rstd = rsqrtf(red[0] / (float)C + eps);
        for (int i = tid, u = 0; i < cv; i += nt, ++u) {
            uint4 wv4;
            switch (PRE ? u : 99) {  // a constant index keeps the prefetched vectors in registers
                case 0: wv4 = wpre[0]; break;
                case 1: wv4 = wpre[UW > 1 ? 1 : 0]; break;
                case 2: wv4 = wpre[UW > 2 ? 2 : 0]; break;
                case 3: wv4 = wpre[UW > 3 ? 3 : 0]; break;
                default: wv4 = __ldg(reinterpret_cast<const uint4*>(norm_w) + i); break;
            }
            const uint32_t ww[4] = {wv4.x, wv4.y, wv4.z, wv4.w};
            const float4 ha = reinterpret_cast<const float4*>(hsm)[2 * i], hb = reinterpret_cast<const float4*>(hsm)[2 * i + 1];
            const float hv8[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
            uint32_t o[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float w0 = bf_lo(ww[k]), w1 = bf_hi(ww[k]);
                const bf16 a = f2bf(hv8[2 * k] * rstd * (centered ? 1.f + w0 : w0));
                const bf16 b = f2bf(hv8[2 * k + 1] * rstd * (centered ? 1.f + w1 : w1));
                o[k] = (uint32_t)__bfloat16_as_ushort(a) | ((uint32_t)__bfloat16_as_ushort(b) << 16);
            }
            reinterpret_cast<uint4*>(xs + (size_t)m * C)[i] = make_uint4(o[0], o[1], o[2], o[3]);
        }
        __syncthreads();
    }
}

// ---- one ring stage into the accumulators --------------------------------------------------------------------------
// stg: the stage (bf16: the segment's weights; pack12: its low bytes, then at `seg` its codes); nch chunks of 8, the
// first global column c0 of `row`. Lane l takes local chunks l, l + 32, .. - segments are multiples of 256 columns,
// so these are the row's chunks l, l + 32, .. in order - and a chunk's elements in index order, one fmaf each.
// xv: x in shared memory [M, C] (XS) or in global memory (read-only path: the standalone kernels' wide passes only).
// ESC: the row has pack12 escapes (most rows have none: their loop carries no test for code 15 at all)
template <int M, int FMT, bool XS, bool ESC>
__device__ __forceinline__ void consume_stage_rows(float (&acc)[M], const uint8_t* stg, int seg, int nch, int c0, int row,
                                                   int C, const bf16* xv, const WidenCtx& W, int lane) {
#pragma unroll 4
    for (int lc = lane; lc < nch; lc += 32) {
        uint32_t wp[4];
        if (FMT == F_FP8) {
            const uint2 wb = *reinterpret_cast<const uint2*>(stg + lc * 8);
            const float sc = __ldg(W.srow + (c0 + lc * 8) / W.bn);
            wp[0] = fp8x2_held_pair(wb.x, sc);
            wp[1] = fp8x2_held_pair(wb.x >> 16, sc);
            wp[2] = fp8x2_held_pair(wb.y, sc);
            wp[3] = fp8x2_held_pair(wb.y >> 16, sc);
        } else {
            if (FMT == F_BF16) {
                const uint4 wv = *reinterpret_cast<const uint4*>(stg + lc * 16);
                wp[0] = wv.x, wp[1] = wv.y, wp[2] = wv.z, wp[3] = wv.w;
            } else {
                const uint2 lo = *reinterpret_cast<const uint2*>(stg + lc * 8);
                const uint32_t codes = *reinterpret_cast<const uint32_t*>(stg + seg + lc * 4);
                p12_chunk(lo.x, lo.y, codes, W.table, wp);
                // a code of 15 is an escape: its high byte comes from the row's list (most rows have none: the test for
                // code 15 is made only in rows that do)
                const uint32_t f = ESC && W.e1 > W.e0 ? codes & (codes >> 1) & (codes >> 2) & (codes >> 3) & 0x11111111u : 0u;
                if (ESC && f != 0u) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        if ((f >> (4 * e)) & 1u) {
                            const int gi = (int)((size_t)row * C + c0 + lc * 8 + e);
                            const uint32_t hb = p12_escape(W.esc_idx, W.esc_val, W.e0, W.e1, gi);
                            const int sh = (e & 1) ? 24 : 8;
                            wp[e >> 1] = (wp[e >> 1] & ~(0xffu << sh)) | (hb << sh);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
            uint4 x4;
            if (XS) x4 = *reinterpret_cast<const uint4*>(xv + (size_t)m * C + c0 + lc * 8);
            else x4 = __ldg(reinterpret_cast<const uint4*>(xv + (size_t)m * C + c0 + lc * 8));  // standalone wide passes
            // the weights as packed bf16 pairs: the chain's eight steps without a widening
            float a = acc[m];
            a = fma2_bf16(wp[0], x4.x, a);
            a = fma2_bf16(wp[1], x4.y, a);
            a = fma2_bf16(wp[2], x4.z, a);
            a = fma2_bf16(wp[3], x4.w, a);
            acc[m] = a;
        }
    }
}
template <int M, int FMT, bool XS>
__device__ __forceinline__ void consume_stage(float (&acc)[M], const uint8_t* stg, int seg, int nch, int c0, int row,
                                              int C, const bf16* xv, const WidenCtx& W, int lane) {
    // (wide passes keep one copy of the loop: their accumulators already fill the register file)
    if (FMT == F_P12 && (M > 8 || W.e1 > W.e0)) consume_stage_rows<M, FMT, XS, true>(acc, stg, seg, nch, c0, row, C, xv, W, lane);
    else consume_stage_rows<M, FMT, XS, M <= 8 ? false : true>(acc, stg, seg, nch, c0, row, C, xv, W, lane);
}
