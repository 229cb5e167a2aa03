// The decode GEMV family for sm_100a: y[m][r] = bf16(sum_c w[r][c] * x[m][c]), bf16 in, f32 accumulate.
//
// Arithmetic (what makes a row's bits): the reference's card order (native/cuda/btb_kernels.cu:83-142 of btb) - a
// row's K-sum is 32 independent f32 chains, chain l taking the 8-element chunks l, l+32, l+64, .. in order and a
// chunk's elements in index order, one fmaf each; the chains are folded by the butterfly xor 16, 8, 4, 2, 1 and the
// sum is rounded to bf16 once. Nothing here depends on M, R, the grid or the order the bytes arrive in, so row r of
// a 32-row verify pass is the one-row step's row r to the bit.
//
// Data movement (what makes it fast on B200): persistent CTAs, one per SM, each owning a contiguous range of rows.
// Every warp runs its own ring of shared-memory stages filled by the TMA unit's 1-D bulk copies
// (cp.async.bulk ... mbarrier::complete_tx) - one elected lane issues, the copy completes on the stage's mbarrier,
// the 32 lanes consume the stage with conflict-free 16-byte shared loads. A CTA keeps ring bytes (~100 KB) in
// flight whatever its register budget, which is what an 8 TB/s part needs (about 40 KB a SM by Little's law). The
// weight copies are issued BEFORE the grid-dependency wait, so under programmatic dependent launch the ring fills
// while the previous kernel of the step is still draining; x (the previous kernel's output) is staged into shared
// memory after the wait. Packed formats are widened to bf16 bit patterns in registers on the way from the stage to
// the FMA: no widened copy exists anywhere.
#include "common.cuh"
#include "btb_b200_internal.h"

B2_DEFINE_STATUS(gemv)

namespace {

// warps a CTA, a ring each: 8 or 16 (the tunable `warps`)

enum Fmt { F_BF16 = 0, F_P12 = 1 };
enum XMode { X_SMEM = 0, X_SMEM_SILU = 1, X_GLOBAL = 2, X_SMEM_NORM = 3 };

struct GemvArgs {
    const uint8_t* w;    // bf16: [R, C] bf16; p12: lo bytes [R*C]
    const uint8_t* hi4;  // p12: codes, two a byte
    const int32_t* esc_idx;
    const uint8_t* esc_val;
    const int32_t* esc_row;  // p12: [R+1] first escape at or past each row's start (a derived index)
    uint32_t table[4];       // p12: the 16 high bytes
    const bf16* x;           // [M, C], or gu [M, 2C] for the SwiGLU fold
    bf16* y;                 // [M, R]
    int R, C;
    int seg;     // elements a stage holds (a multiple of 256)
    int stages;  // ring depth
    int evict_first;
    // the residual + RMSNorm prologue (X_SMEM_NORM): x = rmsnorm(h_in + y) * w computed by every CTA on the way in,
    // h_out = h_in + y written by CTA 0 (h_in is never written here, so no CTA reads a half-updated row)
    const bf16* h_in;
    const bf16* y_add;   // null: no add
    const bf16* norm_w;
    bf16* h_out;         // null when y_add is null
    float eps;
    int centered;
    int T;               // live rows (rows T..M-1 of x are zeros)
};

// a stage's bytes for `n` elements of a row
template <int FMT>
__host__ __device__ constexpr int stage_bytes(int n) {
    return FMT == F_BF16 ? n * 2 : n + n / 2;
}

// the activation of the SwiGLU fold, native/cuda/btb_kernels.cu:159 of the reference: silu in f32 as torch computes it
__device__ __forceinline__ float act_silu(float g) { return g / (1.f + expf(-g)); }

// ---- pack12: eight weights of a chunk as four bf16 pairs ---------------------------------------------------------
// lo: the chunk's 8 low bytes (two words), codes: its 8 nibbles (one word, element e in nibble e). The table's 16
// high bytes sit in four registers; a code picks its byte with two byte-permutes (codes 0-7, 8-15) and a third that
// chooses between them by the code's top bit. Returns pairs p[k] = (elem 2k low half, elem 2k+1 high half).
__device__ __forceinline__ void p12_chunk(uint32_t lo0, uint32_t lo1, uint32_t codes, const uint32_t (&t)[4],
                                          uint32_t (&p)[4]) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t sel = (codes >> (16 * h)) & 0xffffu;  // four codes
        const uint32_t s7 = sel & 0x7777u;
        const uint32_t a = __byte_perm(t[0], t[1], s7);
        const uint32_t b = __byte_perm(t[2], t[3], s7);
        const uint32_t pick = 0x3210u | ((sel & 0x8888u) >> 1);
        const uint32_t hi = __byte_perm(a, b, pick);  // the four high bytes
        const uint32_t lo = h ? lo1 : lo0;
        p[2 * h] = __byte_perm(lo, hi, 0x5140u);      // lo0 hi0 lo1 hi1
        p[2 * h + 1] = __byte_perm(lo, hi, 0x7362u);  // lo2 hi2 lo3 hi3
    }
}

// an escaped element's high byte: the row's escapes are [e0, e1) of the ascending list; binary search for `gi`
__device__ __noinline__ uint32_t p12_escape(const int32_t* __restrict__ esc_idx, const uint8_t* __restrict__ esc_val,
                                            int e0, int e1, int gi) {
    int a = e0, b = e1;
    while (a < b) {
        const int mid = (a + b) >> 1;
        if (__ldg(esc_idx + mid) < gi) a = mid + 1;
        else b = mid;
    }
    return a < e1 ? (uint32_t)__ldg(esc_val + a) : 0u;  // never past the row's run, whatever the list holds
}

template <int M, int FMT, int XM, int NWT>
__global__ void __launch_bounds__(NWT * 32, 1) gemv_stream(const GemvArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int NT = NWT * 32;
    const int R = A.R, C = A.C, seg = A.seg, S = A.stages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nseg = (C + seg - 1) / seg;
    constexpr bool XS = XM != X_GLOBAL;

    // shared memory: [norm scratch][x: M*C bf16 when staged][rings: NWT * S stages][barriers: NWT * S]
    // (the norm prologue adds one f32 row of h and the 256 partial sums in front)
    const int nbytes = XM == X_SMEM_NORM ? ((C * 4 + 256 * 4 + 127) & ~127) : 0;
    const int xbytes = (XS ? ((M * C * 2 + 127) & ~127) : 0) + nbytes;
    const int sbytes = (stage_bytes<FMT>(seg) + 127) & ~127;
    bf16* xs = reinterpret_cast<bf16*>(smem + nbytes);
    uint8_t* ring = smem + xbytes + (size_t)warp * S * sbytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + xbytes + (size_t)NWT * S * sbytes) + warp * S;

    // this CTA's rows [r0, r0 + cnt): an even split, the remainder one extra row to the first CTAs
    const int base = R / gridDim.x, rem = R % gridDim.x;
    const int r0 = blockIdx.x * base + min((int)blockIdx.x, rem);
    const int cnt = base + ((int)blockIdx.x < rem ? 1 : 0);
    // this warp's rows: r0 + warp, + NWT, ..; its items are (row, segment) pairs in order
    const int my_rows = cnt > warp ? (cnt - warp + NWT - 1) / NWT : 0;
    const int n_items = my_rows * nseg;

    if (lane == 0) {
        for (int s = 0; s < S; ++s) mbar_init(smem_u32(bars + s), 1);
        mbar_fence_init();
    }
    __syncwarp();

    const uint64_t pol = A.evict_first ? l2_evict_first_policy() : 0;
    // the producer's cursor: the next item to copy (kept by every lane, issued by lane 0); no division on the way
    int p_row = r0 + warp, p_seg = 0, p_st = 0, issued = 0;
    auto issue_next = [&]() {
        const int c0 = p_seg * seg;
        const int n = min(seg, C - c0);
        if (lane == 0) {
            const uint32_t bar = smem_u32(bars + p_st);
            const uint32_t dst = smem_u32(ring + (size_t)p_st * sbytes);
            const size_t e0 = (size_t)p_row * C + c0;
            if (FMT == F_BF16) {
                mbar_expect_tx(bar, n * 2);
                if (A.evict_first) bulk_g2s_hint(dst, A.w + e0 * 2, n * 2, bar, pol);
                else bulk_g2s(dst, A.w + e0 * 2, n * 2, bar);
            } else {
                mbar_expect_tx(bar, n + n / 2);
                if (A.evict_first) {
                    bulk_g2s_hint(dst, A.w + e0, n, bar, pol);
                    bulk_g2s_hint(dst + seg, A.hi4 + e0 / 2, n / 2, bar, pol);
                } else {
                    bulk_g2s(dst, A.w + e0, n, bar);
                    bulk_g2s(dst + seg, A.hi4 + e0 / 2, n / 2, bar);
                }
            }
        }
        ++issued;
        if (++p_st == S) p_st = 0;
        if (++p_seg == nseg) {
            p_seg = 0;
            p_row += NWT;
        }
    };
    // fill the ring: weights do not depend on the grids before this one
    {
        const int first = min(S, n_items);
        for (int i = 0; i < first; ++i) issue_next();
    }

    pdl_launch_dependents();
    pdl_wait();  // x is the previous kernel's output

    if (XS) {
        if (XM == X_SMEM) {
            const uint4* src = reinterpret_cast<const uint4*>(A.x);
            uint4* dst = reinterpret_cast<uint4*>(xs);
            for (int i = threadIdx.x; i < M * C / 8; i += NT) dst[i] = __ldg(src + i);
        } else if (XM == X_SMEM_SILU) {
            // x[m][c] = bf16(bf16(silu(g)) * u), gu [M, 2C] gate then up: the values btb_silu_mul would have written;
            // eight elements a thread a trip (16-byte loads), elementwise so the order is free
            const int cv = C >> 3;
            for (int i = threadIdx.x; i < M * cv; i += NT) {
                const int m = i / cv, c8 = i - m * cv;
                const uint4 gv = __ldg(reinterpret_cast<const uint4*>(A.x + (size_t)m * 2 * C) + c8);
                const uint4 uv = __ldg(reinterpret_cast<const uint4*>(A.x + (size_t)m * 2 * C + C) + c8);
                const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
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
        } else {
            // residual + RMSNorm on the way in (the arithmetic of add_rmsnorm, native/cuda/btb_kernels.cu:365-393 of
            // the reference): hv = bf16(h + y); thread i of 256 sums hv^2 over i, i + 256, .. in order; the fixed
            // 256 -> 1 tree; x = bf16(hv * rsqrt(ss / H + eps) * w). Every CTA computes the same values; CTA 0
            // writes the new residual.
            float* hsm = reinterpret_cast<float*>(smem);
            float* red = hsm + C;
            const int cv = C >> 3, tid = threadIdx.x;
            for (int m = 0; m < M; ++m) {
                if (m >= A.T) {  // a padding row: zeros
                    for (int i = tid; i < cv; i += NT)
                        reinterpret_cast<uint4*>(xs + (size_t)m * C)[i] = make_uint4(0u, 0u, 0u, 0u);
                    continue;
                }
                for (int i = tid; i < cv; i += NT) {
                    const uint4 hv = __ldg(reinterpret_cast<const uint4*>(A.h_in + (size_t)m * C) + i);
                    uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w};
                    if (A.y_add != nullptr) {
                        const uint4 yv = __ldg(reinterpret_cast<const uint4*>(A.y_add + (size_t)m * C) + i);
                        const uint32_t yw[4] = {yv.x, yv.y, yv.z, yv.w};
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const __nv_bfloat162 pr =
                                __floats2bfloat162_rn(bf_lo(hw[k]) + bf_lo(yw[k]), bf_hi(hw[k]) + bf_hi(yw[k]));
                            hw[k] = *reinterpret_cast<const uint32_t*>(&pr);
                        }
                        if (blockIdx.x == 0)
                            reinterpret_cast<uint4*>(A.h_out + (size_t)m * C)[i] = make_uint4(hw[0], hw[1], hw[2], hw[3]);
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        hsm[i * 8 + 2 * k] = bf_lo(hw[k]);
                        hsm[i * 8 + 2 * k + 1] = bf_hi(hw[k]);
                    }
                }
                __syncthreads();
                if (tid < 256) {  // the reference's 256 strided partial sums, whatever the block's width
                    float ss = 0.f;
                    for (int i = tid; i < C; i += 256) ss = fmaf(hsm[i], hsm[i], ss);
                    red[tid] = ss;
                }
                __syncthreads();
                for (int st = 128; st > 0; st >>= 1) {
                    if (tid < st) red[tid] += red[tid + st];
                    __syncthreads();
                }
                const float rstd = rsqrtf(red[0] / (float)C + A.eps);
                for (int i = tid; i < C; i += NT) {
                    const float wv = bf2f(A.norm_w[i]);
                    xs[(size_t)m * C + i] = f2bf(hsm[i] * rstd * (A.centered ? 1.f + wv : wv));
                }
                __syncthreads();
            }
        }
        __syncthreads();
    }

    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    bool ok = true;
    // the consumer's cursor
    int c_row = r0 + warp, c_seg = 0, c_st = 0;
    uint32_t c_par = 0;
    int i = 0;
    for (; i < n_items; ++i) {
        if (!mbar_wait_bounded(smem_u32(bars + c_st), c_par)) {
            ok = false;
            break;
        }
        const int row = c_row;
        const int c0 = c_seg * seg;
        const int nch = min(seg, C - c0) >> 3;  // the segment's chunks; its first chunk is global chunk c0 / 8
        const uint8_t* stg = ring + (size_t)c_st * sbytes;
        int e0 = 0, e1 = 0;
        if (FMT == F_P12 && A.esc_row != nullptr) {
            e0 = __ldg(A.esc_row + row);
            e1 = __ldg(A.esc_row + row + 1);
        }
#pragma unroll 4
        for (int lc = lane; lc < nch; lc += 32) {
            uint32_t wp[4];
            if (FMT == F_BF16) {
                const uint4 wv = *reinterpret_cast<const uint4*>(stg + lc * 16);
                wp[0] = wv.x, wp[1] = wv.y, wp[2] = wv.z, wp[3] = wv.w;
            } else {
                const uint2 lo = *reinterpret_cast<const uint2*>(stg + lc * 8);
                const uint32_t codes = *reinterpret_cast<const uint32_t*>(stg + seg + lc * 4);
                p12_chunk(lo.x, lo.y, codes, A.table, wp);
                // a code of 15 is an escape: its high byte comes from the row's list
                const uint32_t f = codes & (codes >> 1) & (codes >> 2) & (codes >> 3) & 0x11111111u;
                if (f != 0u && e1 > e0) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        if ((f >> (4 * e)) & 1u) {
                            const int gi = (int)((size_t)row * C + c0 + lc * 8 + e);
                            const uint32_t hb = p12_escape(A.esc_idx, A.esc_val, e0, e1, gi);
                            const int sh = (e & 1) ? 24 : 8;
                            wp[e >> 1] = (wp[e >> 1] & ~(0xffu << sh)) | (hb << sh);
                        }
                    }
                }
            }
#pragma unroll
            for (int m = 0; m < M; ++m) {
                uint4 xv;
                if (XS) xv = *reinterpret_cast<const uint4*>(xs + (size_t)m * C + c0 + lc * 8);
                else xv = __ldg(reinterpret_cast<const uint4*>(A.x + (size_t)m * C + c0 + lc * 8));
                float a = acc[m];
                a = fmaf(bf_lo(wp[0]), bf_lo(xv.x), a);
                a = fmaf(bf_hi(wp[0]), bf_hi(xv.x), a);
                a = fmaf(bf_lo(wp[1]), bf_lo(xv.y), a);
                a = fmaf(bf_hi(wp[1]), bf_hi(xv.y), a);
                a = fmaf(bf_lo(wp[2]), bf_lo(xv.z), a);
                a = fmaf(bf_hi(wp[2]), bf_hi(xv.z), a);
                a = fmaf(bf_lo(wp[3]), bf_lo(xv.w), a);
                a = fmaf(bf_hi(wp[3]), bf_hi(xv.w), a);
                acc[m] = a;
            }
        }
        // the stage is free once every lane has read it (the warp barrier orders their shared loads before the
        // elected lane's copy, as a consumer's release orders them in any TMA pipeline): refill it with the next item
        __syncwarp();
        if (issued < n_items) issue_next();
        if (c_seg == nseg - 1) {
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const float s = warp_sum(acc[m]);
                if (lane == 0) A.y[(size_t)m * R + row] = f2bf(s);
                acc[m] = 0.f;
            }
            c_seg = 0;
            c_row += NWT;
        } else {
            ++c_seg;
        }
        if (++c_st == S) {
            c_st = 0;
            c_par ^= 1u;
        }
    }
    if (!ok) {
        // a copy never landed: say so, then let the copies still in flight land (bounded) before the CTA's shared
        // memory goes away
        if (lane == 0) b2_fail(B2_ERR_TIMEOUT);
        for (int j = i + 1; j < issued; ++j) {
            if (++c_st == S) {
                c_st = 0;
                c_par ^= 1u;
            }
            mbar_wait_bounded(smem_u32(bars + c_st), c_par);
        }
    }
}

// ---- host side -----------------------------------------------------------------------------------------------------

struct Plan {
    int grid, seg, stages, smem, nw;
    bool xs;
};

// ring geometry: split a row into equal segments of at most `max_seg_bytes`, each a multiple of 256 elements (so a
// lane's chunk l + 32 j of the row is chunk l + 32 j' of its segment), as many stages as the per-warp budget holds
template <int FMT>
Plan make_plan(int M, int R, int C, bool want_xs, bool norm = false) {
    const B2Tuning& t = b2_tuning();
    Plan p;
    // wide passes keep 8 warps (their accumulators fill the register file); the narrow ones take the tunable
    const int NW = (M <= 2 && t.warps == 16) ? 16 : 8;
    p.nw = NW;
    const int xbytes = ((M * C * 2 + 127) & ~127) + (norm ? ((C * 4 + 256 * 4 + 127) & ~127) : 0);
    p.xs = want_xs && (M * C * 2) <= t.x_smem_max;
    const int ring = t.ring_bytes;
    int per_warp = ring / NW;
    int max_seg_el = t.seg_bytes / (FMT == F_BF16 ? 2 : 1);  // elements
    max_seg_el = max(256, max_seg_el & ~255);
    int sb = 0;
    auto total = [&](int st) { return (p.xs ? xbytes : 0) + NW * st * sb + NW * st * 8; };
    for (;;) {
        const int nseg = (C + max_seg_el - 1) / max_seg_el;
        int seg = (C + nseg - 1) / nseg;
        seg = (seg + 255) & ~255;
        p.seg = seg;
        sb = (stage_bytes<FMT>(seg) + 127) & ~127;
        p.stages = max(2, min(8, per_warp / sb));
        while (p.stages > 2 && total(p.stages) > 224 * 1024) --p.stages;
        if (total(p.stages) <= 224 * 1024) break;
        if (max_seg_el > 256) {
            max_seg_el = max(256, (max_seg_el / 2) & ~255);  // two stages of this size do not fit: halve the segment
        } else if (p.xs) {
            p.xs = false;  // a very wide x gives its shared memory back to the ring
        } else {
            break;
        }
    }
    p.smem = total(p.stages);
    const int sms = b2_sm_count();
    p.grid = max(1, min(sms * t.ctas_per_sm, (R + 1) / 2));
    return p;
}

template <int M, int FMT, int XM, int NWT>
int launch_nw(const GemvArgs& a, const Plan& p, cudaStream_t stream) {
    auto kern = gemv_stream<M, FMT, XM, NWT>;
    static bool allowed[64];  // the opt-in past 48 KB of dynamic shared memory, once a device
    int rc = b2_allow_smem(reinterpret_cast<const void*>(kern), allowed);
    if (rc) return rc;
    return b2_launch(reinterpret_cast<const void*>(kern), dim3(p.grid), dim3(NWT * 32), p.smem, stream, a, 1);
}
template <int M, int FMT, int XM>
int launch_one(const GemvArgs& a, const Plan& p, cudaStream_t stream) {
    if (M <= 2 && p.nw == 16) return launch_nw<M, FMT, XM, (M <= 2 ? 16 : 8)>(a, p, stream);
    return launch_nw<M, FMT, XM, 8>(a, p, stream);
}

template <int FMT, int XM>
int launch_m(int M, const GemvArgs& a, const Plan& p, cudaStream_t s) {
    switch (M) {
        case 1: return launch_one<1, FMT, XM>(a, p, s);
        case 2: return launch_one<2, FMT, XM>(a, p, s);
        case 4: return launch_one<4, FMT, XM>(a, p, s);
        case 8: return launch_one<8, FMT, XM>(a, p, s);
        default: return B2_ERR_DOMAIN;
    }
}
template <int FMT>
int launch_m_global(int M, const GemvArgs& a, const Plan& p, cudaStream_t s) {
    switch (M) {
        case 1: return launch_one<1, FMT, X_GLOBAL>(a, p, s);
        case 2: return launch_one<2, FMT, X_GLOBAL>(a, p, s);
        case 4: return launch_one<4, FMT, X_GLOBAL>(a, p, s);
        case 8: return launch_one<8, FMT, X_GLOBAL>(a, p, s);
        case 16: return launch_one<16, FMT, X_GLOBAL>(a, p, s);
        case 32: return launch_one<32, FMT, X_GLOBAL>(a, p, s);
        default: return B2_ERR_DOMAIN;
    }
}

int check_dims(const void* w, const void* x, const void* y, int M, int R, int C) {
    if (w == nullptr || x == nullptr || y == nullptr) return B2_ERR_NULL;
    if (R <= 0 || C <= 0 || (C & 7) != 0) return B2_ERR_DOMAIN;
    if (M != 1 && M != 2 && M != 4 && M != 8 && M != 16 && M != 32) return B2_ERR_DOMAIN;
    if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(x) & 15)) return B2_ERR_DOMAIN;
    return B2_OK;
}

}  // namespace

// esc_row[r] = the first escape at or past row r's first element (r = 0..R): the CPU kernel's per-row cursor
// (native/src/gemv.rs:720-735 of btb) computed once when the weights are loaded
namespace {
struct P12RowsArgs {
    const int32_t* esc_idx;
    int32_t* esc_row;
    int n_esc, R, C;
};
__global__ void __launch_bounds__(256) p12_rows(const P12RowsArgs A) {
    const int r = blockIdx.x * 256 + threadIdx.x;
    if (r > A.R) return;
    const long long start = (long long)r * A.C;
    int a = 0, b = A.n_esc;
    while (a < b) {
        const int mid = (a + b) >> 1;
        if ((long long)A.esc_idx[mid] < start) a = mid + 1;
        else b = mid;
    }
    A.esc_row[r] = a;
}
}  // namespace

extern "C" int btb_b200_p12_rows(const void* esc_idx, int n_esc, int R, int C, void* esc_row, void* stream) {
    if (esc_row == nullptr || (n_esc > 0 && esc_idx == nullptr)) return B2_ERR_NULL;
    if (n_esc < 0 || R <= 0 || C <= 0) return B2_ERR_DOMAIN;
    P12RowsArgs a{static_cast<const int32_t*>(esc_idx), static_cast<int32_t*>(esc_row), n_esc, R, C};
    return b2_launch((const void*)p12_rows, dim3((R + 1 + 255) / 256), dim3(256), 0, static_cast<cudaStream_t>(stream),
                     a);
}

extern "C" int btb_b200_gemv_bf16(const void* w, const void* x, void* y, int M, int R, int C, void* stream) {
    int rc = check_dims(w, x, y, M, R, C);
    if (rc) return rc;
    GemvArgs a{};
    a.w = static_cast<const uint8_t*>(w);
    a.x = static_cast<const bf16*>(x);
    a.y = static_cast<bf16*>(y);
    a.R = R, a.C = C;
    Plan p = make_plan<F_BF16>(M, R, C, M <= 8);
    a.seg = p.seg, a.stages = p.stages, a.evict_first = b2_tuning().evict_first;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return p.xs ? launch_m<F_BF16, X_SMEM>(M, a, p, s) : launch_m_global<F_BF16>(M, a, p, s);
}

// x = rmsnorm(h_in + y) * w computed inside the GEMV (bf16 weights, or pack12 when hi4 is not null)
extern "C" int btb_b200_gemv_norm(const void* w, const void* hi4, const void* table, const void* esc_idx,
                                  const void* esc_val, const void* esc_row, const void* h_in, const void* y_add,
                                  const void* norm_w, float eps, int centered, void* h_out, void* y, int T, int M, int R,
                                  int C, void* stream) {
    int rc = check_dims(w, h_in, y, M, R, C);
    if (rc) return rc;
    if (norm_w == nullptr || (y_add != nullptr && h_out == nullptr)) return B2_ERR_NULL;
    if (T <= 0 || T > M || M > 8 || !(eps == eps) || h_out == h_in) return B2_ERR_DOMAIN;
    const bool p12 = hi4 != nullptr;
    if (p12 && (table == nullptr || (C & 31) != 0 || (reinterpret_cast<uintptr_t>(hi4) & 15))) return B2_ERR_DOMAIN;
    GemvArgs a{};
    a.w = static_cast<const uint8_t*>(w);
    a.hi4 = static_cast<const uint8_t*>(hi4);
    a.esc_idx = static_cast<const int32_t*>(esc_idx);
    a.esc_val = static_cast<const uint8_t*>(esc_val);
    a.esc_row = static_cast<const int32_t*>(esc_row);
    if (p12) memcpy(a.table, table, 16);
    a.y = static_cast<bf16*>(y);
    a.R = R, a.C = C;
    a.h_in = static_cast<const bf16*>(h_in), a.y_add = static_cast<const bf16*>(y_add);
    a.norm_w = static_cast<const bf16*>(norm_w), a.h_out = static_cast<bf16*>(h_out);
    a.eps = eps, a.centered = centered, a.T = T;
    Plan p = p12 ? make_plan<F_P12>(M, R, C, true, true) : make_plan<F_BF16>(M, R, C, true, true);
    if (!p.xs) return B2_ERR_DOMAIN;  // too wide to stage: the caller runs btb_b200_add_rmsnorm and the plain GEMV
    a.seg = p.seg, a.stages = p.stages, a.evict_first = b2_tuning().evict_first;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return p12 ? launch_m<F_P12, X_SMEM_NORM>(M, a, p, s) : launch_m<F_BF16, X_SMEM_NORM>(M, a, p, s);
}

extern "C" int btb_b200_gemv_silu_bf16(const void* w, const void* gu, void* y, int M, int R, int C, void* stream) {
    int rc = check_dims(w, gu, y, M, R, C);
    if (rc) return rc;
    GemvArgs a{};
    a.w = static_cast<const uint8_t*>(w);
    a.x = static_cast<const bf16*>(gu);
    a.y = static_cast<bf16*>(y);
    a.R = R, a.C = C;
    Plan p = make_plan<F_BF16>(M, R, C, true);
    // the fold stages the activated x in shared memory; a pass too wide for that takes btb_b200_silu_mul and the
    // plain GEMV (the same bits)
    if (!p.xs || M > 8) return B2_ERR_DOMAIN;
    a.seg = p.seg, a.stages = p.stages, a.evict_first = b2_tuning().evict_first;
    return launch_m<F_BF16, X_SMEM_SILU>(M, a, p, static_cast<cudaStream_t>(stream));
}

// the SwiGLU fold over pack12 weights
extern "C" int btb_b200_gemv_silu_p12(const void* lo, const void* hi4, const void* table, const void* esc_idx,
                                      const void* esc_val, const void* esc_row, const void* gu, void* y, int M, int R,
                                      int C, void* stream) {
    int rc = check_dims(lo, gu, y, M, R, C);
    if (rc) return rc;
    if (hi4 == nullptr || table == nullptr) return B2_ERR_NULL;
    if ((C & 31) != 0 || (reinterpret_cast<uintptr_t>(hi4) & 15)) return B2_ERR_DOMAIN;
    GemvArgs a{};
    a.w = static_cast<const uint8_t*>(lo);
    a.hi4 = static_cast<const uint8_t*>(hi4);
    a.esc_idx = static_cast<const int32_t*>(esc_idx);
    a.esc_val = static_cast<const uint8_t*>(esc_val);
    a.esc_row = static_cast<const int32_t*>(esc_row);
    if (a.esc_row != nullptr && (a.esc_idx == nullptr || a.esc_val == nullptr)) return B2_ERR_NULL;
    memcpy(a.table, table, 16);
    a.x = static_cast<const bf16*>(gu);
    a.y = static_cast<bf16*>(y);
    a.R = R, a.C = C;
    Plan p = make_plan<F_P12>(M, R, C, true);
    if (!p.xs || M > 8) return B2_ERR_DOMAIN;
    a.seg = p.seg, a.stages = p.stages, a.evict_first = b2_tuning().evict_first;
    return launch_m<F_P12, X_SMEM_SILU>(M, a, p, static_cast<cudaStream_t>(stream));
}

extern "C" int btb_b200_gemv_p12(const void* lo, const void* hi4, const void* table, const void* esc_idx,
                                 const void* esc_val, const void* esc_row, const void* x, void* y, int M, int R, int C,
                                 void* stream) {
    int rc = check_dims(lo, x, y, M, R, C);
    if (rc) return rc;
    if (hi4 == nullptr || table == nullptr) return B2_ERR_NULL;
    // a row's low bytes and codes are bulk-copied from their own offsets: both must start on 16 bytes
    if ((C & 31) != 0 || (reinterpret_cast<uintptr_t>(hi4) & 15)) return B2_ERR_DOMAIN;
    GemvArgs a{};
    a.w = static_cast<const uint8_t*>(lo);
    a.hi4 = static_cast<const uint8_t*>(hi4);
    a.esc_idx = static_cast<const int32_t*>(esc_idx);
    a.esc_val = static_cast<const uint8_t*>(esc_val);
    a.esc_row = static_cast<const int32_t*>(esc_row);
    if (a.esc_row != nullptr && (a.esc_idx == nullptr || a.esc_val == nullptr)) return B2_ERR_NULL;
    memcpy(a.table, table, 16);  // host pointer: the 16-byte table travels in the launch's arguments
    a.x = static_cast<const bf16*>(x);
    a.y = static_cast<bf16*>(y);
    a.R = R, a.C = C;
    Plan p = make_plan<F_P12>(M, R, C, M <= 8);
    a.seg = p.seg, a.stages = p.stages, a.evict_first = b2_tuning().evict_first;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return p.xs ? launch_m<F_P12, X_SMEM>(M, a, p, s) : launch_m_global<F_P12>(M, a, p, s);
}
