// The picked experts' matvecs as one streaming launch: stored-format expert rows (bf16, MXFP4 blocks, FP8 with block
// scales) pulled through shared memory by TMA bulk copies and multiplied in the CPU tier's order.
//
// The order is btb's host kernels' (native/src/gemv.rs:46-58, 85-123; the on-card twins btb_gemv_lane16{,_mx4}_f32,
// native/cuda/btb_kernels.cu:1635-1766): column c of a row belongs to chain c mod 16, a chain takes its columns in
// increasing order with one fmaf each, and the sixteen sums fold pairwise (1, 2, 4, 8 apart). A chain is sequential,
// so a row offers sixteen-way parallelism and no more. Here four threads share a row, each running four adjacent
// chains: a warp takes eight rows at a time, a thread reads its four consecutive weights of every sixteen columns
// from shared memory as one word, and the fold is two adds in the thread and two shuffles. The rows arrive by one
// bulk copy a row segment into a per-warp ring (rows padded by 16 bytes, so the eight rows' words fall in distinct
// banks); x is staged once a CTA as f32. Every weight byte is read from DRAM once, in large transfers - the
// per-column byte loads of the plain 16-lane kernel ran at a twentieth of the memory's rate.
#include <cuda_fp8.h>

#include "btb_b200_internal.h"

B2_DEFINE_STATUS(moes)

namespace {

enum { S_BF16 = 0, S_MX4 = 1, S_FP8 = 2 };
constexpr int RB = 8;       // rows a warp takes at a time
constexpr int PAD = 16;     // bytes between the rows of a stage
constexpr int MAXW = 16;    // warps a CTA at most

struct MSArgs {
    const uint8_t* w;       // expert 0's weights
    const uint8_t* scales;  // MX4: e8m0 bytes [R, C/32]; FP8: f32 grid [sr, sc]
    long long w_stride, s_stride;  // bytes from an expert to the next
    const int* idx;         // [n_tasks] the task's expert, or null (expert 0 for all)
    const float* x;         // [rows_x, C] f32
    int x_div;              // task i reads x row i / x_div
    float* y;               // [n_tasks, R] f32
    int R, C, sr, sc, E;
    int ep_rank, ep_size;
    int seg;                // columns a stage holds of each row (a multiple of 32)
    int stages;
};

template <int FMT>
__host__ __device__ constexpr int col_bytes2() { return FMT == S_BF16 ? 4 : FMT == S_FP8 ? 2 : 1; }  // twice a column's bytes

__device__ __forceinline__ float mx4_scale_s(unsigned s) {
    const float f = __uint_as_float((s == 0u ? 1u : s) << 23);
    return s == 0u ? __fmul_rn(f, 0.5f) : f;
}
__device__ __forceinline__ float fp4_value_s(unsigned code) {
    const unsigned m = code & 7u;
    const unsigned mag = m >= 2u ? ((((m >> 1) + 126u) << 7) | ((m & 1u) << 6)) : (m ? 0x3F00u : 0u);
    return __uint_as_float((mag | ((code & 8u) << 12)) << 16);
}

template <int FMT>
__global__ void __launch_bounds__(MAXW * 32, 1) moe_gemv_stream(const MSArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int ri = lane >> 2, q = lane & 3;  // the thread's row of the warp's eight, its four chains 4q .. 4q + 3
    const int task = blockIdx.y;
    const int R = A.R, C = A.C, seg = A.seg, S = A.stages;
    constexpr int CB2 = col_bytes2<FMT>();
    const int row_bytes = C * CB2 / 2;
    const int stride = seg * CB2 / 2 + PAD;  // a stage row
    const int sbytes = RB * stride;
    const int nseg = (C + seg - 1) / seg;
    float* xs = reinterpret_cast<float*>(smem);
    const int xbytes = (C * 4 + 127) & ~127;
    uint8_t* ring = smem + xbytes + (size_t)warp * S * sbytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + xbytes + (size_t)nw * S * sbytes) + warp * S;

    if (lane == 0) {
        for (int s = 0; s < S; ++s) mbar_init(smem_u32(bars + s), 1);
        mbar_fence_init();
    }
    __syncwarp();
    pdl_launch_dependents();
    pdl_wait();  // the picks and x are the kernels' before this one

    int e = 0;
    if (A.idx != nullptr) {
        e = __ldcg(A.idx + task);
        if (e < 0 || e >= A.E) {  // never read outside the experts: record and skip
            if (threadIdx.x == 0 && blockIdx.x == 0) b2_fail(B2_ERR_DOMAIN);
            e = -1;
        }
    }
    bool mine = e >= 0;
    if (mine && A.ep_size > 1) {
        mine = e % A.ep_size == A.ep_rank;
        e = e / A.ep_size;
    }
    // this CTA's groups of eight rows: an even split of the task's groups over the CTAs that share it
    const int groups = (R + RB - 1) / RB;
    const int base = groups / gridDim.x, rem = groups % gridDim.x;
    const int g0 = blockIdx.x * base + min((int)blockIdx.x, rem);
    const int gc = base + ((int)blockIdx.x < rem ? 1 : 0);
    const int my_groups = gc > warp ? (gc - warp + nw - 1) / nw : 0;
    if (!mine) {  // another rank's expert (or a refused pick): zeros, so that the ranks' sum is the whole
        for (int g = g0 + warp; g < g0 + gc; g += nw) {
            const int r = g * RB + ri;
            if (r < R && q == 0) A.y[(size_t)task * R + r] = 0.f;
        }
        return;
    }
    const uint8_t* wbase = A.w + (size_t)e * A.w_stride;
    const uint64_t pol = l2_evict_first_policy();
    const int n_items = my_groups * nseg;
    int p_grp = g0 + warp, p_seg = 0, p_st = 0, issued = 0;
    auto issue_next = [&]() {
        const int c0 = p_seg * seg;
        const int n = min(seg, C - c0);
        const int rows = min(RB, R - p_grp * RB);
        const uint32_t nb = (uint32_t)(n * CB2 / 2);
        const uint32_t bar = smem_u32(bars + p_st);
        if (lane == 0) mbar_expect_tx(bar, nb * rows);
        __syncwarp();
        if (lane < rows) {
            const uint8_t* src = wbase + (size_t)(p_grp * RB + lane) * row_bytes + (size_t)c0 * CB2 / 2;
            bulk_g2s_hint(smem_u32(ring + (size_t)p_st * sbytes + (size_t)lane * stride), src, nb, bar, pol);
        }
        ++issued;
        if (++p_st == S) p_st = 0;
        if (++p_seg == nseg) {
            p_seg = 0;
            p_grp += nw;
        }
    };
    {
        const int first = min(S, n_items);
        for (int i = 0; i < first; ++i) issue_next();
    }
    // x as f32 in shared memory, once a CTA
    {
        const float4* xg = reinterpret_cast<const float4*>(A.x + (size_t)(task / A.x_div) * C);
        for (int i = threadIdx.x; i < C / 4; i += blockDim.x) reinterpret_cast<float4*>(xs)[i] = __ldcg(xg + i);
    }
    __syncthreads();

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    int c_grp = g0 + warp, c_seg = 0, c_st = 0;
    uint32_t c_par = 0;
    bool ok = true;
    int i = 0;
    for (; i < n_items; ++i) {
        const int r = c_grp * RB + ri;
        const bool live = r < R;
        const int c0 = c_seg * seg;
        const int n = min(seg, C - c0);
        // the stage's scales are on their way while the weights land
        float fsc[4] = {1.f, 1.f, 1.f, 1.f};
        unsigned mxs = 0u;
        if (FMT == S_FP8) {
            const int bm = R / A.sr, bn = C / A.sc;
            const float* srow = reinterpret_cast<const float*>(A.scales + (size_t)e * A.s_stride) + (size_t)((live ? r : 0) / bm) * A.sc;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int cb = (c0 + u * 128) / bn;
                fsc[u] = cb < A.sc ? __ldg(srow + cb) : 1.f;
            }
        } else if (FMT == S_MX4) {
            // a row's scale bytes of this stage (one a block of 32 columns): four a thread, shared by shuffle below
            const uint8_t* sr = A.scales + (size_t)e * A.s_stride + (size_t)(live ? r : 0) * (C >> 5) + (c0 >> 5);
            const int nb = n >> 5;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int b = q * 4 + u;
                mxs |= (b < nb ? (unsigned)__ldg(sr + b) : 127u) << (8 * u);
            }
        }
        if (!mbar_wait_bounded(smem_u32(bars + c_st), c_par)) {
            ok = false;
            break;
        }
        const uint8_t* srowp = ring + (size_t)c_st * sbytes + (size_t)ri * stride;
        const float* xp = xs + c0;
        if (FMT == S_FP8) {
            const int bn = C / A.sc;
            const int steps = n >> 4;
#pragma unroll 4
            for (int s = 0; s < steps; ++s) {
                const uint32_t wb = *reinterpret_cast<const uint32_t*>(srowp + s * 16 + q * 4);
                const float4 xv = *reinterpret_cast<const float4*>(xp + s * 16 + q * 4);
                // the block scale of these columns: the stage starts on a multiple of 128 columns when bn is 128
                const float sc = (bn == 128 && (seg & 127) == 0) ? fsc[(s * 16) >> 7]
                                                                 : __ldg(reinterpret_cast<const float*>(A.scales + (size_t)e * A.s_stride) +
                                                                         (size_t)((live ? r : 0) / (R / A.sr)) * A.sc + (c0 + s * 16) / bn);
                const __half2_raw h01 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(wb & 0xffffu), __NV_E4M3);
                const __half2_raw h23 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(wb >> 16), __NV_E4M3);
                const float w0 = bfround(__fmul_rn(__half2float(__ushort_as_half(h01.x)), sc));
                const float w1 = bfround(__fmul_rn(__half2float(__ushort_as_half(h01.y)), sc));
                const float w2 = bfround(__fmul_rn(__half2float(__ushort_as_half(h23.x)), sc));
                const float w3 = bfround(__fmul_rn(__half2float(__ushort_as_half(h23.y)), sc));
                acc[0] = fmaf(w0, xv.x, acc[0]);
                acc[1] = fmaf(w1, xv.y, acc[1]);
                acc[2] = fmaf(w2, xv.z, acc[2]);
                acc[3] = fmaf(w3, xv.w, acc[3]);
            }
        } else if (FMT == S_MX4) {
            const int nb = n >> 5;
#pragma unroll 4
            for (int b = 0; b < nb; ++b) {
                const unsigned pk = __shfl_sync(0xffffffffu, mxs, (lane & ~3) | (b >> 2));
                const float sc = mx4_scale_s((pk >> ((b & 3) * 8)) & 255u);
                // the block's 16 bytes: byte i holds columns 2i (low nibble) and 2i + 1 of its first 16 columns,
                // byte 8 + i the same of its last 16
                const unsigned lo = *reinterpret_cast<const unsigned short*>(srowp + b * 16 + q * 2);
                const unsigned hi = *reinterpret_cast<const unsigned short*>(srowp + b * 16 + 8 + q * 2);
                const float4 xa = *reinterpret_cast<const float4*>(xp + b * 32 + q * 4);
                const float4 xb = *reinterpret_cast<const float4*>(xp + b * 32 + 16 + q * 4);
                acc[0] = fmaf(__fmul_rn(fp4_value_s(lo & 15u), sc), xa.x, acc[0]);
                acc[1] = fmaf(__fmul_rn(fp4_value_s((lo >> 4) & 15u), sc), xa.y, acc[1]);
                acc[2] = fmaf(__fmul_rn(fp4_value_s((lo >> 8) & 15u), sc), xa.z, acc[2]);
                acc[3] = fmaf(__fmul_rn(fp4_value_s((lo >> 12) & 15u), sc), xa.w, acc[3]);
                acc[0] = fmaf(__fmul_rn(fp4_value_s(hi & 15u), sc), xb.x, acc[0]);
                acc[1] = fmaf(__fmul_rn(fp4_value_s((hi >> 4) & 15u), sc), xb.y, acc[1]);
                acc[2] = fmaf(__fmul_rn(fp4_value_s((hi >> 8) & 15u), sc), xb.z, acc[2]);
                acc[3] = fmaf(__fmul_rn(fp4_value_s((hi >> 12) & 15u), sc), xb.w, acc[3]);
            }
        } else {
            const int steps = n >> 4;
#pragma unroll 4
            for (int s = 0; s < steps; ++s) {
                const uint2 wb = *reinterpret_cast<const uint2*>(srowp + s * 32 + q * 8);
                const float4 xv = *reinterpret_cast<const float4*>(xp + s * 16 + q * 4);
                acc[0] = fmaf(bf_lo(wb.x), xv.x, acc[0]);
                acc[1] = fmaf(bf_hi(wb.x), xv.y, acc[1]);
                acc[2] = fmaf(bf_lo(wb.y), xv.z, acc[2]);
                acc[3] = fmaf(bf_hi(wb.y), xv.w, acc[3]);
            }
        }
        __syncwarp();
        if (issued < n_items) issue_next();
        if (c_seg == nseg - 1) {
            // reduce16's pairwise fold: chains 1 apart, 2 apart (both in this thread), 4 and 8 apart (the row's threads)
            float s = (acc[0] + acc[1]) + (acc[2] + acc[3]);
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            if (live && q == 0) A.y[(size_t)task * R + r] = s;
            acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
            c_seg = 0;
            c_grp += nw;
        } else {
            ++c_seg;
        }
        if (++c_st == S) {
            c_st = 0;
            c_par ^= 1u;
        }
    }
    if (!ok) {
        // a copy never landed: say so, then let the copies still in flight land (bounded) before the shared memory goes
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

struct MSPlan {
    int ctas, warps, seg, stages, smem;
};

template <int FMT>
bool plan_stream(int n_tasks, int R, int C, MSPlan& p) {
    const int sms = b2_sm_count();
    const int groups = (R + RB - 1) / RB;
    p.ctas = max(1, min(groups, sms / max(1, n_tasks)));  // CTAs that share a task
    const int per_cta = (groups + p.ctas - 1) / p.ctas;
    p.warps = max(4, min(MAXW, per_cta));
    // even the rows out: with per_cta groups over the warps, fewer warps may idle less (the last round is fuller)
    {
        const int rounds = (per_cta + p.warps - 1) / p.warps;
        p.warps = max(4, (per_cta + rounds - 1) / rounds);
    }
    const int xbytes = (C * 4 + 127) & ~127;
    const int budget = 200 * 1024 - xbytes;
    for (p.seg = min(512, (C + 31) & ~31);; p.seg = max(32, (p.seg / 2) & ~31)) {
        const int stride = p.seg * col_bytes2<FMT>() / 2 + PAD;
        const int sbytes = RB * stride;
        p.stages = max(2, min(6, budget / (p.warps * (sbytes + 8))));
        p.smem = xbytes + p.warps * p.stages * (sbytes + 8);
        if (p.smem <= 220 * 1024 || p.seg == 32) break;  // two stages must fit: a narrower segment
    }
    return p.smem <= 220 * 1024;
}

template <int FMT>
int launch_stream(const MSArgs& a0, int n_tasks, cudaStream_t s) {
    MSPlan p;
    MSArgs a = a0;
    if (!plan_stream<FMT>(n_tasks, a.R, a.C, p)) return B2_ERR_DOMAIN;
    a.seg = p.seg, a.stages = p.stages;
    auto kern = moe_gemv_stream<FMT>;
    static bool allowed[64];
    int rc = b2_allow_smem(reinterpret_cast<const void*>(kern), allowed);
    if (rc) return rc;
    return b2_launch(reinterpret_cast<const void*>(kern), dim3(p.ctas, n_tasks), dim3(p.warps * 32), p.smem, s, a, 2);
}

}  // namespace

// whether the streaming kernel takes the shape: rows and row segments must start on 16 bytes, x rows on 16
bool b2_moe_stream_ok(int fmt, const void* w, const void* scales, long long w_stride, long long s_stride, const void* x,
                      int R, int C, int sr, int sc) {
    if (reinterpret_cast<uintptr_t>(w) & 15 || reinterpret_cast<uintptr_t>(x) & 15 || (w_stride & 15) || (C & 31)) return false;
    if (fmt == S_FP8 && ((reinterpret_cast<uintptr_t>(scales) & 3) || (s_stride & 3) || R % sr || C % sc)) return false;
    return fmt == S_BF16 || fmt == S_MX4 || fmt == S_FP8;
}

int b2_moe_stream_launch(int fmt, const void* w, const void* scales, long long w_stride, long long s_stride, int sr, int sc,
                         const void* idx, int n_tasks, int E, const void* x, int x_div, void* y, int R, int C, int ep_rank,
                         int ep_size, cudaStream_t s) {
    MSArgs a{static_cast<const uint8_t*>(w), static_cast<const uint8_t*>(scales), w_stride, s_stride,
             static_cast<const int*>(idx), static_cast<const float*>(x), x_div, static_cast<float*>(y), R, C,
             sr > 0 ? sr : 1, sc > 0 ? sc : 1, E, ep_rank, ep_size, 0, 0};
    switch (fmt) {
        case S_BF16: return launch_stream<S_BF16>(a, n_tasks, s);
        case S_MX4: return launch_stream<S_MX4>(a, n_tasks, s);
        case S_FP8: return launch_stream<S_FP8>(a, n_tasks, s);
        default: return B2_ERR_DOMAIN;
    }
}
