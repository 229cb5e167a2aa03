// The MoE block's kernels: router top-k, the experts' matvecs over only the picked experts, the gated activation
// between them and the ordered weighted sum.
//
// What the arithmetic follows: on a CUDA device btb multiplies a decode pass's experts with its HOST kernels (or their
// on-card twins btb_gemv_lane16{,_mx4}_f32, native/cuda/btb_kernels.cu:1635-1766), so an expert's output does not
// depend on where it is seated: x widened to f32, 16 lane sums a row (column c to lane c mod 16, one fma each in
// increasing c), the pairwise fold of native/src/gemv.rs:46-58, f32 out. The row's dtype (bf16) comes back between
// the two matvecs for the gated activation and after the second for the bias, the routing weight and the sum over the
// picked experts in ascending expert id (btb/engine/host.py:508-569 `_Experts._one_row`). Weights are read as stored:
// bf16, MXFP4 blocks + e8m0 scales (btb/mxfp4.py:102-124) or FP8 e4m3 + f32 block scales held as bf16
// (btb/fp8.py:36-100) - widened in registers, no widened copy.
#include <cuda_fp8.h>

#include <cooperative_groups.h>

#include "btb_b200_internal.h"
#include "gemv_core.cuh"
#include "moe_widen.cuh"
#include "tp.cuh"
#include "../../include/btb_b200.h"

B2_DEFINE_STATUS(moe)

namespace cg = cooperative_groups;

bool b2_moe_stream_ok(int fmt, const void* w, const void* scales, long long w_stride, long long s_stride, const void* x,
                      int R, int C, int sr, int sc);
int b2_moe_stream_launch(int fmt, const void* w, const void* scales, long long w_stride, long long s_stride, int sr, int sc,
                         const void* idx, int n_tasks, int E, const void* x, int x_div, void* y, int R, int C, int ep_rank,
                         int ep_size, int act_kind, float alpha, float limit, cudaStream_t s, const B2Send* send = nullptr,
                         int glu_kind = -1, void* glu_out = nullptr);

namespace {

// ---- router ---------------------------------------------------------------------------------------------------------
// mode 0 (native/cuda/btb_kernels.cu:861-948; btb/engine/families/qwen4/router.py:42-50): f32 softmax over the E
// logits (thread i of 256 sums its strided terms, then the 256 -> 1 tree), top-k by (p desc, index asc), weights
// p / sum(top k) summed in rank order, rounded to bf16.
// mode 1 (btb/engine/host.py:187-191, gpt-oss): top-k of the logits themselves, then a softmax over the k.
#define ROUTE_THREADS 256
#define ROUTE_MAX_K 32
struct RouteArgs {
    const void* logits;
    int ls, E, k, mode, f32_logits;
    int* idx;
    bf16* w;
};
// the picks of one row from its E logits (`logit(e)`), by a block of ROUTE_THREADS threads; pr: E floats of shared memory
template <typename Logit>
__device__ __forceinline__ void route_row(Logit logit, int t, int E, int k, int mode, int* idx_out, bf16* w_out, float* pr) {
    __shared__ float red[ROUTE_THREADS];
    __shared__ float topv[ROUTE_MAX_K];
    __shared__ int topi[ROUTE_MAX_K];
    const int tid = threadIdx.x;
    if (mode == 0) {
        // the row's max (any order gives the same value)
        float m = NEG_INF;
        for (int e = tid; e < E; e += ROUTE_THREADS) m = fmaxf(m, logit(e));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if ((tid & 31) == 0) red[tid >> 5] = m;
        __syncthreads();
        m = red[0];
#pragma unroll
        for (int w = 1; w < ROUTE_THREADS / 32; ++w) m = fmaxf(m, red[w]);
        __syncthreads();
        // the sum: thread i's strided terms, then the reference's 256 -> 1 tree (red[t] += red[t + st], st = 128 .. 1)
        // with the same pairs in the same order on one warp: lane l holds red[l + 32 k]
        float s = 0.f;
        for (int e = tid; e < E; e += ROUTE_THREADS) {
            const float p = expf(logit(e) - m);
            pr[e] = p;
            s += p;
        }
        red[tid] = s;
        __syncthreads();
        if (tid < 32) {
            float v[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) v[q] = red[tid + 32 * q];
#pragma unroll
            for (int q = 0; q < 4; ++q) v[q] += v[q + 4];
            v[0] += v[2];
            v[1] += v[3];
            v[0] += v[1];
#pragma unroll
            for (int st = 16; st > 0; st >>= 1) v[0] += __shfl_down_sync(0xffffffffu, v[0], st);
            if (tid == 0) red[0] = v[0];
        }
        __syncthreads();
        s = red[0];
        __syncthreads();
        for (int e = tid; e < E; e += ROUTE_THREADS) pr[e] = pr[e] / s;
    } else {
        for (int e = tid; e < E; e += ROUTE_THREADS) pr[e] = logit(e);
    }
    __syncthreads();
    // k rounds of the total order's maximum (value descending, index ascending) on one warp, no block barriers: lane l
    // scans entries l, l + 32, ..; a picked entry leaves the field by having its slot overwritten with a marker (a NaN
    // payload no softmax produces), so any number of experts the shared row holds is served by the same loop
    constexpr int NONE = 0x7fffffff;
    constexpr uint32_t PICKED = 0x7fc0b200u;
    if (tid < 32) {
        for (int j = 0; j < k; ++j) {
            float bv = 0.f;
            int bi = NONE;
            for (int e = tid; e < E; e += 32) {
                const float v = pr[e];
                if (__float_as_uint(v) == PICKED) continue;
                if (bi == NONE || v > bv) bv = v, bi = e;  // e ascends: a tie keeps the lower index
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (oi != NONE && (bi == NONE || ov > bv || (ov == bv && oi < bi))) bv = ov, bi = oi;
            }
            if (tid == 0) {
                topv[j] = bv, topi[j] = bi;
                if (bi != NONE) pr[bi] = __uint_as_float(PICKED);
            }
            __syncwarp();
        }
    }
    __syncthreads();
    if (tid == 0) {
        if (mode == 0) {
            float sum = 0.f;
            for (int j = 0; j < k; ++j) sum += topv[j];
            for (int j = 0; j < k; ++j) {
                idx_out[(size_t)t * k + j] = topi[j];
                w_out[(size_t)t * k + j] = f2bf(topv[j] / sum);
            }
        } else {
            float m = topv[0], sum = 0.f, ex[ROUTE_MAX_K];
            for (int j = 1; j < k; ++j) m = fmaxf(m, topv[j]);
            for (int j = 0; j < k; ++j) {
                ex[j] = expf(topv[j] - m);
                sum += ex[j];
            }
            for (int j = 0; j < k; ++j) {
                idx_out[(size_t)t * k + j] = topi[j];
                w_out[(size_t)t * k + j] = f2bf(ex[j] / sum);
            }
        }
    }
}

__global__ void __launch_bounds__(ROUTE_THREADS) moe_route(const RouteArgs A) {
    extern __shared__ float pr[];  // [E]
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    auto logit = [&](int e) -> float {
        if (A.f32_logits) return __ldcg(static_cast<const float*>(A.logits) + (size_t)t * A.ls + e);
        const unsigned short u = __ldcg(static_cast<const unsigned short*>(A.logits) + (size_t)t * A.ls + e);
        return __uint_as_float((uint32_t)u << 16);
    };
    route_row(logit, t, A.E, A.k, A.mode, A.idx, A.w, pr);
}

// ---- the router's matvec and the picks in one launch: a cluster of 8 CTAs a row ----------------------------------------
// The router is a small matrix ([E, H] bf16: 0.5 MB for 128 experts) whose matvec and top-k were two dependent launches
// of a few microseconds each, mostly launch latency. Here each CTA of the cluster takes an eighth of the experts' rows
// (staged in shared memory by wide loads, multiplied in the host's 16-lane order: column c on lane c mod 16, pairwise
// fold), writes its logits into the leader's shared memory through the cluster's distributed shared memory, and after
// one cluster barrier the leader picks. The logits are btb_b200_gemv_lane16_f32's and the picks btb_b200_moe_route's.
constexpr int RR_CTAS = 8;
struct RouterArgs {
    const bf16* w;   // [E, H]
    const float* x;  // [T, H] f32 (not read when h_in is given)
    float* rl;       // [T, E] the logits, or null
    int* idx;
    bf16* wout;
    int E, H, k, mode;
    // the block's residual + RMSNorm on the way in (btb_add_rmsnorm and the row's widen, btb/engine/host.py:180-186): with
    // h_in, x = float(bf16(rmsnorm(h_in + y_add) * norm_w)) is made by every CTA of the cluster for itself, and the
    // leader writes the new residual to h_out (never h_in's buffer), the widened row to xf_out and, if asked, the bf16
    // row to x_out
    const bf16* h_in;
    const bf16* y_add;
    const bf16* norm_w;
    bf16* h_out;
    float* xf_out;
    bf16* x_out;
    float eps;
    int centered;
};
__global__ void __cluster_dims__(RR_CTAS, 1, 1) __launch_bounds__(ROUTE_THREADS) moe_router_route(const RouterArgs A) {
    cg::cluster_group cl = cg::this_cluster();
    extern __shared__ __align__(16) unsigned char rsm[];
    const int E = A.E, H = A.H, tid = threadIdx.x;
    const int rank = blockIdx.x, t = blockIdx.y;
    float* xs = reinterpret_cast<float*>(rsm);                                  // [H]
    float* lg = xs + H;                                                          // [E] (the leader's is the one read)
    float* pr = lg + E;                                                          // [E]
    const int wstride = H + 8;                                                   // bf16 elements: rows 16 bytes apart in banks
    bf16* wrows = reinterpret_cast<bf16*>(rsm + ((((size_t)H + 2 * (size_t)E) * 4 + 15) & ~(size_t)15));  // [16][H + 8]
    const int per = (E + RR_CTAS - 1) / RR_CTAS;
    const int r_lo = rank * per, r_hi = min(E, r_lo + per);
    const int hv0 = H >> 3;
    auto stage_rows = [&](int g0, int nrow) {
        for (int i = tid; i < nrow * hv0; i += ROUTE_THREADS) {
            const int ri = i / hv0, c8 = i - ri * hv0;
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(A.w + (size_t)(g0 + ri) * H) + c8);
            *reinterpret_cast<uint4*>(wrows + (size_t)ri * wstride + c8 * 8) = v;
        }
    };
    pdl_launch_dependents();
    // the first group of this CTA's experts' rows does not depend on the kernels before: staged ahead of the wait
    if (r_lo < r_hi) stage_rows(r_lo, min(16, r_hi - r_lo));
    pdl_wait();
    if (A.h_in != nullptr) {
        float* scratch = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(wrows) + 16 * (size_t)wstride * 2);  // H + 256 floats
        bf16* xb = reinterpret_cast<bf16*>(scratch + H + 256);  // the normed row, bf16
        stage_x_norm<1, 0, false>(xb, scratch, A.h_in + (size_t)t * H, nullptr,
                                  A.y_add != nullptr ? A.y_add + (size_t)t * H : nullptr, A.norm_w,
                                  A.h_out != nullptr ? A.h_out + (size_t)t * H : nullptr, A.eps, A.centered, 1, H, rank == 0);
        for (int i = tid; i < H; i += ROUTE_THREADS) {
            const float v = bf2f(xb[i]);
            xs[i] = v;
            if (rank == 0) {
                A.xf_out[(size_t)t * H + i] = v;
                if (A.x_out != nullptr) A.x_out[(size_t)t * H + i] = xb[i];
            }
        }
        __syncthreads();
    } else {
        const float4* xg = reinterpret_cast<const float4*>(A.x + (size_t)t * H);
        for (int i = tid; i < H / 4; i += ROUTE_THREADS) reinterpret_cast<float4*>(xs)[i] = __ldcg(xg + i);
    }
    float* lg0 = cl.map_shared_rank(lg, 0);
    for (int g0 = r_lo; g0 < r_hi; g0 += 16) {
        const int nrow = min(16, r_hi - g0);
        if (g0 != r_lo) stage_rows(g0, nrow);
        __syncthreads();
        const int ri = tid >> 4, j = tid & 15;
        float acc = 0.f;
        if (ri < nrow) {
            const unsigned short* wr = reinterpret_cast<const unsigned short*>(wrows + (size_t)ri * wstride);
#pragma unroll 8
            for (int c = j; c < H; c += 16) acc = fmaf(__uint_as_float((unsigned)wr[c] << 16), xs[c], acc);
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        acc += __shfl_xor_sync(0xffffffffu, acc, 4);
        acc += __shfl_xor_sync(0xffffffffu, acc, 8);
        if (ri < nrow && j == 0) {
            lg0[g0 + ri] = acc;
            if (A.rl != nullptr) A.rl[(size_t)t * E + g0 + ri] = acc;
        }
        __syncthreads();
    }
    cl.sync();  // every CTA's logits stand in the leader's shared memory
    if (rank != 0) return;
    auto logit = [&](int e) -> float { return lg[e]; };
    route_row(logit, t, E, A.k, A.mode, A.idx, A.wout, pr);
}

// ---- the same for routers too large for one cluster: a grid of CTAs a row, the last one to finish picks -----------------
// A cluster is eight SMs; a router of 128 experts x 2048 columns read by eight SMs is slower than its matvec spread over
// the card. Here `parts` CTAs a token take E / parts experts each (the norm prologue made by each for itself, the rows
// staged in shared memory, the host's 16-lane order), write their logits to global memory and count themselves in; the
// CTA that arrives last reads all E logits back and picks (no CTA waits for another). One launch for
// btb_b200_add_rmsnorm_wide, the router's matvec and btb_b200_moe_route.
struct RouterGridArgs {
    RouterArgs r;
    int* cnt;  // [T] arrivals, zero between launches
    int parts;
};
__global__ void __launch_bounds__(ROUTE_THREADS) moe_router_grid(const RouterGridArgs G) {
    const RouterArgs& A = G.r;
    extern __shared__ __align__(16) unsigned char rsm[];
    const int E = A.E, H = A.H, tid = threadIdx.x;
    const int part = blockIdx.x, t = blockIdx.y;
    float* xs = reinterpret_cast<float*>(rsm);  // [H]
    float* pr = xs + H;                          // [E]
    const int wstride = H + 8;
    bf16* wrows = reinterpret_cast<bf16*>(rsm + ((((size_t)H + (size_t)E) * 4 + 15) & ~(size_t)15));  // [16][H + 8]
    __shared__ int s_last;
    pdl_launch_dependents();
    // this CTA's experts' rows do not depend on the kernels before: staged ahead of the wait
    const int per = (E + G.parts - 1) / G.parts;
    const int r_lo = part * per, r_hi = min(E, r_lo + per);
    const int hv = H >> 3;
    const bool one_group = r_hi - r_lo <= 16;
    if (one_group) {
        for (int i = tid; i < (r_hi - r_lo) * hv; i += ROUTE_THREADS) {
            const int ri = i / hv, c8 = i - ri * hv;
            *reinterpret_cast<uint4*>(wrows + (size_t)ri * wstride + c8 * 8) =
                __ldg(reinterpret_cast<const uint4*>(A.w + (size_t)(r_lo + ri) * H) + c8);
        }
    }
    pdl_wait();
    if (A.h_in != nullptr) {
        float* scratch = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(wrows) + 16 * (size_t)wstride * 2);  // H + 256 floats
        bf16* xb = reinterpret_cast<bf16*>(scratch + H + 256);  // the normed row, bf16
        stage_x_norm<1, 0, false>(xb, scratch, A.h_in + (size_t)t * H, nullptr,
                                  A.y_add != nullptr ? A.y_add + (size_t)t * H : nullptr, A.norm_w,
                                  A.h_out != nullptr ? A.h_out + (size_t)t * H : nullptr, A.eps, A.centered, 1, H, part == 0);
        for (int i = tid; i < H; i += ROUTE_THREADS) {
            const float v = bf2f(xb[i]);
            xs[i] = v;
            if (part == 0) {
                A.xf_out[(size_t)t * H + i] = v;
                if (A.x_out != nullptr) A.x_out[(size_t)t * H + i] = xb[i];
            }
        }
        __syncthreads();
    } else {
        const float4* xg = reinterpret_cast<const float4*>(A.x + (size_t)t * H);
        for (int i = tid; i < H / 4; i += ROUTE_THREADS) reinterpret_cast<float4*>(xs)[i] = __ldcg(xg + i);
    }
    for (int g0 = r_lo; g0 < r_hi; g0 += 16) {
        const int nrow = min(16, r_hi - g0);
        if (!one_group) {
            for (int i = tid; i < nrow * hv; i += ROUTE_THREADS) {
                const int ri = i / hv, c8 = i - ri * hv;
                *reinterpret_cast<uint4*>(wrows + (size_t)ri * wstride + c8 * 8) =
                    __ldg(reinterpret_cast<const uint4*>(A.w + (size_t)(g0 + ri) * H) + c8);
            }
        }
        __syncthreads();
        const int ri = tid >> 4, j = tid & 15;
        float acc = 0.f;
        if (ri < nrow) {
            const unsigned short* wr = reinterpret_cast<const unsigned short*>(wrows + (size_t)ri * wstride);
#pragma unroll 8
            for (int c = j; c < H; c += 16) acc = fmaf(__uint_as_float((unsigned)wr[c] << 16), xs[c], acc);
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        acc += __shfl_xor_sync(0xffffffffu, acc, 4);
        acc += __shfl_xor_sync(0xffffffffu, acc, 8);
        if (ri < nrow && j == 0) A.rl[(size_t)t * E + g0 + ri] = acc;
        __syncthreads();
    }
    // count this CTA in; the last one to arrive picks
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(G.cnt + t, 1) == G.parts - 1 ? 1 : 0;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    auto logit = [&](int e) -> float { return __ldcg(A.rl + (size_t)t * E + e); };
    route_row(logit, t, E, A.k, A.mode, A.idx, A.wout, pr);
    if (tid == 0) G.cnt[t] = 0;
}

// ---- the 16-lane matvec over stored weights ---------------------------------------------------------------------------
enum L16Fmt { L_BF16 = 0, L_MX4 = 1, L_FP8 = 2 };
struct L16Args {
    const uint8_t* w;       // expert 0's weights
    const uint8_t* scales;  // MX4: e8m0 bytes; FP8: f32 grid
    long long w_stride, s_stride;  // bytes from an expert to the next
    const int* idx;         // [n_tasks] the task's expert, or null (expert 0 for all)
    const float* x;         // [rows_x, C] f32
    int x_div;              // task i reads x row i / x_div (k: one row a token; 1: a row a task)
    float* y;               // [n_tasks, R] f32
    int R, C, sr, sc, E;
    int ep_rank, ep_size;  // expert e lives on rank e % ep_size as its local expert e / ep_size; others' rows are zeros
};

// The matvec for the shapes the streaming kernel does not take (columns not a multiple of 32, rows that do not start on
// 16 bytes): the same sixteen chains a row, four adjacent chains a thread and four threads a row as there, but every
// weight fetched where it lies with an element-sized load and widened by `stored_weight`. A fallback for odd shapes,
// not a fast path: the benchmark's shapes all stream.
template <int FMT>
__device__ __forceinline__ float stored_weight(const L16Args& A, const uint8_t* wbase, const uint8_t* sbase, int r, int c) {
    if (FMT == L_BF16) {
        return __uint_as_float((uint32_t)__ldg(reinterpret_cast<const unsigned short*>(wbase) + (size_t)r * A.C + c) << 16);
    } else if (FMT == L_MX4) {
        const int G = A.C >> 5, g = c >> 5, i = c & 31;
        const uint32_t byte = __ldg(wbase + ((size_t)r * G + g) * 16 + (i >> 1));
        return __fmul_rn(fp4_to_f32((byte >> ((i & 1) * 4)) & 15u), e8m0_to_f32(__ldg(sbase + (size_t)r * G + g)));
    } else {
        const int bm = A.R / A.sr, bn = A.C / A.sc;
        const float sc = __ldg(reinterpret_cast<const float*>(sbase) + (size_t)(r / bm) * A.sc + c / bn);
        return e4m3_held(__ldg(wbase + (size_t)r * A.C + c), sc);
    }
}
template <int FMT>
__global__ void __launch_bounds__(128) gemv_chains16(const L16Args A) {
    pdl_launch_dependents();
    pdl_wait();
    const int q = threadIdx.x & 3;                       // the thread's chains 4 q .. 4 q + 3
    const int r = blockIdx.x * 32 + (threadIdx.x >> 2);  // its row
    const int task = blockIdx.y;
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
        e /= A.ep_size;
    }
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (r < A.R && mine) {
        const uint8_t* wbase = A.w + (size_t)e * A.w_stride;
        const uint8_t* sbase = A.scales != nullptr ? A.scales + (size_t)e * A.s_stride : nullptr;
        const float* x = A.x + (size_t)(task / A.x_div) * A.C;
        for (int c0 = 4 * q; c0 < A.C; c0 += 16) {
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (c0 + u < A.C) acc[u] = fmaf(stored_weight<FMT>(A, wbase, sbase, r, c0 + u), __ldcg(x + c0 + u), acc[u]);
        }
    }
    // the pairwise fold of the sixteen sums: neighbours, pairs of neighbours (both inside the thread), then across the
    // row's four threads
    float s = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if (r < A.R && q == 0 && e >= 0) A.y[(size_t)task * A.R + r] = s;  // zeros for another rank's expert
}

// ---- between the two matvecs: the row dtype, the bias, the gated activation, back to f32 -------------------------------
// kind 0: silu(gate) * up over gate | up halves (btb/engine/host.py:439-441); kind 1: gpt-oss's clamped GLU over
// interleaved lanes, (up + 1) * gate * sigmoid(alpha * gate) (host.py:444-450) - every torch op's bf16 rounding kept.
struct ActArgs2 {
    const float* gu;  // [n, 2I]
    float* h;         // [n, I]
    const bf16* bias;  // [E, 2I] or null
    const int* idx;
    int n, I, kind;
    float alpha, limit;
};
__global__ void __launch_bounds__(256) moe_act(const ActArgs2 A) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t total = (size_t)A.n * A.I;
    for (size_t q = (size_t)blockIdx.x * 256 + threadIdx.x; q < total; q += (size_t)gridDim.x * 256) {
        const size_t i = q / A.I, c = q - i * A.I;
        const size_t gi = A.kind == 0 ? c : 2 * c, ui = A.kind == 0 ? A.I + c : 2 * c + 1;
        float g = bfround(__ldcg(A.gu + i * 2 * A.I + gi)), u = bfround(__ldcg(A.gu + i * 2 * A.I + ui));
        if (A.bias != nullptr) {
            const bf16* b = A.bias + (size_t)__ldcg(A.idx + i) * 2 * A.I;
            g = bfround(g + bf2f(b[gi]));
            u = bfround(u + bf2f(b[ui]));
        }
        float out;
        if (A.kind == 0) {
            out = bfround(bfround(g / (1.f + expf(-g))) * u);
        } else {
            g = fminf(g, A.limit);
            u = fminf(fmaxf(u, -A.limit), A.limit);
            const float t1 = bfround(g * A.alpha);
            const float t2 = bfround(1.f / (1.f + expf(-t1)));
            const float glu = bfround(g * t2);
            out = bfround(bfround(u + 1.f) * glu);
        }
        A.h[q] = out;
    }
}

// ---- the sum: out_e = bf16(down_e) (+ bias) * w_e, final += out_e one add at a time in ascending expert id ----------
struct CombineArgs {
    const float* dn;  // [T, k, H]
    const int* idx;   // [T, k]
    const bf16* w;    // [T, k]
    const bf16* bias;  // [E, H] or null
    bf16* y;          // [T, H]
    int T, k, H;
    B2Recv recv;      // pass set: dn is this rank's copy of the exchanged products, words [T, k, H] carrying bf16(product)
};
__global__ void __launch_bounds__(256) moe_combine(const CombineArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.y, k = A.k;
    __shared__ int order[ROUTE_MAX_K];
    __shared__ int eid[ROUTE_MAX_K];
    if (threadIdx.x < k) eid[threadIdx.x] = __ldcg(A.idx + (size_t)t * k + threadIdx.x);  // one round trip for all
    __syncthreads();
    if (threadIdx.x == 0) {  // the row's picks by ascending expert id (a handful: insertion sort)
        for (int a = 0; a < k; ++a) order[a] = a;
        for (int a = 1; a < k; ++a) {
            const int v = order[a];
            const int ev = eid[v];
            int b = a - 1;
            while (b >= 0 && eid[order[b]] > ev) {
                order[b + 1] = order[b];
                --b;
            }
            order[b + 1] = v;
        }
    }
    __syncthreads();
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= A.H) return;
    const bool marked = A.recv.pass != nullptr;
    const uint32_t mark = marked ? b2_hop_mark(A.recv.pass, A.recv.per_pass, A.recv.base) : 0u;
    float fin = 0.f;
    if (!marked && A.bias == nullptr && k <= 8) {
        // every pick's product and weight on their way at once (the sum itself is a chain): one round trip, not k
        float pv[8];
        unsigned short pw[8];
#pragma unroll
        for (int a = 0; a < 8; ++a) {
            const size_t q = (size_t)t * k + (a < k ? order[a] : 0);
            pv[a] = a < k ? __ldcg(A.dn + q * A.H + c) : 0.f;
            pw[a] = a < k ? __ldcg(reinterpret_cast<const unsigned short*>(A.w) + q) : (unsigned short)0;
        }
#pragma unroll
        for (int a = 0; a < 8; ++a)
            if (a < k) fin = bfround(fin + bfround(bfround(pv[a]) * __uint_as_float((uint32_t)pw[a] << 16)));
        A.y[(size_t)t * A.H + c] = f2bf(fin);
        return;
    }
    for (int a = 0; a < k; ++a) {
        const int s = order[a];
        const size_t q = (size_t)t * k + s;
        float o = marked ? b2_take1(reinterpret_cast<const uint32_t*>(A.dn) + q * A.H + c, mark)
                         : bfround(__ldcg(A.dn + q * A.H + c));
        if (A.bias != nullptr) o = bfround(o + bf2f(A.bias[(size_t)__ldcg(A.idx + q) * A.H + c]));
        const unsigned short wb = __ldcg(reinterpret_cast<const unsigned short*>(A.w) + q);
        o = bfround(o * __uint_as_float((uint32_t)wb << 16));
        fin = bfround(fin + o);
    }
    A.y[(size_t)t * A.H + c] = f2bf(fin);
}

// ---- the sum and the next norm in one launch -----------------------------------------------------------------------
// y = moe_combine's row (kept in `y` for nobody: written only when y is not null), h = bf16(h + y), x = rmsnorm(h) * w
// and xf = x widened when asked: moe_combine followed by add_rmsnorm, with their arithmetic (the ordered bf16 sum; the
// 256 strided partial sums and the 256 -> 1 tree with the reference's pairs).
struct CombineNormArgs {
    const float* dn;
    const int* idx;
    const bf16* rw;
    bf16* h;
    const bf16* nw;
    bf16* x;
    float* xf;
    bf16* y;
    float eps;
    int k, H, centered;
};
__global__ void __launch_bounds__(256) moe_combine_norm(const CombineNormArgs A) {
    extern __shared__ __align__(16) float hsm[];
    __shared__ float red[256];
    __shared__ int order[ROUTE_MAX_K];
    __shared__ int eid[ROUTE_MAX_K];
    __shared__ float wts[ROUTE_MAX_K];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, tid = threadIdx.x, k = A.k, H = A.H;
    if (tid < k) {
        eid[tid] = __ldcg(A.idx + (size_t)t * k + tid);
        const unsigned short wb = __ldcg(reinterpret_cast<const unsigned short*>(A.rw) + (size_t)t * k + tid);
        wts[tid] = __uint_as_float((uint32_t)wb << 16);
    }
    __syncthreads();
    if (tid == 0) {
        for (int a = 0; a < k; ++a) order[a] = a;
        for (int a = 1; a < k; ++a) {
            const int v = order[a], ev = eid[v];
            int b = a - 1;
            while (b >= 0 && eid[order[b]] > ev) {
                order[b + 1] = order[b];
                --b;
            }
            order[b + 1] = v;
        }
    }
    __syncthreads();
    bf16* hr = A.h + (size_t)t * H;
    float ss = 0.f;
    for (int c = tid; c < H; c += 256) {
        float fin = 0.f;
        for (int a = 0; a < k; ++a) {
            const int sl = order[a];
            float o = bfround(__ldcg(A.dn + ((size_t)t * k + sl) * H + c));
            o = bfround(o * wts[sl]);
            fin = bfround(fin + o);
        }
        if (A.y != nullptr) A.y[(size_t)t * H + c] = f2bf(fin);
        const float hv = bfround(bf2f(hr[c]) + fin);
        hr[c] = f2bf(hv);
        hsm[c] = hv;
        ss = fmaf(hv, hv, ss);  // thread i's strided terms i, i + 256, .. in order: the reference's partial sums
    }
    red[tid] = ss;
    __syncthreads();
    if (tid < 32) {
        float v[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) v[q] = red[tid + 32 * q];
#pragma unroll
        for (int q = 0; q < 4; ++q) v[q] += v[q + 4];
        v[0] += v[2];
        v[1] += v[3];
        v[0] += v[1];
#pragma unroll
        for (int st = 16; st > 0; st >>= 1) v[0] += __shfl_down_sync(0xffffffffu, v[0], st);
        if (tid == 0) red[0] = v[0];
    }
    __syncthreads();
    const float rstd = rsqrtf(red[0] / (float)H + A.eps);
    for (int c = tid; c < H; c += 256) {
        const float wv = bf2f(A.nw[c]);
        const bf16 o = f2bf(hsm[c] * rstd * (A.centered ? 1.f + wv : wv));
        A.x[(size_t)t * H + c] = o;
        if (A.xf != nullptr) A.xf[(size_t)t * H + c] = bf2f(o);
    }
}

// bf16 [n] -> f32 [n] (the experts' and the router's x is the normed row widened)
struct WidenArgs {
    const bf16* x;
    float* y;
    int n;
};
__global__ void __launch_bounds__(256) widen_f32(const WidenArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    for (int i = blockIdx.x * 256 + threadIdx.x; i < A.n; i += gridDim.x * 256) {
        const unsigned short u = __ldcg(reinterpret_cast<const unsigned short*>(A.x) + i);
        A.y[i] = __uint_as_float((uint32_t)u << 16);
    }
}

}  // namespace

extern "C" int btb_b200_moe_route(const void* logits, int ls, int E, int k, int mode, int f32_logits, void* idx, void* w,
                                  int T, void* stream) {
    if (!logits || !idx || !w) return B2_ERR_NULL;
    if (T <= 0 || E <= 0 || k <= 0 || k > E || k > ROUTE_MAX_K || ls < E || E > 8192 || (mode != 0 && mode != 1))
        return B2_ERR_DOMAIN;
    RouteArgs a{logits, ls, E, k, mode, f32_logits, static_cast<int*>(idx), static_cast<bf16*>(w)};
    return b2_launch((const void*)moe_route, dim3(T), dim3(ROUTE_THREADS), (size_t)E * 4, static_cast<cudaStream_t>(stream), a, 4);
}

static int lane16_launch(int fmt, const L16Args& a, int n_tasks, cudaStream_t s) {
    if (n_tasks > 65535) return B2_ERR_DOMAIN;
    // every shape the streaming kernel takes goes there (one task a pass row for the plain matvec entry points)
    if (b2_tuning().moe_stream && b2_moe_stream_ok(fmt, a.w, a.scales, a.w_stride, a.s_stride, a.x, a.R, a.C, a.sr, a.sc))
        return b2_moe_stream_launch(fmt, a.w, a.scales, a.w_stride, a.s_stride, a.sr, a.sc, a.idx, n_tasks, a.E, a.x, a.x_div,
                                    a.y, a.R, a.C, a.ep_rank, a.ep_size, -1, 0.f, 0.f, s);
    const dim3 grid((a.R + 31) / 32, n_tasks);
    switch (fmt) {
        case L_BF16: return b2_launch((const void*)gemv_chains16<L_BF16>, grid, dim3(128), 0, s, a, 4);
        case L_MX4: return b2_launch((const void*)gemv_chains16<L_MX4>, grid, dim3(128), 0, s, a, 4);
        case L_FP8: return b2_launch((const void*)gemv_chains16<L_FP8>, grid, dim3(128), 0, s, a, 4);
        default: return B2_ERR_DOMAIN;
    }
}

extern "C" int btb_b200_gemv_lane16_f32(const void* w, const void* x, void* y, int M, int R, int C, void* stream) {
    if (!w || !x || !y) return B2_ERR_NULL;
    if (M <= 0 || R <= 0 || C <= 0) return B2_ERR_DOMAIN;
    L16Args a{static_cast<const uint8_t*>(w), nullptr, 0, 0, nullptr, static_cast<const float*>(x), 1,
              static_cast<float*>(y), R, C, 1, 1, 1, 0, 1};
    return lane16_launch(L_BF16, a, M, static_cast<cudaStream_t>(stream));
}

extern "C" int btb_b200_gemv_lane16_mx4_f32(const void* blocks, const void* scales, const void* x, void* y, int M, int R,
                                            int C, void* stream) {
    if (!blocks || !scales || !x || !y) return B2_ERR_NULL;
    if (M <= 0 || R <= 0 || C <= 0 || (C & 31)) return B2_ERR_DOMAIN;
    L16Args a{static_cast<const uint8_t*>(blocks), static_cast<const uint8_t*>(scales), 0, 0, nullptr,
              static_cast<const float*>(x), 1, static_cast<float*>(y), R, C, 1, 1, 1, 0, 1};
    return lane16_launch(L_MX4, a, M, static_cast<cudaStream_t>(stream));
}

extern "C" int btb_b200_gemv_lane16_fp8_f32(const void* w, const void* scales, int sr, int sc, const void* x, void* y,
                                            int M, int R, int C, void* stream) {
    if (!w || !scales || !x || !y) return B2_ERR_NULL;
    if (M <= 0 || R <= 0 || C <= 0 || sr <= 0 || sc <= 0 || R % sr || C % sc) return B2_ERR_DOMAIN;
    L16Args a{static_cast<const uint8_t*>(w), static_cast<const uint8_t*>(scales), 0, 0, nullptr,
              static_cast<const float*>(x), 1, static_cast<float*>(y), R, C, sr, sc, 1, 0, 1};
    return lane16_launch(L_FP8, a, M, static_cast<cudaStream_t>(stream));
}

// the picked experts' matvecs in one launch: task i = (row i / k, pick i % k) multiplies expert idx[i]'s [R, C]
// matrix with x row (i / x_div). fmt 0 bf16, 1 MXFP4, 2 FP8.
extern "C" int btb_b200_moe_gemv(int fmt, const void* w, const void* scales, long long w_stride, long long s_stride,
                                 int sr, int sc, const void* idx, int n_tasks, int E, const void* x, int x_div, void* y,
                                 int R, int C, int ep_rank, int ep_size, void* stream) {
    if (!w || !x || !y || (fmt != L_BF16 && !scales)) return B2_ERR_NULL;  // idx null: every task is matrix 0
    if (n_tasks <= 0 || R <= 0 || C <= 0 || x_div <= 0 || E <= 0 || ep_size < 1 || ep_rank < 0 || ep_rank >= ep_size)
        return B2_ERR_DOMAIN;
    if (fmt == L_MX4 && (C & 31)) return B2_ERR_DOMAIN;
    if (fmt == L_FP8 && (sr <= 0 || sc <= 0 || R % sr || C % sc)) return B2_ERR_DOMAIN;
    // the streaming kernel takes every shape whose rows start on 16 bytes; the rest take the element-load kernel
    L16Args a{static_cast<const uint8_t*>(w), static_cast<const uint8_t*>(scales), w_stride, s_stride,
              static_cast<const int*>(idx), static_cast<const float*>(x), x_div, static_cast<float*>(y), R, C,
              sr > 0 ? sr : 1, sc > 0 ? sc : 1, E, ep_rank, ep_size};
    return lane16_launch(fmt, a, n_tasks, static_cast<cudaStream_t>(stream));
}

// btb_b200_moe_gemv with the experts cut over ranks and the exchange folded in: an expert this rank holds
// (expert e on rank e % ep_size) writes bf16(output) as marked words into every rank's copy of the [n_tasks, R] vector;
// the other picks' rows are their owners'. Shapes the streaming kernel takes only.
extern "C" int btb_b200_moe_gemv_x(int fmt, const void* w, const void* scales, long long w_stride, long long s_stride,
                                   int sr, int sc, const void* idx, int n_tasks, int E, const void* x, int x_div, int R,
                                   int C, int ep_rank, int ep_size, const btb_b200_send* send, void* stream) {
    if (!w || !x || !send || (fmt != L_BF16 && !scales)) return B2_ERR_NULL;
    if (n_tasks <= 0 || n_tasks > 65535 || R <= 0 || C <= 0 || x_div <= 0 || E <= 0 || ep_size < 1 || ep_rank < 0 ||
        ep_rank >= ep_size)
        return B2_ERR_DOMAIN;
    if (fmt == L_FP8 && (sr <= 0 || sc <= 0 || R % sr || C % sc)) return B2_ERR_DOMAIN;
    if (send->n < 1 || send->n > B2_MAX_RANKS || send->stride < R || send->offset != 0) return B2_ERR_DOMAIN;
    if (send->pass == nullptr) return B2_ERR_NULL;
    B2Send sd{};
    sd.n = send->n, sd.stride = send->stride, sd.offset = 0;
    sd.pass = static_cast<const unsigned*>(send->pass), sd.per_pass = send->per_pass, sd.base = send->base;
    for (int p = 0; p < send->n; ++p) {
        if (send->out[p] == nullptr) return B2_ERR_NULL;
        sd.out[p] = static_cast<uint32_t*>(send->out[p]);
    }
    if (!b2_moe_stream_ok(fmt, w, scales, w_stride, s_stride, x, R, C, sr, sc)) return B2_ERR_DOMAIN;
    return b2_moe_stream_launch(fmt, w, scales, w_stride, s_stride, sr, sc, idx, n_tasks, E, x, x_div, nullptr, R, C, ep_rank,
                                ep_size, -1, 0.f, 0.f, static_cast<cudaStream_t>(stream), &sd);
}

// the picked experts' DOWN matvecs with the gated activation made on the way in: x row of task i = act(gu row i).
// btb_b200_moe_act followed by btb_b200_moe_gemv (x_div 1), one launch and no [n, I] buffer. No bias.
extern "C" int btb_b200_moe_gemv_act(int fmt, const void* w, const void* scales, long long w_stride, long long s_stride,
                                     int sr, int sc, const void* idx, int n_tasks, int E, const void* gu, int kind,
                                     float alpha, float limit, void* y, int R, int C, int ep_rank, int ep_size,
                                     void* stream) {
    if (!w || !gu || !y || (fmt != L_BF16 && !scales)) return B2_ERR_NULL;
    if (n_tasks <= 0 || n_tasks > 65535 || R <= 0 || C <= 0 || E <= 0 || ep_size < 1 || ep_rank < 0 || ep_rank >= ep_size ||
        (kind != 0 && kind != 1))
        return B2_ERR_DOMAIN;
    if (fmt == L_FP8 && (sr <= 0 || sc <= 0 || R % sr || C % sc)) return B2_ERR_DOMAIN;
    if (!b2_moe_stream_ok(fmt, w, scales, w_stride, s_stride, gu, R, C, sr, sc)) return B2_ERR_DOMAIN;
    return b2_moe_stream_launch(fmt, w, scales, w_stride, s_stride, sr, sc, idx, n_tasks, E, gu, 1, y, R, C, ep_rank,
                                ep_size, kind, alpha, limit, static_cast<cudaStream_t>(stream));
}

// the picked experts' GATE/UP matvecs with the gated activation made on the way out: h row of task i [R/2] = act(the
// task's [R] outputs). btb_b200_moe_gemv followed by btb_b200_moe_act, one launch and no [n, R] buffer. No bias.
extern "C" int btb_b200_moe_gemv_glu(int fmt, const void* w, const void* scales, long long w_stride, long long s_stride,
                                     int sr, int sc, const void* idx, int n_tasks, int E, const void* x, int x_div, void* h,
                                     int R, int C, int kind, float alpha, float limit, int ep_rank, int ep_size,
                                     void* stream) {
    if (!w || !x || !h || (fmt != L_BF16 && !scales)) return B2_ERR_NULL;
    if (n_tasks <= 0 || n_tasks > 65535 || R <= 0 || C <= 0 || x_div <= 0 || E <= 0 || ep_size < 1 || ep_rank < 0 ||
        ep_rank >= ep_size || (kind != 0 && kind != 1))
        return B2_ERR_DOMAIN;
    if (fmt == L_FP8 && (sr <= 0 || sc <= 0 || R % sr || C % sc)) return B2_ERR_DOMAIN;
    if (!b2_moe_stream_ok(fmt, w, scales, w_stride, s_stride, x, R, C, sr, sc)) return B2_ERR_DOMAIN;
    return b2_moe_stream_launch(fmt, w, scales, w_stride, s_stride, sr, sc, idx, n_tasks, E, x, x_div, nullptr, R, C, ep_rank,
                                ep_size, -1, alpha, limit, static_cast<cudaStream_t>(stream), nullptr, kind, h);
}

extern "C" int btb_b200_moe_act(const void* gu, void* h, const void* bias, const void* idx, int n, int I, int kind,
                                float alpha, float limit, void* stream) {
    if (!gu || !h || (bias && !idx)) return B2_ERR_NULL;
    if (n <= 0 || I <= 0 || (kind != 0 && kind != 1)) return B2_ERR_DOMAIN;
    ActArgs2 a{static_cast<const float*>(gu), static_cast<float*>(h), static_cast<const bf16*>(bias),
               static_cast<const int*>(idx), n, I, kind, alpha, limit};
    const long long tot = (long long)n * I;
    const int grid = (int)((tot + 255) / 256 < 1184 ? (tot + 255) / 256 : 1184);
    return b2_launch((const void*)moe_act, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), a, 4);
}

static int combine_impl(const void* dn, const void* idx, const void* w, const void* bias, void* y, int T, int k, int H,
                        const btb_b200_recv* recv, void* stream) {
    if (!dn || !idx || !w || !y) return B2_ERR_NULL;
    if (T <= 0 || k <= 0 || k > ROUTE_MAX_K || H <= 0) return B2_ERR_DOMAIN;
    CombineArgs a{static_cast<const float*>(dn), static_cast<const int*>(idx), static_cast<const bf16*>(w),
                  static_cast<const bf16*>(bias), static_cast<bf16*>(y), T, k, H, B2Recv{nullptr, 0u, 0u}};
    if (recv != nullptr && recv->pass != nullptr) a.recv = B2Recv{static_cast<const unsigned*>(recv->pass), recv->per_pass, recv->base};
    return b2_launch((const void*)moe_combine, dim3((H + 255) / 256, T), dim3(256), 0, static_cast<cudaStream_t>(stream), a, 4);
}

extern "C" int btb_b200_moe_combine(const void* dn, const void* idx, const void* w, const void* bias, void* y, int T,
                                    int k, int H, void* stream) {
    return combine_impl(dn, idx, w, bias, y, T, k, H, nullptr, stream);
}

// experts cut over ranks: dn is this rank's copy of the exchanged products (marked words [T, k, H], each bf16(product))
extern "C" int btb_b200_moe_combine_x(const void* dn_words, const void* idx, const void* w, const void* bias, void* y, int T,
                                      int k, int H, const btb_b200_recv* recv, void* stream) {
    if (recv == nullptr || recv->pass == nullptr) return B2_ERR_NULL;
    return combine_impl(dn_words, idx, w, bias, y, T, k, H, recv, stream);
}

extern "C" int btb_b200_widen_f32(const void* x, void* y, int n, void* stream) {
    if (!x || !y) return B2_ERR_NULL;
    if (n <= 0) return B2_ERR_DOMAIN;
    WidenArgs a{static_cast<const bf16*>(x), static_cast<float*>(y), n};
    const int grid = (n + 255) / 256 < 296 ? (n + 255) / 256 : 296;
    return b2_launch((const void*)widen_f32, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), a, 4);
}

extern "C" int btb_b200_moe_combine_norm(const void* dn, const void* idx, const void* w, int k, void* h, const void* norm_w,
                                         float eps, void* x, void* xf, void* y, int T, int H, int centered, void* stream) {
    if (!dn || !idx || !w || !h || !norm_w || !x) return B2_ERR_NULL;
    if (T <= 0 || k <= 0 || k > ROUTE_MAX_K || H <= 0 || (size_t)H * 4 > 200 * 1024 || !(eps == eps)) return B2_ERR_DOMAIN;
    CombineNormArgs a{static_cast<const float*>(dn), static_cast<const int*>(idx), static_cast<const bf16*>(w),
                      static_cast<bf16*>(h), static_cast<const bf16*>(norm_w), static_cast<bf16*>(x),
                      static_cast<float*>(xf), static_cast<bf16*>(y), eps, k, H, centered};
    static bool allowed[64];
    if (const int rc = b2_allow_smem((const void*)moe_combine_norm, allowed)) return rc;
    return b2_launch((const void*)moe_combine_norm, dim3(T), dim3(256), (size_t)H * 4, static_cast<cudaStream_t>(stream), a, 4);
}

// the router's matvec and the picks as one cluster launch; shapes it does not take (H not a multiple of 8, more than 1024
// experts, unaligned pointers) are refused: use btb_b200_gemv_lane16_f32 and btb_b200_moe_route
static int moe_router_launch(RouterArgs a, const void* align_a, const void* align_b, int T, void* stream) {
    const int E = a.E, H = a.H, k = a.k;
    if (!a.w || !a.idx || !a.wout) return B2_ERR_NULL;
    if (T <= 0 || T > 65535 || E <= 0 || E > 1024 || k <= 0 || k > E || k > ROUTE_MAX_K || H <= 0 || (H & 7) ||
        (a.mode != 0 && a.mode != 1))
        return B2_ERR_DOMAIN;
    if ((reinterpret_cast<uintptr_t>(a.w) & 15) || (reinterpret_cast<uintptr_t>(align_a) & 15) ||
        (reinterpret_cast<uintptr_t>(align_b) & 15))
        return B2_ERR_DOMAIN;
    const size_t smem = ((((size_t)H + 2 * (size_t)E) * 4 + 15) & ~(size_t)15) + 16 * ((size_t)H + 8) * 2 +
                        (a.h_in != nullptr ? ((size_t)H + 256) * 4 + (size_t)H * 2 : 0);  // + the norm's own scratch
    if (smem > 200 * 1024) return B2_ERR_DOMAIN;
    static bool allowed[64];
    if (const int rc = b2_allow_smem((const void*)moe_router_route, allowed)) return rc;
    return b2_launch((const void*)moe_router_route, dim3(RR_CTAS, T), dim3(ROUTE_THREADS), smem,
                     static_cast<cudaStream_t>(stream), a, 4);
}

extern "C" int btb_b200_moe_router(const void* w, const void* x, void* logits, int E, int H, int k, int mode, void* idx,
                                   void* wout, int T, void* stream) {
    if (!x) return B2_ERR_NULL;
    RouterArgs a{};
    a.w = static_cast<const bf16*>(w), a.x = static_cast<const float*>(x), a.rl = static_cast<float*>(logits);
    a.idx = static_cast<int*>(idx), a.wout = static_cast<bf16*>(wout), a.E = E, a.H = H, a.k = k, a.mode = mode;
    return moe_router_launch(a, x, nullptr, T, stream);
}

// the same with the block's residual add, RMSNorm and widen in its prologue: one launch for btb_b200_add_rmsnorm_wide and
// btb_b200_moe_router (the same operations in the same order: the same bits)
extern "C" int btb_b200_moe_router_norm(const void* w, const void* h_in, const void* y_add, const void* norm_w, float eps,
                                        int centered, void* h_out, void* x_out, void* xf_out, void* logits, int E, int H,
                                        int k, int mode, void* idx, void* wout, int T, void* stream) {
    if (!h_in || !norm_w || !xf_out || (y_add && !h_out)) return B2_ERR_NULL;
    if (h_out == h_in || !(eps == eps)) return B2_ERR_DOMAIN;
    if ((reinterpret_cast<uintptr_t>(y_add) | reinterpret_cast<uintptr_t>(h_out) | reinterpret_cast<uintptr_t>(xf_out) |
         reinterpret_cast<uintptr_t>(x_out)) & 15)
        return B2_ERR_DOMAIN;
    RouterArgs a{};
    a.w = static_cast<const bf16*>(w), a.rl = static_cast<float*>(logits);
    a.idx = static_cast<int*>(idx), a.wout = static_cast<bf16*>(wout), a.E = E, a.H = H, a.k = k, a.mode = mode;
    a.h_in = static_cast<const bf16*>(h_in), a.y_add = static_cast<const bf16*>(y_add);
    a.norm_w = static_cast<const bf16*>(norm_w), a.h_out = static_cast<bf16*>(h_out);
    a.xf_out = static_cast<float*>(xf_out), a.x_out = static_cast<bf16*>(x_out), a.eps = eps, a.centered = centered;
    return moe_router_launch(a, h_in, norm_w, T, stream);
}

// btb_b200_moe_router_norm for routers of any size: `parts` CTAs a token over the whole card instead of one cluster, the
// last CTA to finish picks. logits f32 [T, E] (required: the CTAs meet there) and cnt i32 [T] (zero before the first
// launch; the kernel leaves it zero). h_in null: x f32 [T, H] is read as btb_b200_moe_router reads it (pass it as xf_out).
extern "C" int btb_b200_moe_router_grid(const void* w, const void* h_in, const void* y_add, const void* norm_w, float eps,
                                        int centered, void* h_out, void* x_out, void* xf_out, void* logits, void* cnt, int E,
                                        int H, int k, int mode, void* idx, void* wout, int T, void* stream) {
    if (!w || !xf_out || !logits || !cnt || !idx || !wout || (h_in && !norm_w) || (y_add && !h_out)) return B2_ERR_NULL;
    if (T <= 0 || T > 65535 || E <= 0 || E > 8192 || k <= 0 || k > E || k > ROUTE_MAX_K || H <= 0 || (H & 7) ||
        (mode != 0 && mode != 1) || (h_in && h_out == h_in) || !(eps == eps))
        return B2_ERR_DOMAIN;
    if ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(h_in) | reinterpret_cast<uintptr_t>(y_add) |
         reinterpret_cast<uintptr_t>(norm_w) | reinterpret_cast<uintptr_t>(h_out) | reinterpret_cast<uintptr_t>(xf_out) |
         reinterpret_cast<uintptr_t>(x_out)) & 15)
        return B2_ERR_DOMAIN;
    const size_t smem = ((((size_t)H + (size_t)E) * 4 + 15) & ~(size_t)15) + 16 * ((size_t)H + 8) * 2 +
                        (h_in != nullptr ? ((size_t)H + 256) * 4 + (size_t)H * 2 : 0);  // + the norm's own scratch
    if (smem > 200 * 1024) return B2_ERR_DOMAIN;
    RouterGridArgs g{};
    RouterArgs& a = g.r;
    a.w = static_cast<const bf16*>(w), a.rl = static_cast<float*>(logits);
    a.x = h_in ? nullptr : static_cast<const float*>(xf_out);
    a.idx = static_cast<int*>(idx), a.wout = static_cast<bf16*>(wout), a.E = E, a.H = H, a.k = k, a.mode = mode;
    a.h_in = static_cast<const bf16*>(h_in), a.y_add = static_cast<const bf16*>(y_add);
    a.norm_w = static_cast<const bf16*>(norm_w), a.h_out = static_cast<bf16*>(h_out);
    a.xf_out = static_cast<float*>(xf_out), a.x_out = static_cast<bf16*>(x_out), a.eps = eps, a.centered = centered;
    g.cnt = static_cast<int*>(cnt);
    // four experts a CTA where the card has CTAs to spare (a row offers sixteen chains: 64 threads work, 256 stage)
    const int per = T * ((E + 3) / 4) <= 2 * b2_sm_count() ? 4 : 16;
    g.parts = (E + per - 1) / per;
    static bool allowed[64];
    if (const int rc = b2_allow_smem((const void*)moe_router_grid, allowed)) return rc;
    return b2_launch((const void*)moe_router_grid, dim3(g.parts, T), dim3(ROUTE_THREADS), smem,
                     static_cast<cudaStream_t>(stream), g, 4);
}
