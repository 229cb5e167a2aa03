// The whole decode step as ONE persistent kernel: embed -> L x [norm + qkv GEMV, RoPE + cache write, attention,
// o GEMV, norm + gate/up GEMV, SwiGLU + down GEMV] -> final norm + head GEMV -> greedy pick -> publish, for one or
// more steps a launch.
//
// Why: at batch 1 a Qwen3-4B-sized layer is 202 MB of weights - 31 us at HBM rate - cut into four GEMVs of 21-100 MB.
// As separate launches each pays a fixed ~3.5 us (launch, barrier init, first-byte latency, tail) and the HBM pipe
// idles through every boundary. Here 148 CTAs stay resident for the whole step and walk a small program of phases
// (btb's card graph body, btb/engine/cuda.py:1722-1834, as data). Every warp keeps its TMA ring running ACROSS
// phases: when it has issued the last weight copy of the GEMV it is consuming it goes on issuing the first copies of
// the next GEMV of the program - weights depend on nothing - so when the grid barrier between two phases opens, the
// next phase's first stages are already in shared memory. Phases are separated by a grid barrier (one atomic
// arrival + a bounded acquire spin per CTA); the launch is cooperative, so all CTAs are co-resident by construction.
//
// The arithmetic is the standalone kernels' (gemv_core.cuh, attn_core.cuh): same chains, same trees, same folds -
// a step computed here is bit-identical to the step computed by the separate launches (tests/test_gpu_step.py).
// Buffers other SMs rewrote earlier in the launch are read with L2-coherent loads.
#include "btb_b200_internal.h"
#include "gemv_core.cuh"
#include "attn_core.cuh"
#include "../../include/btb_b200.h"

B2_DEFINE_STATUS(step)

namespace {

constexpr int NWS = 16;        // warps a CTA
constexpr int NTS = NWS * 32;  // 512 threads

enum OpKind { OP_END = 0, OP_GEMV = 1, OP_ROPE = 2, OP_ATTN = 3, OP_PICK = 4 };
enum XKind { XK_COPY = 0, XK_SILU = 1, XK_NORM = 2 };

// one phase of the program. The layout is mirrored by ctypes in btb_b200/step.py: keep the two in step.
struct StepOp {
    int32_t kind, fmt, xkind, R, C, seg, next_gemv, centered;
    float eps, scale;
    int32_t win, pad0;
    const uint8_t* w;  // bf16 weights, or pack12 low bytes
    const uint8_t* hi4;
    const int32_t* esc_idx;
    const uint8_t* esc_val;
    const int32_t* esc_row;
    uint32_t table[4];
    const bf16* x;  // GEMV input (COPY), gate/up block (SILU); ROPE: the qkv block
    bf16* y;        // GEMV output
    const bf16* h_in;
    const bf16* y_add;
    const bf16* norm_w;
    bf16* h_out;
    const long long* rows;  // NORM: input row m is h_in + rows[m] * C (the embedding gather)
    const bf16* wq;         // ROPE: q/k norm weights
    const bf16* wk;
    bf16* K;  // ROPE / ATTN: the layer's cache
    bf16* V;
    bf16* q;    // ROPE out / ATTN in
    bf16* att;  // ATTN out
};

struct StepArgs {
    const StepOp* ops;
    int32_t n_ops, first_gemv, T, steps, S, stage_cap, front_bytes, norm_bytes;
    int32_t cap, Hq, Hk, vocab;
    long long hs, rs;
    int* n0;
    const int* depth;
    const int* par;
    const int* tbl;
    const float* sinks;
    const bf16* cos_t;
    const bf16* sin_t;
    float* part_m;
    float* part_l;
    float* part_acc;
    int* cnt;
    unsigned* bar;    // grid barrier counter, zero at launch
    int* abort_flag;  // zero at launch
    const bf16* logits;
    unsigned long long* pick_keys;  // [T], zero at launch and left zero
    long long* ids;                 // [T] the step's token ids in, the picked ids out
    long long* tok_out;             // [steps] every step's first-row pick (may be null)
    long long* pin_tok;             // pinned host handoff (may be null)
    int* pin_n0;
    long long* pin_ts;
    int32_t advance;  // n0 += advance after each step
    int32_t pick;     // 1: the program ends with a PICK phase whose result feeds the next step
    long long* trace;  // null, or [n_ops * 2] device clock (ns) of one CTA: a phase's start, its arrival at the barrier
    int32_t trace_cta, pad1;
};

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// a barrier over the (co-resident) grid: arrive once, then a bounded spin until everyone has. Returns false when the
// wait ran out or another CTA gave up: the caller leaves the kernel.
#define GRID_SPIN_LIMIT (1u << 24)
__device__ __forceinline__ bool grid_sync(unsigned* counter, unsigned target, int* abort_flag, int* s_ok) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(counter, 1u);
        int ok = 1;
        unsigned it = 0;
        while (ld_acquire_u32(counter) < target) {
            if (++it > GRID_SPIN_LIMIT || *reinterpret_cast<volatile int*>(abort_flag) != 0) {
                ok = 0;
                break;
            }
        }
        if (!ok) {
            atomicExch(abort_flag, 1);
            b2_fail(B2_ERR_TIMEOUT);
        }
        __threadfence();
        *s_ok = ok;
    }
    __syncthreads();
    return *s_ok != 0;
}

__device__ __forceinline__ unsigned long long pick_key64(float v, int idx) {
    const unsigned b = __float_as_uint(v);
    const unsigned u = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned long long)(0xffffffffu - (unsigned)idx);
}

template <int M, int D, int G>
__global__ void __launch_bounds__(NTS, 1) step_kernel(const StepArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_ok;
    __shared__ unsigned long long s_best[NWS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = A.S, cap_b = A.stage_cap;
    float* norm_scratch = reinterpret_cast<float*>(smem);
    bf16* xs = reinterpret_cast<bf16*>(smem + A.norm_bytes);
    uint8_t* attn_scratch = smem;  // shares the front region with x: never live together
    uint8_t* ring = smem + A.front_bytes + (size_t)warp * S * cap_b;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + A.front_bytes + (size_t)NWS * S * cap_b) + warp * S;
    const StepOp* ops = A.ops;

    if (lane == 0) {
        for (int s = 0; s < S; ++s) mbar_init(smem_u32(bars + s), 1);
        mbar_fence_init();
    }
    __syncwarp();
    const uint64_t pol = l2_evict_first_policy();

    // this CTA's rows of a GEMV of R rows, and this warp's share of them
    auto my_rows = [&](int R, int& r0) {
        const int base = R / gridDim.x, rem = R % gridDim.x;
        r0 = blockIdx.x * base + min((int)blockIdx.x, rem);
        const int cnt = base + ((int)blockIdx.x < rem ? 1 : 0);
        return cnt > warp ? (cnt - warp + NWS - 1) / NWS : 0;
    };

    // ---- the producer: streams the program's GEMV weights through this warp's ring, in program order ------------
    int p_op = A.first_gemv, p_row = 0, p_seg = 0, p_left = 0, p_nseg = 1, p_segel = 256, p_C = 0, p_fmt = 0;
    int p_st = 0, inflight = 0, p_round = 0;  // p_round: how many times the producer wrapped to the next step
    const uint8_t* p_w = nullptr;
    const uint8_t* p_hi4 = nullptr;
    auto begin_stream = [&](int oi) {
        p_op = oi;
        p_C = ops[oi].C, p_segel = ops[oi].seg, p_fmt = ops[oi].fmt;
        p_w = ops[oi].w, p_hi4 = ops[oi].hi4;
        p_nseg = (p_C + p_segel - 1) / p_segel;
        int r0;
        p_left = my_rows(ops[oi].R, r0) * p_nseg;
        p_row = r0 + warp, p_seg = 0;
    };
    // fill free stages; the producer may run ahead into op `limit` (the GEMV after the one being consumed) at most
    auto issue_some = [&](int limit, int limit_round) {
        while (inflight < S) {
            if (p_left == 0) {
                if (p_op == limit && p_round == limit_round) break;
                int nx = ops[p_op].next_gemv;
                if (nx < 0) break;
                if (nx <= p_op) {  // wraps into the next step of this launch
                    if (p_round + 1 >= A.steps) break;
                    ++p_round;
                }
                begin_stream(nx);
                continue;
            }
            const int c0 = p_seg * p_segel;
            const int n = min(p_segel, p_C - c0);
            if (lane == 0) {
                const uint32_t bar = smem_u32(bars + p_st);
                const uint32_t dst = smem_u32(ring + (size_t)p_st * cap_b);
                const size_t e0 = (size_t)p_row * p_C + c0;
                if (p_fmt == F_BF16) {
                    mbar_expect_tx(bar, n * 2);
                    bulk_g2s_hint(dst, p_w + e0 * 2, n * 2, bar, pol);
                } else {
                    mbar_expect_tx(bar, n + n / 2);
                    bulk_g2s_hint(dst, p_w + e0, n, bar, pol);
                    bulk_g2s_hint(dst + p_segel, p_hi4 + e0 / 2, n / 2, bar, pol);
                }
            }
            ++inflight;
            --p_left;
            if (++p_st == S) p_st = 0;
            if (++p_seg == p_nseg) {
                p_seg = 0;
                p_row += NWS;
            }
        }
    };
    begin_stream(A.first_gemv);
    issue_some(A.first_gemv, 0);

    int c_st = 0;
    uint32_t c_par = 0;
    unsigned bar_target = 0;
    bool alive = true;
    // leave cleanly: let this warp's copies in flight land (bounded) before the shared memory goes away
    auto drain = [&]() {
        while (inflight > 0) {
            mbar_wait_bounded(smem_u32(bars + c_st), c_par);
            if (++c_st == S) {
                c_st = 0;
                c_par ^= 1u;
            }
            --inflight;
        }
    };
#define STEP_BARRIER()                                                \
    do {                                                              \
        if (tracing) {                                                \
            unsigned long long ts_;                                   \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ts_));   \
            A.trace[2 * oi + 1] = (long long)ts_;                     \
        }                                                             \
        bar_target += gridDim.x;                                      \
        if (!grid_sync(A.bar, bar_target, A.abort_flag, &s_ok)) {     \
            alive = false;                                            \
        }                                                             \
    } while (0)

    for (int step = 0; step < A.steps && alive; ++step) {
        for (int oi = 0; oi < A.n_ops && alive; ++oi) {
            const int kind = ops[oi].kind;
            const bool tracing = A.trace != nullptr && (int)blockIdx.x == A.trace_cta && threadIdx.x == 0;
            if (tracing) {
                unsigned long long ts;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ts));
                A.trace[2 * oi] = (long long)ts;
            }
            if (kind == OP_GEMV) {
                const StepOp& op = ops[oi];
                const int C = op.C, R = op.R, seg = op.seg, fmt = op.fmt;
                // x on the way in (the previous phase's output, visible after the barrier)
                if (op.xkind == XK_COPY) stage_x_copy<M, NTS>(xs, op.x, C);
                else if (op.xkind == XK_SILU) stage_x_silu<M, NTS, 1>(xs, op.x, C);
                else
                    stage_x_norm<M, NTS, false>(xs, norm_scratch, op.h_in, op.rows, op.y_add, op.norm_w, op.h_out, op.eps,
                                         op.centered, A.T, C, blockIdx.x == 0);
                __syncthreads();
                const int nseg = (C + seg - 1) / seg;
                int r0;
                const int n_items = my_rows(R, r0) * nseg;
                int c_row = r0 + warp, c_seg = 0;
                const int limit = op.next_gemv < 0 ? oi : op.next_gemv;
                const int limit_round = (op.next_gemv >= 0 && op.next_gemv <= oi) ? step + 1 : step;
                uint32_t table[4] = {op.table[0], op.table[1], op.table[2], op.table[3]};
                float acc[M];
#pragma unroll
                for (int m = 0; m < M; ++m) acc[m] = 0.f;
                for (int i = 0; i < n_items; ++i) {
                    if (!mbar_wait_bounded(smem_u32(bars + c_st), c_par)) {
                        if (lane == 0) {
                            b2_fail(B2_ERR_TIMEOUT);
                            atomicExch(A.abort_flag, 1);
                        }
                        break;  // the grid barrier below sees the flag; this warp's copies are drained at exit
                    }
                    const int c0 = c_seg * seg;
                    const int nch = min(seg, C - c0) >> 3;
                    const uint8_t* stg = ring + (size_t)c_st * cap_b;
                    WidenCtx wc;
                    wc.esc_idx = op.esc_idx, wc.esc_val = op.esc_val, wc.e0 = 0, wc.e1 = 0, wc.srow = nullptr, wc.bn = 8;
                    wc.table[0] = table[0], wc.table[1] = table[1], wc.table[2] = table[2], wc.table[3] = table[3];
                    if (fmt == F_BF16) {
                        consume_stage<M, F_BF16, true>(acc, stg, seg, nch, c0, c_row, C, xs, wc, lane);
                    } else {
                        if (op.esc_row != nullptr) {
                            wc.e0 = __ldg(op.esc_row + c_row);
                            wc.e1 = __ldg(op.esc_row + c_row + 1);
                        }
                        consume_stage<M, F_P12, true>(acc, stg, seg, nch, c0, c_row, C, xs, wc, lane);
                    }
                    __syncwarp();
                    --inflight;
                    if (++c_st == S) {
                        c_st = 0;
                        c_par ^= 1u;
                    }
                    issue_some(limit, limit_round);
                    if (c_seg == nseg - 1) {
#pragma unroll
                        for (int m = 0; m < M; ++m) {
                            const float s = warp_sum(acc[m]);
                            if (lane == 0) op.y[(size_t)m * R + c_row] = f2bf(s);
                            acc[m] = 0.f;
                        }
                        c_seg = 0;
                        c_row += NWS;
                    } else {
                        ++c_seg;
                    }
                }
                issue_some(limit, limit_round);  // a warp without rows here still runs its ring ahead
                STEP_BARRIER();
            } else if (kind == OP_ROPE) {
                const StepOp& op = ops[oi];
                RopeArgs ra;
                ra.rw = nullptr;
                ra.qkv = op.x, ra.wq = op.wq, ra.wk = op.wk, ra.cos_t = A.cos_t, ra.sin_t = A.sin_t;
                ra.n0p = A.n0, ra.depth = A.depth, ra.tbl = A.tbl, ra.K = op.K, ra.V = op.V, ra.qo = op.q;
                ra.eps = op.eps, ra.T = A.T, ra.Hq = A.Hq, ra.Hk = A.Hk, ra.centered = op.centered;
                ra.hs = A.hs, ra.rs = A.rs, ra.cap = A.cap;
                const int heads = A.Hq + 2 * A.Hk, items = heads * A.T;
                for (int it = blockIdx.x * NWS + warp; it < items; it += gridDim.x * NWS)
                    rope_item<D, true>(ra, it % heads, it / heads, lane);
                STEP_BARRIER();
            } else if (kind == OP_ATTN) {
                const StepOp& op = ops[oi];
                AttnArgs aa;
                aa.rw = nullptr;
                aa.q = op.q, aa.K = op.K, aa.V = op.V, aa.out = op.att, aa.n0p = A.n0, aa.par = A.par, aa.tbl = A.tbl;
                aa.sinks = A.sinks, aa.part_m = A.part_m, aa.part_l = A.part_l, aa.part_acc = A.part_acc, aa.cnt = A.cnt;
                aa.scale = op.scale, aa.T = A.T, aa.Hq = A.Hq, aa.Hk = A.Hk, aa.win = op.win, aa.cap = A.cap;
                aa.hs = A.hs, aa.rs = A.rs;
                const int Sg = (A.cap + GK - 1) / GK, items = A.T * A.Hk * Sg;
                for (int it = blockIdx.x; it < items; it += gridDim.x)
                    attn_item<D, G, true>(aa, it % Sg, (it / Sg) % A.Hk, it / (Sg * A.Hk), attn_scratch);
                STEP_BARRIER();
            } else if (kind == OP_PICK) {
                // lowest-index argmax of every row: each CTA folds its slice into a 64-bit key, one atomicMax a row
                const int V = A.vocab;
                for (int t = 0; t < A.T; ++t) {
                    const bf16* row = A.logits + (size_t)t * V;
                    unsigned long long best = 0ull;
                    const bool vec = (V & 7) == 0;
                    const int nvec = vec ? V >> 3 : 0;
                    for (int c = blockIdx.x * NTS + threadIdx.x; c < nvec; c += gridDim.x * NTS) {
                        const uint4 v = ldcg16(reinterpret_cast<const uint4*>(row) + c);
                        const uint32_t wds[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const unsigned long long a = pick_key64(bf_lo(wds[k]), c * 8 + 2 * k);
                            const unsigned long long b = pick_key64(bf_hi(wds[k]), c * 8 + 2 * k + 1);
                            best = best > a ? best : a;
                            best = best > b ? best : b;
                        }
                    }
                    if (!vec)
                        for (int i = blockIdx.x * NTS + threadIdx.x; i < V; i += gridDim.x * NTS) {
                            const unsigned short u = __ldcg(reinterpret_cast<const unsigned short*>(row + i));
                            const unsigned long long a = pick_key64(__uint_as_float((uint32_t)u << 16), i);
                            best = best > a ? best : a;
                        }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
                        best = best > other ? best : other;
                    }
                    if (lane == 0) s_best[warp] = best;
                    __syncthreads();
                    if (threadIdx.x == 0) {
                        for (int w = 1; w < NWS; ++w) best = best > s_best[w] ? best : s_best[w];
                        atomicMax(A.pick_keys + t, best);
                    }
                    __syncthreads();
                }
                STEP_BARRIER();
                if (!alive) break;
                if (blockIdx.x == 0 && threadIdx.x == 0) {
                    for (int t = 0; t < A.T; ++t) {
                        const unsigned long long k = atomicExch(A.pick_keys + t, 0ull);
                        A.ids[t] = (long long)(0xffffffffu - (unsigned)(k & 0xffffffffull));
                    }
                }
            }
        }
        if (!alive) break;
        // the step's end: the cache grows, the token goes out (btb_publish, native/cuda/btb_kernels.cu:455-465)
        if (blockIdx.x == 0 && threadIdx.x == 0) {
            const int n = __ldcg(A.n0) + A.advance;
            *A.n0 = n;
            if (A.tok_out != nullptr) A.tok_out[step] = A.ids[0];
            if (A.pin_tok != nullptr) {
                *A.pin_tok = A.ids[0];
                unsigned long long ts;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ts));
                *A.pin_ts = (long long)ts;
                __threadfence_system();
                *A.pin_n0 = n;
            }
        }
        if (step + 1 < A.steps) {
            const bool tracing = false;
            const int oi = 0;
            (void)oi;
            STEP_BARRIER();  // the next step reads ids and n0
        }
    }
    drain();
#undef STEP_BARRIER
}

template <int M, int D, int G>
int launch_step(const StepArgs& a, int smem, cudaStream_t stream) {
    auto kern = step_kernel<M, D, G>;
    static bool allowed[64];
    int rc = b2_allow_smem(reinterpret_cast<const void*>(kern), allowed);
    if (rc) return rc;
    // every CTA must be resident for the grid barrier: one a SM, checked, and a cooperative launch
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, NTS, smem) != cudaSuccess || per_sm < 1) {
        (void)cudaGetLastError();
        return B2_ERR_CUDA;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(b2_sm_count());
    cfg.blockDim = dim3(NTS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;
    at[0].val.cooperative = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    void* params[1] = {const_cast<StepArgs*>(&a)};
    if (cudaLaunchKernelExC(&cfg, reinterpret_cast<const void*>(kern), params) != cudaSuccess) {
        (void)cudaGetLastError();
        return B2_ERR_CUDA;
    }
    return B2_OK;
}

}  // namespace

extern "C" size_t btb_b200_step_op_bytes(void) { return sizeof(StepOp); }
extern "C" size_t btb_b200_step_args_bytes(void) { return sizeof(StepArgs); }

// `args`: a HOST StepArgs image (btb_b200/step.py builds it); M rows padded, D head dim, G query heads a kv head.
extern "C" int btb_b200_step(const void* args, int M, int D, int G, void* stream) {
    if (args == nullptr) return B2_ERR_NULL;
    StepArgs a;
    memcpy(&a, args, sizeof a);
    if (a.ops == nullptr || a.n0 == nullptr || a.depth == nullptr || a.par == nullptr || a.bar == nullptr ||
        a.abort_flag == nullptr || a.cos_t == nullptr || a.sin_t == nullptr || a.ids == nullptr)
        return B2_ERR_NULL;
    if (a.n_ops <= 0 || a.T <= 0 || a.T > M || a.steps <= 0 || a.S < 2 || a.stage_cap < 512 || (a.stage_cap & 127) ||
        (a.front_bytes & 127) || (a.steps > 1 && (a.T != 1 || !a.pick)))
        return B2_ERR_DOMAIN;
    const int smem = a.front_bytes + NWS * a.S * a.stage_cap + NWS * a.S * 8;
    if (smem > 226 * 1024) return B2_ERR_DOMAIN;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (D == 128 && G == 4) {
        if ((size_t)a.front_bytes < sizeof(AttnSmem<128, 4>)) return B2_ERR_DOMAIN;
        if (M == 1) return launch_step<1, 128, 4>(a, smem, s);
        if (M == 2) return launch_step<2, 128, 4>(a, smem, s);
    } else if (D == 128 && G == 8) {
        if ((size_t)a.front_bytes < sizeof(AttnSmem<128, 8>)) return B2_ERR_DOMAIN;
        if (M == 1) return launch_step<1, 128, 8>(a, smem, s);
        if (M == 2) return launch_step<2, 128, 8>(a, smem, s);
    } else if (D == 128 && G == 2) {
        if ((size_t)a.front_bytes < sizeof(AttnSmem<128, 2>)) return B2_ERR_DOMAIN;
        if (M == 1) return launch_step<1, 128, 2>(a, smem, s);
        if (M == 2) return launch_step<2, 128, 2>(a, smem, s);
    }
    return B2_ERR_DOMAIN;
}
