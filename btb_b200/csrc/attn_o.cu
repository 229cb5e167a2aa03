// The decode step's attention row and the output projection that reads it, as ONE launch.
//
// Separately they are two dependent kernels: the projection's 21 MB of weights (Qwen3-4B) cannot start moving until
// the attention - a latency-bound kernel that keeps a handful of SMs busy for microseconds and the memory system idle
// - has finished and a kernel boundary has passed. Here every CTA first fills its ring with its rows of the
// projection's weights (they depend on nothing), then the grid's CTAs share out the attention's blocks
// (attn_step_item: q/k-norm, RoPE, cache write, attention), meet at one bounded grid barrier, stage the attention's
// output and multiply: the weights stream while the attention runs, and one kernel boundary is gone. The arithmetic
// is the two kernels' (the same device functions), so the bits are theirs.
//
// The launch is cooperative (every CTA must be resident for the barrier to pass); the wait is bounded like every wait
// here: a CTA that gives up records ERR_TIMEOUT, lets its copies land and leaves.
#include "btb_b200_internal.h"
#include "gemv_core.cuh"
#include "attn_core.cuh"

B2_DEFINE_STATUS(attno)

namespace {

constexpr int NWO = NWA;  // sixteen warps: what the attention's tiles need

struct AttnOArgs {
    AttnArgs a;
    RopeArgs r;
    const uint8_t* w;  // the projection [R, C] bf16
    bf16* y;           // [1, R]
    int R, C, seg, stages, evict_first;
    int S;             // key groups of the cache
    unsigned* bar;     // [2] arrivals and generation, zero before the first launch
    int attn_bytes;    // the attention's shared memory (the front region)
};

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

constexpr int SPLIT_ROWS_O = 4096;  // as attn_step: under this many cached rows a block a query head
#define ATTNO_SPIN_LIMIT (1u << 22)

template <int D, int G>
__global__ void __launch_bounds__(NWO * 32, 1) attn_o_step(const AttnOArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_ok;
    const int R = A.R, C = A.C, seg = A.seg, S = A.stages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int nw = NWO;
    const int nseg = (C + seg - 1) / seg;
    // shared memory: [attention scratch][x: C bf16][rings][barriers]
    const int xbytes = (C * 2 + 127) & ~127;
    const int sbytes = (seg * 2 + 127) & ~127;
    uint8_t* attn_scratch = smem;
    bf16* xs = reinterpret_cast<bf16*>(smem + A.attn_bytes);
    uint8_t* ring = smem + A.attn_bytes + xbytes + (size_t)warp * S * sbytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + A.attn_bytes + xbytes + (size_t)nw * S * sbytes) + warp * S;

    const int base = R / gridDim.x, rem = R % gridDim.x;
    const int r0 = blockIdx.x * base + min((int)blockIdx.x, rem);
    const int cnt = base + ((int)blockIdx.x < rem ? 1 : 0);
    const int my_rows = cnt > warp ? (cnt - warp + nw - 1) / nw : 0;
    const int n_items = my_rows * nseg;

    if (lane == 0) {
        for (int s = 0; s < S; ++s) mbar_init(smem_u32(bars + s), 1);
        mbar_fence_init();
    }
    __syncwarp();
    const uint64_t pol = A.evict_first ? l2_evict_first_policy() : 0;
    int p_row = r0 + warp, p_seg = 0, p_st = 0, issued = 0;
    auto issue_next = [&]() {
        const int c0 = p_seg * seg;
        const int n = min(seg, C - c0);
        if (lane == 0) {
            const uint32_t bar = smem_u32(bars + p_st);
            const uint32_t dst = smem_u32(ring + (size_t)p_st * sbytes);
            const uint8_t* src = A.w + ((size_t)p_row * C + c0) * 2;
            mbar_expect_tx(bar, n * 2);
            if (A.evict_first) bulk_g2s_hint(dst, src, n * 2, bar, pol);
            else bulk_g2s(dst, src, n * 2, bar);
        }
        ++issued;
        if (++p_st == S) p_st = 0;
        if (++p_seg == nseg) {
            p_seg = 0;
            p_row += nw;
        }
    };
    {
        const int first = min(S, n_items);
        for (int i = 0; i < first; ++i) issue_next();  // the projection's weights are on their way
    }
    pdl_launch_dependents();
    pdl_wait();  // qkv is the kernel's before this one

    // ---- the attention's blocks, shared out over the grid ------------------------------------------------------
    const unsigned gen = ld_acquire_u32(A.bar + 1);  // this launch's generation, read before anyone can finish it
    {
        const int Hk = A.a.Hk;
        const bool split = G > 1 && *A.a.n0p < SPLIT_ROWS_O;
        const int zs = split ? G : 1;
        const int items = A.S * Hk * zs;
        for (int it = blockIdx.x; it < items; it += gridDim.x) {
            const int z = it % zs, g = (it / zs) % Hk, grp = it / (zs * Hk);
            __syncthreads();  // the block's previous item is done with the scratch
            if (split) attn_step_item<D, 1, G, false>(A.a, A.r, grp, g, z, attn_scratch);
            else attn_step_item<D, G, G, false>(A.a, A.r, grp, g, 0, attn_scratch);
        }
    }
    // ---- every block's share of the attention is written: one barrier over the grid ------------------------------
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        int ok = 1;
        if (atomicAdd(A.bar, 1u) == gridDim.x - 1) {
            atomicExch(A.bar, 0u);  // the last to arrive opens the next generation
            __threadfence();
            atomicAdd(A.bar + 1, 1u);
        } else {
            unsigned it = 0;
            while (ld_acquire_u32(A.bar + 1) == gen) {
                if (++it > ATTNO_SPIN_LIMIT) {
                    ok = 0;
                    break;
                }
                __nanosleep(64);
            }
        }
        if (!ok) b2_fail(B2_ERR_TIMEOUT);
        __threadfence();
        s_ok = ok;
    }
    __syncthreads();
    bool ok = s_ok != 0;

    float acc[1] = {0.f};
    int c_row = r0 + warp, c_seg = 0, c_st = 0;
    uint32_t c_par = 0;
    int i = 0;
    if (ok) {
        stage_x_copy<1, NWO * 32>(xs, A.a.out, C);  // L2-coherent loads: other SMs wrote it in this launch
        __syncthreads();
        for (; i < n_items; ++i) {
            if (!mbar_wait_bounded(smem_u32(bars + c_st), c_par)) {
                ok = false;
                if (lane == 0) b2_fail(B2_ERR_TIMEOUT);
                break;
            }
            const int row = c_row;
            const int c0 = c_seg * seg;
            const int nch = min(seg, C - c0) >> 3;
            const uint8_t* stg = ring + (size_t)c_st * sbytes;
            WidenCtx wc;
            wc.esc_idx = nullptr, wc.esc_val = nullptr, wc.e0 = 0, wc.e1 = 0, wc.srow = nullptr, wc.bn = 8;
            wc.table[0] = wc.table[1] = wc.table[2] = wc.table[3] = 0u;
            consume_stage<1, F_BF16, true>(acc, stg, seg, nch, c0, row, C, xs, wc, lane);
            __syncwarp();
            if (issued < n_items) issue_next();
            if (c_seg == nseg - 1) {
                const float s = warp_sum(acc[0]);
                if (lane == 0) A.y[row] = f2bf(s);
                acc[0] = 0.f;
                c_seg = 0;
                c_row += nw;
            } else {
                ++c_seg;
            }
            if (++c_st == S) {
                c_st = 0;
                c_par ^= 1u;
            }
        }
    }
    if (!ok) {
        // gave up: the copies still in flight land (bounded) before the shared memory goes
        for (int j = i; j < issued; ++j) {
            mbar_wait_bounded(smem_u32(bars + c_st), c_par);
            if (++c_st == S) {
                c_st = 0;
                c_par ^= 1u;
            }
        }
    }
}

template <int D, int G>
int launch_attn_o(AttnOArgs& a, cudaStream_t stream) {
    auto kern = attn_o_step<D, G>;
    static bool allowed[64];
    int rc = b2_allow_smem(reinterpret_cast<const void*>(kern), allowed);
    if (rc) return rc;
    const B2Tuning& t = b2_tuning();
    a.attn_bytes = (int)((sizeof(AttnSmem<D, G>) + 127) & ~(size_t)127);
    const int xbytes = (a.C * 2 + 127) & ~127;
    // the ring takes what is left: whole rows a warp if they fit (the weights then all arrive during the attention)
    const int budget = 224 * 1024 - a.attn_bytes - xbytes;
    int max_seg_el = max(256, (t.seg_bytes / 2) & ~255);
    const int nseg = (a.C + max_seg_el - 1) / max_seg_el;
    a.seg = ((a.C + nseg - 1) / nseg + 255) & ~255;
    const int sb = (a.seg * 2 + 127) & ~127;
    a.stages = max(2, min(8, budget / (NWO * (sb + 8))));
    const int smem = a.attn_bytes + xbytes + NWO * a.stages * (sb + 8);
    if (smem > 226 * 1024) return B2_ERR_DOMAIN;
    a.evict_first = t.evict_first;
    const int grid = b2_sm_count();
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NWO * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeCooperative;
    at[0].val.cooperative = 1;
    int n_at = 1;
    if (t.pdl & 1) {
        at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[1].val.programmaticStreamSerializationAllowed = 1;
        n_at = 2;
    }
    cfg.attrs = at;
    cfg.numAttrs = n_at;
    void* params[1] = {&a};
    if (cudaLaunchKernelExC(&cfg, reinterpret_cast<const void*>(kern), params) != cudaSuccess) {
        (void)cudaGetLastError();
        return B2_ERR_CUDA;
    }
    return B2_OK;
}

template <int D>
int launch_attn_o_g(int G, AttnOArgs& a, cudaStream_t s) {
    switch (G) {
        case 1: return launch_attn_o<D, 1>(a, s);
        case 2: return launch_attn_o<D, 2>(a, s);
        case 4: return launch_attn_o<D, 4>(a, s);
        case 8: return launch_attn_o<D, 8>(a, s);
        default: return B2_ERR_DOMAIN;
    }
}

}  // namespace

extern "C" int btb_b200_attn_o_step(const void* qkv, const void* wq, const void* wk, float eps, const void* cos_t,
                                    const void* sin_t, const void* n0p, const void* depth, void* K, void* V, void* q,
                                    void* att, int Hq, int Hk, int D, long long hs, long long rs, int centered,
                                    float scale, void* part_m, void* part_l, void* part_acc, void* cnt, int win,
                                    const void* sinks, int cap, const void* w_o, void* y, int R, void* bar,
                                    void* stream) {
    if (!qkv || !cos_t || !sin_t || !n0p || !depth || !K || !V || !q || !att || !part_m || !part_l || !part_acc || !cnt ||
        !w_o || !y || !bar)
        return B2_ERR_NULL;
    if (Hk <= 0 || Hq <= 0 || Hq % Hk || (Hq / Hk != 1 && Hq / Hk != 2 && Hq / Hk != 4 && Hq / Hk != 8) || cap <= 0 ||
        !(scale == scale) || R <= 0)
        return B2_ERR_DOMAIN;
    if ((hs & 7) || (rs & 7) || (reinterpret_cast<uintptr_t>(K) & 15) || (reinterpret_cast<uintptr_t>(V) & 15))
        return B2_ERR_DOMAIN;
    if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(wq) | reinterpret_cast<uintptr_t>(wk) |
         reinterpret_cast<uintptr_t>(cos_t) | reinterpret_cast<uintptr_t>(sin_t) | reinterpret_cast<uintptr_t>(q) |
         reinterpret_cast<uintptr_t>(att) | reinterpret_cast<uintptr_t>(w_o)) & 15)
        return B2_ERR_DOMAIN;
    if (reinterpret_cast<uintptr_t>(bar) & 7) return B2_ERR_DOMAIN;
    AttnOArgs A{};
    AttnArgs& a = A.a;
    a.q = static_cast<const bf16*>(q), a.K = static_cast<const bf16*>(K), a.V = static_cast<const bf16*>(V);
    a.out = static_cast<bf16*>(att), a.n0p = static_cast<const int*>(n0p), a.par = nullptr, a.tbl = nullptr;
    a.sinks = static_cast<const float*>(sinks);
    a.part_m = static_cast<float*>(part_m), a.part_l = static_cast<float*>(part_l);
    a.part_acc = static_cast<float*>(part_acc), a.cnt = static_cast<int*>(cnt);
    a.scale = scale, a.T = 1, a.Hq = Hq, a.Hk = Hk, a.win = win, a.cap = cap, a.hs = hs, a.rs = rs;
    A.r = RopeArgs{static_cast<const bf16*>(qkv), static_cast<const bf16*>(wq), static_cast<const bf16*>(wk),
                   static_cast<const bf16*>(cos_t), static_cast<const bf16*>(sin_t), static_cast<const int*>(n0p),
                   static_cast<const int*>(depth), nullptr, nullptr, static_cast<bf16*>(K), static_cast<bf16*>(V),
                   static_cast<bf16*>(q), eps, 1, Hq, Hk, centered, hs, rs, cap};
    A.w = static_cast<const uint8_t*>(w_o), A.y = static_cast<bf16*>(y), A.R = R, A.C = Hq * D;
    A.S = (cap + GK - 1) / GK;
    A.bar = static_cast<unsigned*>(bar);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (D) {
        case 64: return launch_attn_o_g<64>(Hq / Hk, A, s);
        case 128: return launch_attn_o_g<128>(Hq / Hk, A, s);
        default: return B2_ERR_DOMAIN;
    }
}
