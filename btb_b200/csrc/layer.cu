// The step's small kernels: embedding gather, residual + RMSNorm, q/k norm + RoPE + cache write, SwiGLU product,
// greedy pick, the token's handoff to pinned host memory. Each is the arithmetic of the reference's kernel of the same
// name (native/cuda/btb_kernels.cu of btb, lines cited per kernel): same per-element operations, same reduction
// trees, so the bits are the reference's; what changes is that every kernel waits on the grid dependency itself
// (programmatic dependent launch) and nothing traps.
#include "common.cuh"
#include "btb_b200_internal.h"
#include "attn_core.cuh"

B2_DEFINE_STATUS(layer)

namespace {

// ---- embedding gather: h[t, :] = table[ids[t], :] (btb/engine/cuda.py:2227-2232) -----------------------------------
struct EmbedArgs {
    const bf16* table;
    const long long* ids;
    bf16* h;
    int T, H, V;
};
__global__ void __launch_bounds__(256) embed_rows(const EmbedArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    long long id = A.ids[t];
    if (id < 0 || id >= A.V) {  // never read outside the table: record and clamp
        if (threadIdx.x == 0) b2_fail(B2_ERR_DOMAIN);
        id = 0;
    }
    const uint4* src = reinterpret_cast<const uint4*>(A.table + (size_t)id * A.H);
    uint4* dst = reinterpret_cast<uint4*>(A.h + (size_t)t * A.H);
    for (int i = threadIdx.x; i < A.H / 8; i += 256) dst[i] = __ldg(src + i);
}

// ---- residual + RMSNorm (btb_kernels.cu:365-393) -------------------------------------------------------------------
// thread i of 256 sums the squares of elements i, i + 256, .. in order, then the fixed 256 -> 1 tree.
struct NormArgs {
    bf16* h;
    const bf16* y;
    const bf16* w;
    bf16* x;
    float* xf;  // the same values as f32, or null (the MoE block's router and experts read x widened)
    float eps;
    int H, centered;
};
// One block a row. The arithmetic is the reference's: hv = bf16(h + y); thread i of 256 sums hv^2 over i, i + 256, ..;
// the 256 -> 1 tree red[t] += red[t + st], st = 128 .. 1 (here with the same pairs in the same order on one warp);
// x = bf16(hv * rsqrt(ss / H + eps) * w). The row is read once, as 16-byte runs when H allows, and kept in shared
// memory (dynamic: H floats) between the two passes; the norm's weights are on their way before the reduction.
__global__ void __launch_bounds__(256) add_rmsnorm(const NormArgs A) {
    extern __shared__ __align__(16) float hsm[];
    __shared__ float red[256];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, tid = threadIdx.x, H = A.H;
    bf16* hr = A.h + (size_t)t * H;
    const bf16* yr = A.y == nullptr ? nullptr : A.y + (size_t)t * H;
    bf16* xr = A.x + (size_t)t * H;
    const bool vec = (H & 7) == 0 && ((reinterpret_cast<uintptr_t>(A.h) | reinterpret_cast<uintptr_t>(A.y) |
                                       reinterpret_cast<uintptr_t>(A.w) | reinterpret_cast<uintptr_t>(A.x)) & 15) == 0;
    if (vec) {
        const int cv = H >> 3;
        for (int i = tid; i < cv; i += 256) {
            const uint4 hv = *(reinterpret_cast<const uint4*>(hr) + i);
            uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w};
            if (yr != nullptr) {
                const uint4 yv = *(reinterpret_cast<const uint4*>(yr) + i);
                const uint32_t yw[4] = {yv.x, yv.y, yv.z, yv.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const __nv_bfloat162 pr = __floats2bfloat162_rn(bf_lo(hw[k]) + bf_lo(yw[k]), bf_hi(hw[k]) + bf_hi(yw[k]));
                    hw[k] = *reinterpret_cast<const uint32_t*>(&pr);
                }
                *(reinterpret_cast<uint4*>(hr) + i) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
            }
            reinterpret_cast<float4*>(hsm)[2 * i] = make_float4(bf_lo(hw[0]), bf_hi(hw[0]), bf_lo(hw[1]), bf_hi(hw[1]));
            reinterpret_cast<float4*>(hsm)[2 * i + 1] = make_float4(bf_lo(hw[2]), bf_hi(hw[2]), bf_lo(hw[3]), bf_hi(hw[3]));
        }
    } else {
        for (int i = tid; i < H; i += 256) {
            float hv = bf2f(hr[i]);
            if (yr != nullptr) {
                hv = bfround(hv + bf2f(yr[i]));
                hr[i] = f2bf(hv);
            }
            hsm[i] = hv;
        }
    }
    __syncthreads();
    float ss = 0.f;
    for (int i = tid; i < H; i += 256) ss = fmaf(hsm[i], hsm[i], ss);
    red[tid] = ss;
    __syncthreads();
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
    const float rstd = rsqrtf(red[0] / (float)H + A.eps);
    float* xfr = A.xf == nullptr ? nullptr : A.xf + (size_t)t * H;
    if (vec) {
        const int cv = H >> 3;
        for (int i = tid; i < cv; i += 256) {
            const uint4 wv4 = __ldg(reinterpret_cast<const uint4*>(A.w) + i);
            const uint32_t ww[4] = {wv4.x, wv4.y, wv4.z, wv4.w};
            const float4 ha = reinterpret_cast<const float4*>(hsm)[2 * i], hb = reinterpret_cast<const float4*>(hsm)[2 * i + 1];
            const float hv8[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
            uint32_t o[4];
            float of[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float w0 = bf_lo(ww[k]), w1 = bf_hi(ww[k]);
                const bf16 a = f2bf(hv8[2 * k] * rstd * (A.centered ? 1.f + w0 : w0));
                const bf16 b = f2bf(hv8[2 * k + 1] * rstd * (A.centered ? 1.f + w1 : w1));
                o[k] = (uint32_t)__bfloat16_as_ushort(a) | ((uint32_t)__bfloat16_as_ushort(b) << 16);
                of[2 * k] = bf2f(a), of[2 * k + 1] = bf2f(b);
            }
            *(reinterpret_cast<uint4*>(xr) + i) = make_uint4(o[0], o[1], o[2], o[3]);
            if (xfr != nullptr) {
                reinterpret_cast<float4*>(xfr)[2 * i] = make_float4(of[0], of[1], of[2], of[3]);
                reinterpret_cast<float4*>(xfr)[2 * i + 1] = make_float4(of[4], of[5], of[6], of[7]);
            }
        }
    } else {
        for (int i = tid; i < H; i += 256) {
            const float wv = bf2f(A.w[i]);
            const bf16 o = f2bf(hsm[i] * rstd * (A.centered ? 1.f + wv : wv));
            xr[i] = o;
            if (xfr != nullptr) xfr[i] = bf2f(o);
        }
    }
}

// ---- act(g) * up over a [T, 2I] block (btb_kernels.cu:470-480) -----------------------------------------------------
struct ActArgs {
    const bf16* gu;
    bf16* m;
    int T, I;
};
__global__ void __launch_bounds__(256) silu_mul(const ActArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t n = (size_t)A.T * A.I;
    for (size_t k = (size_t)blockIdx.x * 256 + threadIdx.x; k < n; k += (size_t)gridDim.x * 256) {
        const size_t t = k / A.I, i = k - t * A.I;
        const float g = bf2f(A.gu[t * (2 * (size_t)A.I) + i]);
        const float u = bf2f(A.gu[t * (2 * (size_t)A.I) + A.I + i]);
        const float s = bfround(g / (1.f + expf(-g)));
        A.m[k] = f2bf(s * u);
    }
}

template <int D>
__global__ void __launch_bounds__(32) norm_rope_kv(const RopeArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    rope_item<D, false>(A, blockIdx.x, blockIdx.y, threadIdx.x);
}

// ---- greedy pick: lowest-index argmax over a bf16 logits row (btb/engine/cuda.py:2237; ties as
// native/src/sample.rs:57-67) --------------------------------------------------------------------------------------
// Every block folds its slice into one 64-bit key - the value's ordered bits above the complemented index - and
// atomicMax'es it into the row's slot of `scratch`; the last block to arrive writes the token and clears the slot
// and the counter for the next launch. scratch: T u64 keys then T u32 counters, zero before the first launch.
struct ArgmaxArgs {
    const bf16* logits;
    unsigned long long* keys;
    unsigned int* counts;
    long long* out;
    int V;
};
__device__ __forceinline__ unsigned long long pick_key(float v, int idx) {
    const unsigned b = __float_as_uint(v);
    const unsigned u = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned long long)(0xffffffffu - (unsigned)idx);
}
__global__ void __launch_bounds__(256) argmax_rows(const ArgmaxArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.y;
    const bf16* row = A.logits + (size_t)t * A.V;
    unsigned long long best = 0ull;
    // 16-byte loads only where every row starts on 16 bytes: the vocabulary a multiple of 8 and the base aligned
    const bool vec = (A.V & 7) == 0 && (reinterpret_cast<uintptr_t>(A.logits) & 15) == 0;
    const int nvec = vec ? A.V >> 3 : 0;
    for (int c = blockIdx.x * 256 + threadIdx.x; c < nvec; c += gridDim.x * 256) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(row) + c);
        const uint32_t wds[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const unsigned long long a = pick_key(bf_lo(wds[k]), c * 8 + 2 * k);
            const unsigned long long b = pick_key(bf_hi(wds[k]), c * 8 + 2 * k + 1);
            best = best > a ? best : a;
            best = best > b ? best : b;
        }
    }
    if (!vec)  // element by element
        for (int i = blockIdx.x * 256 + threadIdx.x; i < A.V; i += gridDim.x * 256) {
            const unsigned long long a = pick_key(bf2f(row[i]), i);
            best = best > a ? best : a;
        }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = best > other ? best : other;
    }
    __shared__ unsigned long long wbest[8];
    __shared__ int last;
    if ((threadIdx.x & 31) == 0) wbest[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) best = best > wbest[w] ? best : wbest[w];
        atomicMax(A.keys + t, best);
        __threadfence();
        last = atomicAdd(A.counts + t, 1u) == gridDim.x - 1;
        if (last) {
            __threadfence();
            const unsigned long long k = atomicExch(A.keys + t, 0ull);
            A.out[t] = (long long)(0xffffffffu - (unsigned)(k & 0xffffffffull));
            A.counts[t] = 0u;
        }
    }
}

// ---- the step's handoff (btb_kernels.cu:455-465): token and device clock, a system fence, then the length -------
struct PublishArgs {
    int* n0;
    const long long* ids;
    long long* out_tok;
    int* out_n0;
    long long* out_ts;
    int advance;  // n0 += advance before it is published (the graph advances itself)
};
__global__ void publish_step(const PublishArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        const int n = *A.n0 + A.advance;
        *A.n0 = n;
        if (A.out_tok != nullptr) {
            *A.out_tok = *A.ids;
            unsigned long long ts;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ts));
            *A.out_ts = (long long)ts;
            __threadfence_system();
            *A.out_n0 = n;
        }
    }
}

// ---- the accepted branch's rows gathered to the cache's front (btb/engine/cuda.py:3563-3575 `ad`) -------------------
// A verify pass wrote its T rows at slots n0 .. n0 + T - 1; the kept path's node path[j] moves to slot n0 + j. Nodes
// are numbered parents first, so path[j] >= j and the moves run in ascending j: a row is read before its slot is
// written. One block per (layer, K or V); the block's threads copy a row, then the next.
struct CommitArgs {
    bf16* K;
    bf16* V;
    const int* n0p;
    const int* path;
    const int* tbl;
    long long layer_stride, rs;
    int len, row_el, cap;
};
__global__ void __launch_bounds__(256) kv_commit(const CommitArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    bf16* base = (blockIdx.y == 0 ? A.K : A.V) + (size_t)blockIdx.x * A.layer_stride;
    const int n0 = *A.n0p;
    for (int j = 0; j < A.len; ++j) {
        const int p = A.path[j];
        if (p < j || n0 + p >= A.cap) {  // not a parents-first path, or past the cache: refuse, move nothing more
            if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) b2_fail(B2_ERR_DOMAIN);
            return;
        }
        if (p != j) {
            int src = n0 + p, dst = n0 + j;
            if (A.tbl != nullptr) src = A.tbl[src], dst = A.tbl[dst];
            const uint4* s4 = reinterpret_cast<const uint4*>(base + (size_t)src * A.rs);
            uint4* d4 = reinterpret_cast<uint4*>(base + (size_t)dst * A.rs);
            for (int i = threadIdx.x; i < A.row_el / 8; i += 256) d4[i] = s4[i];
        }
        __syncthreads();
    }
}

}  // namespace

// ---- C-ABI ------------------------------------------------------------------------------------------------------------

extern "C" int btb_b200_embed(const void* table, const void* ids, void* h, int T, int H, int V, void* stream) {
    if (!table || !ids || !h) return B2_ERR_NULL;
    if (T <= 0 || H <= 0 || (H & 7) || V <= 0) return B2_ERR_DOMAIN;
    if ((reinterpret_cast<uintptr_t>(table) & 15) || (reinterpret_cast<uintptr_t>(h) & 15)) return B2_ERR_DOMAIN;
    EmbedArgs a{static_cast<const bf16*>(table), static_cast<const long long*>(ids), static_cast<bf16*>(h), T, H, V};
    return b2_launch((const void*)embed_rows, dim3(T), dim3(256), 0, static_cast<cudaStream_t>(stream), a);
}

static int add_rmsnorm_launch(void* h, const void* y, const void* w, float eps, void* x, void* xf, int T, int H,
                              int centered, void* stream) {
    if (!h || !w || !x) return B2_ERR_NULL;
    if (T <= 0 || H <= 0 || !(eps == eps)) return B2_ERR_DOMAIN;
    if ((size_t)H * 4 > 200 * 1024) return B2_ERR_DOMAIN;  // the row is held in shared memory as f32
    if (xf != nullptr && (reinterpret_cast<uintptr_t>(xf) & 15)) return B2_ERR_DOMAIN;
    NormArgs a{static_cast<bf16*>(h), static_cast<const bf16*>(y), static_cast<const bf16*>(w), static_cast<bf16*>(x),
               static_cast<float*>(xf), eps, H, centered};
    static bool allowed[64];
    if (const int rc = b2_allow_smem((const void*)add_rmsnorm, allowed)) return rc;
    return b2_launch((const void*)add_rmsnorm, dim3(T), dim3(256), (size_t)H * 4, static_cast<cudaStream_t>(stream), a);
}

extern "C" int btb_b200_add_rmsnorm(void* h, const void* y, const void* w, float eps, void* x, int T, int H,
                                    int centered, void* stream) {
    return add_rmsnorm_launch(h, y, w, eps, x, nullptr, T, H, centered, stream);
}

extern "C" int btb_b200_add_rmsnorm_wide(void* h, const void* y, const void* w, float eps, void* x, void* xf, int T, int H,
                                         int centered, void* stream) {
    if (!xf) return B2_ERR_NULL;
    return add_rmsnorm_launch(h, y, w, eps, x, xf, T, H, centered, stream);
}

extern "C" int btb_b200_silu_mul(const void* gu, void* m, int T, int I, void* stream) {
    if (!gu || !m) return B2_ERR_NULL;
    if (T <= 0 || I <= 0) return B2_ERR_DOMAIN;
    ActArgs a{static_cast<const bf16*>(gu), static_cast<bf16*>(m), T, I};
    const long long n = (long long)T * I;
    const int grid = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    return b2_launch((const void*)silu_mul, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), a);
}

static int norm_rope_kv_impl(const void* qkv, const void* wq, const void* wk, float eps, const void* cos_t,
                             const void* sin_t, const void* n0p, const void* depth, const void* rw, void* K, void* V,
                             void* q, int T, int Hq, int Hk, int D, long long hs, long long rs, int centered,
                             const void* tbl, int cap, void* stream) {
    if (!qkv || !cos_t || !sin_t || (!rw && (!n0p || !depth)) || !K || !V || !q) return B2_ERR_NULL;
    if (T <= 0 || Hq <= 0 || Hk <= 0 || cap <= 0) return B2_ERR_DOMAIN;
    // a lane reads its D/32 elements of a head, a norm weight or a table row as one load
    if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(wq) | reinterpret_cast<uintptr_t>(wk) |
         reinterpret_cast<uintptr_t>(cos_t) | reinterpret_cast<uintptr_t>(sin_t) | reinterpret_cast<uintptr_t>(q) |
         reinterpret_cast<uintptr_t>(K) | reinterpret_cast<uintptr_t>(V)) & 15)
        return B2_ERR_DOMAIN;
    if ((hs & 7) || (rs & 7)) return B2_ERR_DOMAIN;
    RopeArgs a{static_cast<const bf16*>(qkv), static_cast<const bf16*>(wq), static_cast<const bf16*>(wk),
               static_cast<const bf16*>(cos_t), static_cast<const bf16*>(sin_t), static_cast<const int*>(n0p),
               static_cast<const int*>(depth), static_cast<const int*>(tbl), static_cast<const int*>(rw),
               static_cast<bf16*>(K), static_cast<bf16*>(V), static_cast<bf16*>(q), eps, T, Hq, Hk, centered, hs, rs, cap};
    const dim3 grid(Hq + 2 * Hk, T);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (D) {
        case 64: return b2_launch((const void*)norm_rope_kv<64>, grid, dim3(32), 0, s, a);
        case 128: return b2_launch((const void*)norm_rope_kv<128>, grid, dim3(32), 0, s, a);
        case 256: return b2_launch((const void*)norm_rope_kv<256>, grid, dim3(32), 0, s, a);
        default: return B2_ERR_DOMAIN;
    }
}

extern "C" int btb_b200_norm_rope_kv(const void* qkv, const void* wq, const void* wk, float eps, const void* cos_t,
                                     const void* sin_t, const void* n0p, const void* depth, void* K, void* V, void* q,
                                     int T, int Hq, int Hk, int D, long long hs, long long rs, int centered,
                                     const void* tbl, int cap, void* stream) {
    return norm_rope_kv_impl(qkv, wq, wk, eps, cos_t, sin_t, n0p, depth, nullptr, K, V, q, T, Hq, Hk, D, hs, rs, centered,
                             tbl, cap, stream);
}

// the rows layout: row t a sequence of its own, its token at position len + step, written to its step's cache row
extern "C" int btb_b200_norm_rope_kv_rows(const void* qkv, const void* wq, const void* wk, float eps, const void* cos_t,
                                          const void* sin_t, const void* rw, void* K, void* V, void* q, int T, int Hq,
                                          int Hk, int D, long long hs, long long rs, int centered, int cap, void* stream) {
    if (!rw) return B2_ERR_NULL;
    return norm_rope_kv_impl(qkv, wq, wk, eps, cos_t, sin_t, nullptr, nullptr, rw, K, V, q, T, Hq, Hk, D, hs, rs, centered,
                             nullptr, cap, stream);
}

extern "C" int btb_b200_argmax_bf16(const void* logits, int T, int V, void* scratch, void* out, void* stream) {
    if (!logits || !scratch || !out) return B2_ERR_NULL;
    if (T <= 0 || V <= 0 || (reinterpret_cast<uintptr_t>(scratch) & 7)) return B2_ERR_DOMAIN;
    ArgmaxArgs a{static_cast<const bf16*>(logits), static_cast<unsigned long long*>(scratch),
                 reinterpret_cast<unsigned int*>(static_cast<unsigned long long*>(scratch) + T),
                 static_cast<long long*>(out), V};
    int blocks = (V / 8 + 255) / 256;
    blocks = blocks < 1 ? 1 : (blocks > 148 ? 148 : blocks);
    return b2_launch((const void*)argmax_rows, dim3(blocks, T), dim3(256), 0, static_cast<cudaStream_t>(stream), a);
}

extern "C" size_t btb_b200_argmax_scratch_bytes(int T) { return (size_t)T * 12 + 4; }

// ---- the greedy pick for callers that cannot allocate -----------------------------------------------------------------
// Some callers have no way to hand this library a scratch buffer: a host that got its whole device budget granted up
// front and may not ask the driver for more in the middle of a decode, or code that is already inside a stream capture,
// where cudaMalloc is not allowed. For them the pick's scratch (one 64-bit key and one arrival counter a row) lives in
// this array inside the library's own image. It costs every device that loads the library these few hundred bytes
// until the process exits.
#define B2_PICK_STATIC_ROWS 32
static __device__ __align__(256) unsigned char g_pick_static[B2_PICK_STATIC_ROWS * 12 + 4];

extern "C" int btb_b200_argmax_bf16_static(const void* logits, int T, int V, void* out, void* stream) {
    if (!logits || !out) return B2_ERR_NULL;
    if (T <= 0 || V <= 0) return B2_ERR_DOMAIN;
    if (T > B2_PICK_STATIC_ROWS) return B2_ERR_DOMAIN;  // the built-in scratch holds 32 rows, a pass's widest
    // In host code `g_pick_static` is only a handle: the array's device address has to be asked for, once per device,
    // with that device current. This happens on the first call on each device - make that call before any stream
    // capture starts.
    static void* addr[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B2_ERR_CUDA;
    if (addr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_pick_static) != cudaSuccess || p == nullptr) {
            (void)cudaGetLastError();
            return B2_ERR_CUDA;
        }
        addr[dev] = p;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // every call shares the one array and it keeps what the last call left: the keys and counters must start at zero
    if (cudaMemsetAsync(addr[dev], 0, (size_t)T * 12 + 4, s) != cudaSuccess) {
        (void)cudaGetLastError();
        return B2_ERR_CUDA;
    }
    return btb_b200_argmax_bf16(logits, T, V, addr[dev], out, stream);
}

extern "C" int btb_b200_kv_commit(void* K, void* V, long long layer_stride, int layers, const void* n0p, const void* path,
                                  int len, int row_el, long long rs, const void* tbl, int cap, void* stream) {
    if (!K || !V || !n0p || !path) return B2_ERR_NULL;
    if (layers <= 0 || len <= 0 || len > 32 || row_el <= 0 || (row_el & 7) || (rs & 7) || rs < row_el || cap <= 0 ||
        (reinterpret_cast<uintptr_t>(K) & 15) || (reinterpret_cast<uintptr_t>(V) & 15) || (layer_stride & 7))
        return B2_ERR_DOMAIN;
    CommitArgs a{static_cast<bf16*>(K), static_cast<bf16*>(V), static_cast<const int*>(n0p), static_cast<const int*>(path),
                 static_cast<const int*>(tbl), layer_stride, rs, len, row_el, cap};
    return b2_launch((const void*)kv_commit, dim3(layers, 2), dim3(256), 0, static_cast<cudaStream_t>(stream), a);
}

extern "C" int btb_b200_publish(void* n0, const void* ids, void* out_tok, void* out_n0, void* out_ts, int advance,
                                void* stream) {
    if (!n0) return B2_ERR_NULL;
    if (out_tok != nullptr && (!ids || !out_n0 || !out_ts)) return B2_ERR_NULL;
    PublishArgs a{static_cast<int*>(n0), static_cast<const long long*>(ids), static_cast<long long*>(out_tok),
                  static_cast<int*>(out_n0), static_cast<long long*>(out_ts), advance};
    return b2_launch((const void*)publish_step, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), a);
}
