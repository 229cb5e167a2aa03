// Paged GQA decode attention for sm_100a: a step's row, or a verify pass's chain or tree of T <= 32 rows, over a
// position-major bf16 cache [rows, Hk, D] read through an optional row map (64-row pages).
//
// The fold structure is the reference's (native/cuda/btb_attn_flash.cuh:7-14 of btb): a row's keys [first, last] are
// cut at fixed boundaries into tiles of 64 keys and groups of 8 tiles; a TILE's state (max, sum, output) is computed
// from nothing - scores scaled to log2 units, 2^(s - max) weights, the weights rounded to bf16 before they multiply V;
// a GROUP's state is its tiles' folded in tile order, the ROW's its groups' folded in group order, the output O / L
// in bf16. No tile waits on another and nothing depends on how many rows share the launch, so a verify pass's row is
// the step's row. The dot products here are f32 FMA chains in index order on the SIMT cores (decode attention is bound
// by the cache's bytes, not by math), so results agree with the reference's tensor-core tiles to rounding, not to
// the bit; the tests hold them to 2^-6 of the row's largest output like the reference's own attention test.
//
// Launch: block (grp, g, t) takes group grp of kv head g for token t's G query heads (G = 1, 2, 4 or 8); two warps
// take each tile of the group (a lane one key for the scores, D/32 dims for the output; the halves share the tile's
// max and their sums and outputs are added). Groups past the row's keys return at once, so
// one captured launch serves every length up to the capacity. A row reaching several groups stores each group's
// state and the last block to arrive folds them in group order - no block ever waits for another.
#include "common.cuh"
#include "btb_b200_internal.h"
#include "attn_core.cuh"

B2_DEFINE_STATUS(attn)

#include "../../include/btb_b200.h"

namespace {

template <int D, int G>
__global__ void __launch_bounds__(NWA * 32) attn_decode(const AttnArgs A) {
    extern __shared__ __align__(16) uint8_t dsm_raw[];
    pdl_launch_dependents();
    pdl_wait();
    attn_item<D, G, false>(A, blockIdx.x, blockIdx.y, blockIdx.z, dsm_raw);
}

template <int D, int G>
int launch_attn(const AttnArgs& a, dim3 grid, cudaStream_t s) {
    auto kern = attn_decode<D, G>;
    static bool allowed[64];
    int rc = b2_allow_smem(reinterpret_cast<const void*>(kern), allowed);
    if (rc) return rc;
    return b2_launch(reinterpret_cast<const void*>(kern), grid, dim3(NWA * 32), sizeof(AttnSmem<D, G>), s, a);
}
// the step's row: norm + RoPE + cache write + attention, one launch (T = 1)
constexpr int SPLIT_ROWS = 4096;
struct StepAttnArgs {
    AttnArgs a;
    RopeArgs r;
    int B;                   // sequences decoded side by side (row b of the pass belongs to sequence b), 1 for a step
    long long seq_stride;    // elements from a sequence's cache to the next one's
    // The step's attention row moves a few hundred KB and is a chain of dependent latencies; the memory system idles
    // under it. Blocks past the attention's own (grid x >= S) spend that time pulling the NEXT kernels' weights into
    // L2 (the output projection's, then the start of gate/up's): `warm` ranges of 16-byte-aligned bytes.
    const uint8_t* warm[2];
    long long warm_bytes[2];
    int S;                   // the attention's own extent of grid x
};
// a range of global memory into L2, 4 KB a request (the bulk-copy unit's prefetch form: no destination, no barrier)
__device__ __forceinline__ void l2_prefetch(const uint8_t* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
template <int D, int G>
__global__ void __launch_bounds__(NWA * 32) attn_step(const StepAttnArgs A) {
    extern __shared__ __align__(16) uint8_t dsm_raw[];
    if ((int)blockIdx.x >= A.S) {  // a warming block: weights do not depend on the kernels before this one
        const long long nblk = (long long)(gridDim.x - A.S) * gridDim.y * gridDim.z;
        const long long me = ((long long)(blockIdx.x - A.S) * gridDim.y + blockIdx.y) * gridDim.z + blockIdx.z;
        constexpr long long CH = 4096;
        for (int k = 0; k < 2; ++k) {
            const long long n = (A.warm_bytes[k] + CH - 1) / CH;
            for (long long c = me * blockDim.x + threadIdx.x; c < n; c += nblk * blockDim.x) {
                const long long left = A.warm_bytes[k] - c * CH;
                l2_prefetch(A.warm[k] + c * CH, (uint32_t)(left < CH ? left : CH));
            }
        }
        return;
    }
    pdl_wait();  // the trigger for the next kernel is inside, after the values are read
    if (A.B > 1) {
        // sequence b's row: its slice of qkv, its own cache, length, partials and counters. The adjusted arguments are made
        // once a block in shared memory (a per-thread copy of the two structs lives in local memory: slower to read)
        __shared__ __align__(16) unsigned char sa_raw[sizeof(AttnArgs)];
        __shared__ __align__(16) unsigned char sr_raw[sizeof(RopeArgs)];
        AttnArgs& sa = *reinterpret_cast<AttnArgs*>(sa_raw);
        RopeArgs& sr = *reinterpret_cast<RopeArgs*>(sr_raw);
        const int b = blockIdx.y / A.a.Hk, g = blockIdx.y - b * A.a.Hk;
        if (threadIdx.x == 0) {
            AttnArgs a = A.a;
            RopeArgs r = A.r;
            const int Hq = a.Hq, Hk = a.Hk;
            const size_t S = A.S;
            r.qkv += (size_t)b * (Hq + 2 * Hk) * D, r.n0p += b, r.depth += b, r.K += (size_t)b * A.seq_stride;
            r.V += (size_t)b * A.seq_stride, r.qo += (size_t)b * Hq * D;
            a.q = r.qo, a.K = r.K, a.V = r.V, a.out += (size_t)b * Hq * D, a.n0p = r.n0p;
            a.part_m += (size_t)b * S * Hq, a.part_l += (size_t)b * S * Hq, a.part_acc += (size_t)b * S * Hq * D, a.cnt += (size_t)b * Hq;
            sa = a, sr = r;
        }
        __syncthreads();
        if (G > 1 && *sa.n0p < SPLIT_ROWS) {
            attn_step_item<D, 1, G, true, true>(sa, sr, blockIdx.x, g, blockIdx.z, dsm_raw);
        } else if (blockIdx.z == 0) {
            attn_step_item<D, G, G, true, true>(sa, sr, blockIdx.x, g, 0, dsm_raw);
        }
        return;
    }
    // Below this many cached rows the group's heads take a block each (grid z); above, block z = 0 takes them all -
    // a long cache has blocks enough, and each key row is then read once.
    if (G > 1 && *A.a.n0p < SPLIT_ROWS) {
        attn_step_item<D, 1, G, true, true>(A.a, A.r, blockIdx.x, blockIdx.y, blockIdx.z, dsm_raw);
    } else if (blockIdx.z == 0) {
        attn_step_item<D, G, G, true, true>(A.a, A.r, blockIdx.x, blockIdx.y, 0, dsm_raw);
    }
}
template <int D, int G>
int launch_attn_step(const StepAttnArgs& a, dim3 grid, cudaStream_t s) {
    auto kern = attn_step<D, G>;
    static bool allowed[64];
    int rc = b2_allow_smem(reinterpret_cast<const void*>(kern), allowed);
    if (rc) return rc;
    // (the split form runs attn_step_item<D, 1, G>: its AttnSmem is the smaller one, the staging area starts no later)
    return b2_launch(reinterpret_cast<const void*>(kern), grid, dim3(NWA * 32),
                     attn_vstage_offset<D, G>() + attn_vstage_bytes<D>(), s, a);
}
template <int D>
int launch_attn_step_g(int G, const StepAttnArgs& a, dim3 grid, cudaStream_t s) {
    switch (G) {
        case 1: return launch_attn_step<D, 1>(a, grid, s);
        case 2: return launch_attn_step<D, 2>(a, grid, s);
        case 4: return launch_attn_step<D, 4>(a, grid, s);
        case 8: return launch_attn_step<D, 8>(a, grid, s);
        default: return B2_ERR_DOMAIN;
    }
}

template <int D>
int launch_attn_g(int G, const AttnArgs& a, dim3 grid, cudaStream_t s) {
    switch (G) {
        case 1: return launch_attn<D, 1>(a, grid, s);
        case 2: return launch_attn<D, 2>(a, grid, s);
        case 4: return launch_attn<D, 4>(a, grid, s);
        case 8: return launch_attn<D, 8>(a, grid, s);
        default: return B2_ERR_DOMAIN;
    }
}

}  // namespace

// the C-ABI's send descriptor into the kernels' own (a slice of T rows of Hq * D elements)
static int take_send(const btb_b200_send* send, int Hq, int D, B2Send& out) {
    if (send == nullptr || send->n == 0) return B2_OK;
    if (send->n < 0 || send->n > B2_MAX_RANKS || send->stride <= 0 || send->offset < 0 || send->offset + Hq * D > send->stride)
        return B2_ERR_DOMAIN;
    if (send->pass == nullptr) return B2_ERR_NULL;
    out.n = send->n, out.stride = send->stride, out.offset = send->offset;
    out.pass = static_cast<const unsigned*>(send->pass), out.per_pass = send->per_pass, out.base = send->base;
    for (int p = 0; p < send->n; ++p) {
        if (send->out[p] == nullptr) return B2_ERR_NULL;
        out.out[p] = static_cast<uint32_t*>(send->out[p]);
    }
    return B2_OK;
}

extern "C" size_t btb_b200_attn_scratch_floats(int S, int T, int Hq, int D) {
    return (size_t)S * T * Hq * (D + 2);
}

static int attn_decode_impl(const void* q, const void* K, const void* V, void* out, const void* n0p,
                                    const void* par, int T, int Hq, int Hk, int D, long long hs, long long rs,
                                    float scale, void* part_m, void* part_l, void* part_acc, void* cnt, int win,
                                    const void* tbl, const void* sinks, int cap, const btb_b200_send* send, void* stream,
                                    const void* rw = nullptr) {
    const bool sends = send != nullptr && send->n != 0;
    if (!q || !K || !V || (!out && !sends) || (!rw && (!n0p || !par)) || !part_m || !part_l || !part_acc || !cnt) return B2_ERR_NULL;
    if (T <= 0 || T > TMAX || Hk <= 0 || Hq <= 0 || Hq % Hk || (Hq / Hk != 1 && Hq / Hk != 2 && Hq / Hk != 4 && Hq / Hk != 8) || cap <= 0 || !(scale == scale))
        return B2_ERR_DOMAIN;
    // a key row is read as 16-byte chunks, a value row as D/32-element runs
    if ((hs & 7) || (rs & 7) || (reinterpret_cast<uintptr_t>(K) & 15) || (reinterpret_cast<uintptr_t>(V) & 15))
        return B2_ERR_DOMAIN;
    AttnArgs a{};
    a.q = static_cast<const bf16*>(q), a.K = static_cast<const bf16*>(K), a.V = static_cast<const bf16*>(V);
    a.out = static_cast<bf16*>(out), a.n0p = static_cast<const int*>(n0p), a.par = static_cast<const int*>(par);
    a.tbl = static_cast<const int*>(tbl), a.sinks = static_cast<const float*>(sinks);
    a.rw = static_cast<const int*>(rw);
    a.part_m = static_cast<float*>(part_m), a.part_l = static_cast<float*>(part_l);
    a.part_acc = static_cast<float*>(part_acc), a.cnt = static_cast<int*>(cnt);
    a.scale = scale, a.T = T, a.Hq = Hq, a.Hk = Hk, a.win = win, a.cap = cap, a.hs = hs, a.rs = rs;
    if (const int rc = take_send(send, Hq, D, a.send)) return rc;
    const int S = (cap + GK - 1) / GK;
    const dim3 grid(S, Hk, T);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (D) {
        case 64: return launch_attn_g<64>(Hq / Hk, a, grid, s);
        case 128: return launch_attn_g<128>(Hq / Hk, a, grid, s);
        default: return B2_ERR_DOMAIN;
    }
}

extern "C" int btb_b200_attn_decode(const void* q, const void* K, const void* V, void* out, const void* n0p,
                                    const void* par, int T, int Hq, int Hk, int D, long long hs, long long rs,
                                    float scale, void* part_m, void* part_l, void* part_acc, void* cnt, int win,
                                    const void* tbl, const void* sinks, int cap, void* stream) {
    return attn_decode_impl(q, K, V, out, n0p, par, T, Hq, Hk, D, hs, rs, scale, part_m, part_l, part_acc, cnt, win, tbl,
                            sinks, cap, nullptr, stream);
}

// the rows layout: row t a sequence of its own - its prefix, then its own steps - read in logical order, the order a
// one-row step of that sequence alone reads them in, so a row's bits are its own decode's whatever rows step beside it
extern "C" int btb_b200_attn_decode_rows(const void* q, const void* K, const void* V, void* out, const void* rw, int T,
                                         int Hq, int Hk, int D, long long hs, long long rs, float scale, void* part_m,
                                         void* part_l, void* part_acc, void* cnt, int win, const void* sinks, int cap,
                                         void* stream) {
    if (!rw) return B2_ERR_NULL;
    return attn_decode_impl(q, K, V, out, nullptr, nullptr, T, Hq, Hk, D, hs, rs, scale, part_m, part_l, part_acc, cnt, win,
                            nullptr, sinks, cap, nullptr, stream, rw);
}

// btb_b200_attn_decode in a model cut over ranks by kv head: the output rows go, marked, to every rank's copy
extern "C" int btb_b200_attn_decode_x(const void* q, const void* K, const void* V, const void* n0p, const void* par, int T,
                                      int Hq, int Hk, int D, long long hs, long long rs, float scale, void* part_m,
                                      void* part_l, void* part_acc, void* cnt, int win, const void* tbl, const void* sinks,
                                      int cap, const btb_b200_send* send, void* stream) {
    if (send == nullptr || send->n == 0) return B2_ERR_NULL;
    return attn_decode_impl(q, K, V, nullptr, n0p, par, T, Hq, Hk, D, hs, rs, scale, part_m, part_l, part_acc, cnt, win,
                            tbl, sinks, cap, send, stream);
}

static int attn_step_launch(const void* qkv, const void* wq, const void* wk, float eps, const void* cos_t,
                            const void* sin_t, const void* n0p, const void* depth, void* K, void* V, void* q, void* out,
                            int Hq, int Hk, int D, long long hs, long long rs, int centered, float scale, void* part_m,
                            void* part_l, void* part_acc, void* cnt, int win, const void* tbl, const void* sinks, int cap,
                            int B, long long seq_stride, void* stream, const btb_b200_send* send = nullptr,
                            const void* warm_a = nullptr, long long bytes_a = 0, const void* warm_b = nullptr,
                            long long bytes_b = 0) {
    const bool sends = send != nullptr && send->n != 0;
    if (!qkv || !cos_t || !sin_t || !n0p || !depth || !K || !V || !q || (!out && !sends) || !part_m || !part_l || !part_acc || !cnt)
        return B2_ERR_NULL;
    if (Hk <= 0 || Hq <= 0 || Hq % Hk || (Hq / Hk != 1 && Hq / Hk != 2 && Hq / Hk != 4 && Hq / Hk != 8) || cap <= 0 ||
        !(scale == scale))
        return B2_ERR_DOMAIN;
    if ((hs & 7) || (rs & 7) || (reinterpret_cast<uintptr_t>(K) & 15) || (reinterpret_cast<uintptr_t>(V) & 15))
        return B2_ERR_DOMAIN;
    // a lane reads its D/32 elements of a head, a norm weight or a table row as one load
    if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(wq) | reinterpret_cast<uintptr_t>(wk) |
         reinterpret_cast<uintptr_t>(cos_t) | reinterpret_cast<uintptr_t>(sin_t) | reinterpret_cast<uintptr_t>(q)) & 15)
        return B2_ERR_DOMAIN;
    StepAttnArgs sa{};
    AttnArgs& a = sa.a;
    a.q = static_cast<const bf16*>(q), a.K = static_cast<const bf16*>(K), a.V = static_cast<const bf16*>(V);
    a.out = static_cast<bf16*>(out), a.n0p = static_cast<const int*>(n0p), a.par = nullptr;
    a.tbl = static_cast<const int*>(tbl), a.sinks = static_cast<const float*>(sinks);
    a.part_m = static_cast<float*>(part_m), a.part_l = static_cast<float*>(part_l);
    a.part_acc = static_cast<float*>(part_acc), a.cnt = static_cast<int*>(cnt);
    a.scale = scale, a.T = 1, a.Hq = Hq, a.Hk = Hk, a.win = win, a.cap = cap, a.hs = hs, a.rs = rs;
    sa.r = RopeArgs{static_cast<const bf16*>(qkv), static_cast<const bf16*>(wq), static_cast<const bf16*>(wk),
                    static_cast<const bf16*>(cos_t), static_cast<const bf16*>(sin_t), static_cast<const int*>(n0p),
                    static_cast<const int*>(depth), static_cast<const int*>(tbl), nullptr, static_cast<bf16*>(K),
                    static_cast<bf16*>(V), static_cast<bf16*>(q), eps, 1, Hq, Hk, centered, hs, rs, cap};
    if (const int rc = take_send(send, Hq, D, a.send)) return rc;
    const int S = (cap + GK - 1) / GK;
    sa.B = B, sa.seq_stride = seq_stride, sa.S = S;
    // warming blocks: as many as fill the card beside the attention's, for at most `l2_warm_kb` of the next weights
    int extra = 0;
    {
        long long budget = (long long)b2_tuning().l2_warm_kb * 1024;
        const void* wp[2] = {warm_a, warm_b};
        const long long wb[2] = {bytes_a, bytes_b};
        for (int k = 0; k < 2; ++k) {
            if (wp[k] == nullptr || wb[k] <= 0 || budget <= 0) continue;
            if ((reinterpret_cast<uintptr_t>(wp[k]) & 15) || (wb[k] & 15)) return B2_ERR_DOMAIN;
            sa.warm[k] = static_cast<const uint8_t*>(wp[k]);
            sa.warm_bytes[k] = wb[k] < budget ? wb[k] : (budget & ~15LL);
            budget -= sa.warm_bytes[k];
        }
        if (sa.warm_bytes[0] + sa.warm_bytes[1] > 0) {
            const int per_x = Hk * B * (Hq / Hk);
            const int want = b2_tuning().l2_warm_ctas > 0 ? b2_tuning().l2_warm_ctas : b2_sm_count() - S * per_x;
            extra = want > 0 ? (want + per_x - 1) / per_x : 0;
        }
    }
    const dim3 grid(S + extra, Hk * B, Hq / Hk);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (D) {
        case 64: return launch_attn_step_g<64>(Hq / Hk, sa, grid, s);
        case 128: return launch_attn_step_g<128>(Hq / Hk, sa, grid, s);
        default: return B2_ERR_DOMAIN;
    }
}

extern "C" int btb_b200_attn_step(const void* qkv, const void* wq, const void* wk, float eps, const void* cos_t,
                                  const void* sin_t, const void* n0p, const void* depth, void* K, void* V, void* q,
                                  void* out, int Hq, int Hk, int D, long long hs, long long rs, int centered,
                                  float scale, void* part_m, void* part_l, void* part_acc, void* cnt, int win,
                                  const void* tbl, const void* sinks, int cap, void* stream) {
    return attn_step_launch(qkv, wq, wk, eps, cos_t, sin_t, n0p, depth, K, V, q, out, Hq, Hk, D, hs, rs, centered, scale,
                            part_m, part_l, part_acc, cnt, win, tbl, sinks, cap, 1, 0, stream);
}

// btb_b200_attn_step with idle SMs pulling the next kernels' weights into L2 while the row's latencies run their course
extern "C" int btb_b200_attn_step_w(const void* qkv, const void* wq, const void* wk, float eps, const void* cos_t,
                                    const void* sin_t, const void* n0p, const void* depth, void* K, void* V, void* q,
                                    void* out, int Hq, int Hk, int D, long long hs, long long rs, int centered, float scale,
                                    void* part_m, void* part_l, void* part_acc, void* cnt, int win, const void* tbl,
                                    const void* sinks, int cap, const btb_b200_send* send, const void* warm_a,
                                    long long bytes_a, const void* warm_b, long long bytes_b, void* stream) {
    return attn_step_launch(qkv, wq, wk, eps, cos_t, sin_t, n0p, depth, K, V, q, out, Hq, Hk, D, hs, rs, centered, scale,
                            part_m, part_l, part_acc, cnt, win, tbl, sinks, cap, 1, 0, stream, send, warm_a, bytes_a, warm_b,
                            bytes_b);
}

// btb_b200_attn_step in a model cut over ranks by kv head: the step's output row goes, marked, to every rank's copy
extern "C" int btb_b200_attn_step_x(const void* qkv, const void* wq, const void* wk, float eps, const void* cos_t,
                                    const void* sin_t, const void* n0p, const void* depth, void* K, void* V, void* q, int Hq,
                                    int Hk, int D, long long hs, long long rs, int centered, float scale, void* part_m,
                                    void* part_l, void* part_acc, void* cnt, int win, const void* tbl, const void* sinks,
                                    int cap, const btb_b200_send* send, void* stream) {
    if (send == nullptr || send->n == 0) return B2_ERR_NULL;
    return attn_step_launch(qkv, wq, wk, eps, cos_t, sin_t, n0p, depth, K, V, q, nullptr, Hq, Hk, D, hs, rs, centered, scale,
                            part_m, part_l, part_acc, cnt, win, tbl, sinks, cap, 1, 0, stream, send);
}

extern "C" int btb_b200_attn_step_batch(const void* qkv, const void* wq, const void* wk, float eps, const void* cos_t,
                                        const void* sin_t, const void* n0p, const void* depth, void* K, void* V, void* q,
                                        void* out, int B, long long seq_stride, int Hq, int Hk, int D, long long hs,
                                        long long rs, int centered, float scale, void* part_m, void* part_l,
                                        void* part_acc, void* cnt, int win, const void* sinks, int cap, void* stream) {
    if (B <= 0 || B > 32 || (long long)Hk * B > 65535 || seq_stride <= 0 || (seq_stride & 7)) return B2_ERR_DOMAIN;
    return attn_step_launch(qkv, wq, wk, eps, cos_t, sin_t, n0p, depth, K, V, q, out, Hq, Hk, D, hs, rs, centered, scale,
                            part_m, part_l, part_acc, cnt, win, nullptr, sinks, cap, B, seq_stride, stream);
}
