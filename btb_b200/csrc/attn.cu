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

B2_DEFINE_STATUS(attn)

namespace {

constexpr int BN = 64;        // keys a tile
constexpr int GT = 8;         // tiles a group: one a warp
constexpr int GK = BN * GT;   // keys a group
constexpr int TMAX = 32;      // rows a pass at most
#define LOG2E 1.4426950408889634f

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// a state (m, l) folded into the running (M, L): each side scaled to the larger max, the larger side's factor
// exactly 1; an empty side (max -inf) contributes nothing. Returns the factors for the outputs' fold.
__device__ __forceinline__ void fold_ml(float& M, float& L, float m, float l, float& cO, float& co) {
    const bool em = m == NEG_INF, eM = M == NEG_INF;
    const float hi = fmaxf(M, m), lo = fminf(M, m);
    const float e = ex2(em || eM ? 0.f : __fsub_rn(lo, hi));
    cO = em ? 1.f : eM ? 0.f : (M >= m ? 1.f : e);
    co = em ? 0.f : eM ? 1.f : (M > m ? e : 1.f);
    L = __fmaf_rn(l, co, __fmul_rn(L, cO));
    M = hi;
}
__device__ __forceinline__ float fold_e(float O, float o, float cO, float co) {
    return __fmaf_rn(o, co, __fmul_rn(O, cO));
}

struct AttnArgs {
    const bf16* q;    // [T, Hq, D]
    const bf16* K;    // head g, slot j at g * hs + j * rs
    const bf16* V;
    bf16* out;        // [T, Hq * D]
    const int* n0p;   // rows standing before the pass
    const int* par;   // [T] parents, -1 the root
    const int* tbl;   // logical slot -> cache row, or null
    const float* sinks;  // [Hq] a logit joined to the denominator, or null
    float* part_m;    // [S, T, Hq]
    float* part_l;
    float* part_acc;  // [S, T, Hq, D]
    int* cnt;         // [T, Hk] arrivals, zero between launches
    float scale;
    int T, Hq, Hk, win, cap;
    long long hs, rs;
};

constexpr int NWA = 2 * GT;  // warps a block: two a tile, 32 keys each (a lane one key)

// The block's shared memory (dynamic): the token's queries, the half-tiles' maxima and sums, each warp's weights
// (bf16-rounded) and each warp's partial outputs.
template <int D, int G>
struct AttnSmem {
    float qs[G][D];
    float hmax[GT][2][G];
    float hsum[GT][2][G];
    float ps[NWA][G][32];
    float ho[NWA][G][D];
};

template <int D, int G>
__global__ void __launch_bounds__(NWA * 32) attn_decode(const AttnArgs A) {
    constexpr int E = D / 32;  // dims a lane owns of an output row
    pdl_launch_dependents();
    pdl_wait();
    const int grp = blockIdx.x, g = blockIdx.y, t = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = warp >> 1, half = warp & 1;
    const int Hq = A.Hq, Hk = A.Hk, T = A.T;
    const int n0 = *A.n0p;

    __shared__ int anc[TMAX];  // token t's path, root first
    __shared__ int s_len;
    __shared__ int s_last_block;
    extern __shared__ __align__(16) uint8_t dsm_raw[];
    AttnSmem<D, G>& sm = *reinterpret_cast<AttnSmem<D, G>*>(dsm_raw);

    if (threadIdx.x == 0) {
        int len = 0;
        for (int p = t; p >= 0 && p < T && len < TMAX; p = A.par[p]) ++len;
        int k = len;
        for (int p = t; k > 0; p = A.par[p]) anc[--k] = p;
        s_len = len;
    }
    __syncthreads();
    const int last = n0 + s_len - 1;
    const int first = A.win > 0 ? max(last + 1 - A.win, 0) : 0;
    const int lo = grp * GK, hi = lo + GK - 1;
    if (lo > last || hi < first || last >= A.cap) {
        if (last >= A.cap && threadIdx.x == 0 && grp == 0) b2_fail(B2_ERR_DOMAIN);
        return;  // the group holds none of the row's keys: nothing stored, nothing counted
    }
    for (int i = threadIdx.x; i < G * D; i += NWA * 32) {
        const int hh = i / D, d = i - hh * D;
        sm.qs[hh][d] = bf2f(A.q[((size_t)t * Hq + g * G + hh) * D + d]);
    }
    __syncthreads();

    const float scale2 = __fmul_rn(A.scale, LOG2E);
    const bf16* Kg = A.K + (size_t)g * A.hs;
    const bf16* Vg = A.V + (size_t)g * A.hs;
    // ---- this warp's half of its tile: one key a lane ------------------------------------------------------------
    const int j = lo + tile * BN + half * 32 + lane;
    int row = -1;
    if (j >= first && j <= last) {
        int sl = j < n0 ? j : n0 + anc[j - n0];
        if (A.tbl != nullptr) sl = A.tbl[sl];
        row = sl;
    }
    float s[G];
    {
        // the key's whole row in flight at once (D/8 independent 16-byte loads), then the G dot products, each an
        // f32 chain over the dims in index order
        uint4 kv[D / 8];
        const uint4* kr = reinterpret_cast<const uint4*>(Kg + (size_t)(row >= 0 ? row : 0) * A.rs);
#pragma unroll
        for (int c = 0; c < D / 8; ++c) kv[c] = row >= 0 ? __ldg(kr + c) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int hh = 0; hh < G; ++hh) s[hh] = 0.f;
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
            const float kf[8] = {bf_lo(kv[c].x), bf_hi(kv[c].x), bf_lo(kv[c].y), bf_hi(kv[c].y),
                                 bf_lo(kv[c].z), bf_hi(kv[c].z), bf_lo(kv[c].w), bf_hi(kv[c].w)};
#pragma unroll
            for (int hh = 0; hh < G; ++hh) {
                float a = s[hh];
#pragma unroll
                for (int e = 0; e < 8; ++e) a = fmaf(kf[e], sm.qs[hh][c * 8 + e], a);
                s[hh] = a;
            }
        }
    }
#pragma unroll
    for (int hh = 0; hh < G; ++hh) {
        s[hh] = row >= 0 ? __fmul_rn(s[hh], scale2) : NEG_INF;
        float m = s[hh];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) sm.hmax[tile][half][hh] = m;
    }
    __syncthreads();
    // the tile's weights against the tile's max (both halves'), this half's sum and its share of P . V
    {
        float o[G][E];
#pragma unroll
        for (int hh = 0; hh < G; ++hh) {
            const float m = fmaxf(sm.hmax[tile][0][hh], sm.hmax[tile][1][hh]);
            const float p = (m == NEG_INF || row < 0) ? 0.f : ex2(__fsub_rn(s[hh], m));
            float l = p;
#pragma unroll
            for (int k = 16; k > 0; k >>= 1) l = __fadd_rn(l, __shfl_xor_sync(0xffffffffu, l, k));
            sm.ps[warp][hh][lane] = bfround(p);
            if (lane == 0) sm.hsum[tile][half][hh] = l;
#pragma unroll
            for (int e = 0; e < E; ++e) o[hh][e] = 0.f;
        }
        __syncwarp();
        // sixteen keys' value runs in flight at a time; a key the row does not see has weight 0 over zeros
        constexpr int VB = 16;
#pragma unroll 1
        for (int i0 = 0; i0 < 32; i0 += VB) {
            float vf[VB][E];
#pragma unroll
            for (int u = 0; u < VB; ++u) {
                const int rk = __shfl_sync(0xffffffffu, row, i0 + u);
                const bf16* vr = Vg + (size_t)(rk >= 0 ? rk : 0) * A.rs + lane * E;
                if (E == 4) {
                    const uint2 vv = rk >= 0 ? __ldg(reinterpret_cast<const uint2*>(vr)) : make_uint2(0u, 0u);
                    vf[u][0] = bf_lo(vv.x), vf[u][1] = bf_hi(vv.x), vf[u][2] = bf_lo(vv.y), vf[u][3] = bf_hi(vv.y);
                } else {
                    const uint32_t vv = rk >= 0 ? __ldg(reinterpret_cast<const uint32_t*>(vr)) : 0u;
                    vf[u][0] = bf_lo(vv), vf[u][E - 1] = bf_hi(vv);
                }
            }
#pragma unroll
            for (int u = 0; u < VB; ++u) {
#pragma unroll
                for (int hh = 0; hh < G; ++hh) {
                    const float p = sm.ps[warp][hh][i0 + u];
#pragma unroll
                    for (int e = 0; e < E; ++e) o[hh][e] = fmaf(p, vf[u][e], o[hh][e]);
                }
            }
        }
#pragma unroll
        for (int hh = 0; hh < G; ++hh)
#pragma unroll
            for (int e = 0; e < E; ++e) sm.ho[warp][hh][lane * E + e] = o[hh][e];
    }
    __syncthreads();

    // ---- the group's state: the tiles folded in tile order, a thread a run of (head, dim) elements -------------
    const int s_first = first / GK, s_last = last / GK;
    const bool single = s_first == s_last;
    for (int i = threadIdx.x; i < G * D; i += NWA * 32) {
        const int hh = i / D, d = i - hh * D;
        float M = NEG_INF, L = 0.f, O = 0.f;
        for (int w = 0; w < GT; ++w) {
            const float m = fmaxf(sm.hmax[w][0][hh], sm.hmax[w][1][hh]);
            if (m == NEG_INF) continue;  // an empty tile changes nothing
            const float l = __fadd_rn(sm.hsum[w][0][hh], sm.hsum[w][1][hh]);
            const float o = __fadd_rn(sm.ho[2 * w][hh][d], sm.ho[2 * w + 1][hh][d]);
            float cO, co;
            fold_ml(M, L, m, l, cO, co);
            O = fold_e(O, o, cO, co);
        }
        const size_t rowi = (size_t)t * Hq + g * G + hh;
        if (single) {
            if (A.sinks != nullptr) {
                float cO, co;
                fold_ml(M, L, __fmul_rn(A.sinks[g * G + hh], LOG2E), 1.f, cO, co);
                O = __fmul_rn(O, cO);
            }
            A.out[rowi * D + d] = f2bf(__fmul_rn(O, __fdiv_rn(1.f, L)));
        } else {
            const size_t idx = (size_t)grp * T * Hq + rowi;
            if (d == 0) {
                A.part_m[idx] = M;
                A.part_l[idx] = L;
            }
            A.part_acc[idx * D + d] = O;
        }
    }
    if (single) return;
    // ---- several groups: count this block in; the last one folds the row's groups in group order ----------------
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last_block = atomicAdd(A.cnt + (size_t)t * Hk + g, 1) == s_last - s_first ? 1 : 0;
    __syncthreads();
    if (!s_last_block) return;
    __threadfence();
    for (int i = threadIdx.x; i < G * D; i += NWA * 32) {
        const int hh = i / D, d = i - hh * D;
        const size_t rowi = (size_t)t * Hq + g * G + hh;
        float M = NEG_INF, L = 0.f, O = 0.f;
        for (int sp = s_first; sp <= s_last; ++sp) {
            const size_t iu = (size_t)sp * T * Hq + rowi;
            float cO, co;
            fold_ml(M, L, __ldcg(A.part_m + iu), __ldcg(A.part_l + iu), cO, co);
            O = fold_e(O, __ldcg(A.part_acc + iu * D + d), cO, co);
        }
        if (A.sinks != nullptr) {
            float cO, co;
            fold_ml(M, L, __fmul_rn(A.sinks[g * G + hh], LOG2E), 1.f, cO, co);
            O = __fmul_rn(O, cO);
        }
        A.out[rowi * D + d] = f2bf(__fmul_rn(O, __fdiv_rn(1.f, L)));
    }
    if (threadIdx.x == 0) A.cnt[(size_t)t * Hk + g] = 0;
}

template <int D, int G>
int launch_attn(const AttnArgs& a, dim3 grid, cudaStream_t s) {
    auto kern = attn_decode<D, G>;
    static bool allowed[64];
    int rc = b2_allow_smem(reinterpret_cast<const void*>(kern), allowed);
    if (rc) return rc;
    return b2_launch(reinterpret_cast<const void*>(kern), grid, dim3(NWA * 32), sizeof(AttnSmem<D, G>), s, a);
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

extern "C" size_t btb_b200_attn_scratch_floats(int S, int T, int Hq, int D) {
    return (size_t)S * T * Hq * (D + 2);
}

extern "C" int btb_b200_attn_decode(const void* q, const void* K, const void* V, void* out, const void* n0p,
                                    const void* par, int T, int Hq, int Hk, int D, long long hs, long long rs,
                                    float scale, void* part_m, void* part_l, void* part_acc, void* cnt, int win,
                                    const void* tbl, const void* sinks, int cap, void* stream) {
    if (!q || !K || !V || !out || !n0p || !par || !part_m || !part_l || !part_acc || !cnt) return B2_ERR_NULL;
    if (T <= 0 || T > TMAX || Hk <= 0 || Hq <= 0 || Hq % Hk || (Hq / Hk != 1 && Hq / Hk != 2 && Hq / Hk != 4 && Hq / Hk != 8) || cap <= 0 || !(scale == scale))
        return B2_ERR_DOMAIN;
    // a key row is read as 16-byte chunks, a value row as D/32-element runs
    if ((hs & 7) || (rs & 7) || (reinterpret_cast<uintptr_t>(K) & 15) || (reinterpret_cast<uintptr_t>(V) & 15))
        return B2_ERR_DOMAIN;
    AttnArgs a{};
    a.q = static_cast<const bf16*>(q), a.K = static_cast<const bf16*>(K), a.V = static_cast<const bf16*>(V);
    a.out = static_cast<bf16*>(out), a.n0p = static_cast<const int*>(n0p), a.par = static_cast<const int*>(par);
    a.tbl = static_cast<const int*>(tbl), a.sinks = static_cast<const float*>(sinks);
    a.part_m = static_cast<float*>(part_m), a.part_l = static_cast<float*>(part_l);
    a.part_acc = static_cast<float*>(part_acc), a.cnt = static_cast<int*>(cnt);
    a.scale = scale, a.T = T, a.Hq = Hq, a.Hk = Hk, a.win = win, a.cap = cap, a.hs = hs, a.rs = rs;
    const int S = (cap + GK - 1) / GK;
    const dim3 grid(S, Hk, T);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (D) {
        case 64: return launch_attn_g<64>(Hq / Hk, a, grid, s);
        case 128: return launch_attn_g<128>(Hq / Hk, a, grid, s);
        default: return B2_ERR_DOMAIN;
    }
}
