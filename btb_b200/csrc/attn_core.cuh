// The decode attention's arithmetic and the q/k-norm + RoPE + cache-write arithmetic as device functions, shared by
// the standalone kernels (attn.cu, layer.cu) and the whole-step kernel (step.cu).
#pragma once

#include "common.cuh"
#include "tp.cuh"


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

// The rows layout (native/cuda/btb_kernels.cu:228-248 of btb): a pass's T rows as T sequences a token each - a fork's
// rows or a batch's - each at its own position. One int32 array on the card: [base, step, W, then (col, off, len) a row].
// Row t's keys in logical order are its prefix - `len` cache rows from `off` (forks share one prefix) - and then its own
// steps, step i at cache row base + i * W + col (every row's step i in one stretch of W rows). len < 0: padding, the
// row computes nothing.
struct RowSeq {
    int base, step, W, col, off, len;
    __device__ __forceinline__ RowSeq(const int* rw, int t, bool on = true)
        : base(on ? rw[0] : 0), step(on ? rw[1] : 0), W(on ? rw[2] : 0), col(on ? rw[3 + 3 * t] : 0),
          off(on ? rw[4 + 3 * t] : 0), len(on ? rw[5 + 3 * t] : 0) {}
    __device__ __forceinline__ int slot(int j) const { return j < len ? off + j : base + (j - len) * W + col; }
    __device__ __forceinline__ int position() const { return len + step; }  // of the token this pass adds
};

struct AttnArgs {
    const bf16* q;    // [T, Hq, D]
    const bf16* K;    // head g, slot j at g * hs + j * rs
    const bf16* V;
    bf16* out;        // [T, Hq * D]
    const int* n0p;   // rows standing before the pass
    const int* par;   // [T] parents, -1 the root
    const int* tbl;   // logical slot -> cache row, or null
    const int* rw;    // the rows layout (RowSeq), or null; with it n0p, par and tbl are not read
    const float* sinks;  // [Hq] a logit joined to the denominator, or null
    float* part_m;    // [S, T, Hq]
    float* part_l;
    float* part_acc;  // [S, T, Hq, D]
    int* cnt;         // [T, Hk] arrivals, zero between launches
    float scale;
    int T, Hq, Hk, win, cap;
    long long hs, rs;
    // a model cut over ranks by kv head (tp.cuh): with send.n > 0 a finished output element goes, marked, to every rank's
    // copy of the full [T, stride] vector at [t][send.offset + head * D + d] instead of `out`
    B2Send send{};
};

// a finished output element: the local row, or every rank's copy of the exchanged vector
__device__ __forceinline__ void attn_store(const AttnArgs& A, int t, int head, int d, int D, bf16 v, uint32_t mark) {
    if (A.send.n == 0) {
        A.out[((size_t)t * A.Hq + head) * D + d] = v;
        return;
    }
    const size_t at = (size_t)t * A.send.stride + A.send.offset + (size_t)head * D + d;
    const uint32_t word = b2_word(v, mark);
#pragma unroll 1
    for (int p = 0; p < A.send.n; ++p) A.send.out[p][at] = word;
}

constexpr int NWA = 2 * GT;  // warps a block: two a tile, 32 keys each (a lane one key)

// The block's shared memory (dynamic): the token's queries, the half-tiles' maxima and sums, each warp's weights
// (bf16-rounded) and each warp's partial outputs.
template <int D, int G>
struct AttnSmem {
    uint32_t qs[G][D / 2];  // the queries as packed bf16 pairs (what the mixed-precision fma multiplies with)
    float hmax[GT][2][G];
    float hsum[GT][2][G];
    unsigned short ps[NWA][G][32];  // the weights, bf16
    float ho[NWA][G][D];
};

// ---- a block's tiles folded into its group's state, and a row's groups into the row -------------------------------
// `sm` holds the tiles' maxima, sums and partial outputs; [first, last] the row's keys. A row inside one group is
// written out at once; else the group's state is stored and the last block to arrive folds the groups in order.
template <int D, int G>
__device__ __forceinline__ void attn_finish(const AttnArgs& A, AttnSmem<D, G>& sm, int grp, int hbase, int ci, int t,
                                            int first, int last, int* s_last_block_p) {
    // hbase: the first of the block's G query heads; ci: the block's arrival counter (one a set of blocks that share
    // a row's groups)
    const int Hq = A.Hq, T = A.T;
    int& s_last_block = *s_last_block_p;
    const uint32_t mark = A.send.n != 0 ? b2_hop_mark(A.send.pass, A.send.per_pass, A.send.base) : 0u;
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
        const size_t rowi = (size_t)t * Hq + hbase + hh;
        if (single) {
            if (A.sinks != nullptr) {
                float cO, co;
                fold_ml(M, L, __fmul_rn(A.sinks[hbase + hh], LOG2E), 1.f, cO, co);
                O = __fmul_rn(O, cO);
            }
            attn_store(A, t, hbase + hh, d, D, f2bf(__fmul_rn(O, __fdiv_rn(1.f, L))), mark);
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
    if (threadIdx.x == 0) s_last_block = atomicAdd(A.cnt + ci, 1) == s_last - s_first ? 1 : 0;
    __syncthreads();
    if (!s_last_block) return;
    __threadfence();
    for (int i = threadIdx.x; i < G * D; i += NWA * 32) {
        const int hh = i / D, d = i - hh * D;
        const size_t rowi = (size_t)t * Hq + hbase + hh;
        float M = NEG_INF, L = 0.f, O = 0.f;
        for (int sp = s_first; sp <= s_last; ++sp) {
            const size_t iu = (size_t)sp * T * Hq + rowi;
            float cO, co;
            fold_ml(M, L, __ldcg(A.part_m + iu), __ldcg(A.part_l + iu), cO, co);
            O = fold_e(O, __ldcg(A.part_acc + iu * D + d), cO, co);
        }
        if (A.sinks != nullptr) {
            float cO, co;
            fold_ml(M, L, __fmul_rn(A.sinks[hbase + hh], LOG2E), 1.f, cO, co);
            O = __fmul_rn(O, cO);
        }
        attn_store(A, t, hbase + hh, d, D, f2bf(__fmul_rn(O, __fdiv_rn(1.f, L))), mark);
    }
    if (threadIdx.x == 0) A.cnt[ci] = 0;
}

// one block's work: group grp of kv head g for row t. COHERENT: q and the cache are read with L2-coherent loads
// (the whole-step kernel, where other SMs wrote them earlier in the same launch).
template <int D, int G, bool COHERENT>
__device__ __forceinline__ void attn_item(const AttnArgs& A, int grp, int g, int t, uint8_t* dsm_raw) {
    constexpr int E = D / 32;  // dims a lane owns of an output row
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = warp >> 1, half = warp & 1;
    const int Hq = A.Hq, Hk = A.Hk, T = A.T;
    const int n0 = A.rw != nullptr ? 0 : (COHERENT ? __ldcg(A.n0p) : *A.n0p);

    __shared__ int anc[TMAX];  // token t's path, root first
    __shared__ int s_len;
    __shared__ int s_last_block;
    AttnSmem<D, G>& sm = *reinterpret_cast<AttnSmem<D, G>*>(dsm_raw);

    __syncthreads();  // the block's previous item is done with the shared state
    const bool rows = A.rw != nullptr;
    RowSeq rp(rows ? A.rw : nullptr, rows ? t : 0, rows);
    if (rows && rp.len < 0) return;  // padding
    if (threadIdx.x == 0 && !rows) {
        int len = 0;
        for (int p = t; p >= 0 && p < T && len < TMAX; p = A.par[p]) ++len;
        int k = len;
        for (int p = t; k > 0; p = A.par[p]) anc[--k] = p;
        s_len = len;
    }
    __syncthreads();
    const int last = rows ? rp.position() : n0 + s_len - 1;
    const int first = A.win > 0 ? max(last + 1 - A.win, 0) : 0;
    const int lo = grp * GK, hi = lo + GK - 1;
    if (lo > last || hi < first || (!rows && last >= A.cap)) {
        if (!rows && last >= A.cap && threadIdx.x == 0 && grp == 0) b2_fail(B2_ERR_DOMAIN);
        return;  // the group holds none of the row's keys: nothing stored, nothing counted
    }
    for (int i = threadIdx.x; i < G * D; i += NWA * 32) {
        const int hh = i / D, d = i - hh * D;
        const bf16* qp = A.q + ((size_t)t * Hq + g * G + hh) * D + d;
        reinterpret_cast<unsigned short*>(&sm.qs[hh][0])[d] =
            COHERENT ? __ldcg(reinterpret_cast<const unsigned short*>(qp)) : *reinterpret_cast<const unsigned short*>(qp);
    }
    __syncthreads();

    const float scale2 = __fmul_rn(A.scale, LOG2E);
    const bf16* Kg = A.K + (size_t)g * A.hs;
    const bf16* Vg = A.V + (size_t)g * A.hs;
    // ---- this warp's half of its tile: one key a lane ------------------------------------------------------------
    const int j = lo + tile * BN + half * 32 + lane;
    int row = -1;
    if (j >= first && j <= last) {
        if (rows) {
            row = rp.slot(j);
            if (row < 0 || row >= A.cap) {  // a layout that points outside the cache: refused, the key not read
                b2_fail(B2_ERR_DOMAIN);
                row = -1;
            }
        } else {
            int sl = j < n0 ? j : n0 + anc[j - n0];
            if (A.tbl != nullptr) sl = A.tbl[sl];
            row = sl;
        }
    }
    float s[G];
    {
        // the key's whole row in flight at once (D/8 independent 16-byte loads), then the G dot products, each an
        // f32 chain over the dims in index order
        uint4 kv[D / 8];
        const uint4* kr = reinterpret_cast<const uint4*>(Kg + (size_t)(row >= 0 ? row : 0) * A.rs);
#pragma unroll
        for (int c = 0; c < D / 8; ++c) kv[c] = row >= 0 ? (COHERENT ? __ldcg(kr + c) : __ldg(kr + c)) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int hh = 0; hh < G; ++hh) s[hh] = 0.f;
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
            // eight dims of the chain: the key's and the query's bf16 multiplied where they lie, the sum f32 (the bits
            // of fmaf over the widened values, in index order)
#pragma unroll
            for (int hh = 0; hh < G; ++hh) {
                const uint4 q4 = *reinterpret_cast<const uint4*>(&sm.qs[hh][c * 4]);
                float a = s[hh];
                a = fma2_bf16(kv[c].x, q4.x, a);
                a = fma2_bf16(kv[c].y, q4.y, a);
                a = fma2_bf16(kv[c].z, q4.z, a);
                a = fma2_bf16(kv[c].w, q4.w, a);
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
            sm.ps[warp][hh][lane] = __bfloat16_as_ushort(f2bf(p));
            if (lane == 0) sm.hsum[tile][half][hh] = l;
#pragma unroll
            for (int e = 0; e < E; ++e) o[hh][e] = 0.f;
        }
        __syncwarp();
        // sixteen keys' value runs in flight at a time; a key the row does not see has weight 0 over zeros
        constexpr int VB = 16;
#pragma unroll 1
        for (int i0 = 0; i0 < 32; i0 += VB) {
            unsigned short vf[VB][E];  // bf16 as loaded: the mixed-precision fma multiplies them with the bf16 weights
#pragma unroll
            for (int u = 0; u < VB; ++u) {
                const int rk = __shfl_sync(0xffffffffu, row, i0 + u);
                const bf16* vr = Vg + (size_t)(rk >= 0 ? rk : 0) * A.rs + lane * E;
                if (E == 4) {
                    const uint2 vv = rk >= 0 ? (COHERENT ? __ldcg(reinterpret_cast<const uint2*>(vr)) : __ldg(reinterpret_cast<const uint2*>(vr)))
                                             : make_uint2(0u, 0u);
                    split_bf16(vv.x, vf[u][0], vf[u][1]);
                    split_bf16(vv.y, vf[u][2], vf[u][3]);
                } else {
                    const uint32_t vv = rk >= 0 ? (COHERENT ? __ldcg(reinterpret_cast<const uint32_t*>(vr)) : __ldg(reinterpret_cast<const uint32_t*>(vr)))
                                            : 0u;
                    split_bf16(vv, vf[u][0], vf[u][E - 1]);
                }
            }
#pragma unroll
            for (int u = 0; u < VB; ++u) {
#pragma unroll
                for (int hh = 0; hh < G; ++hh) {
                    const unsigned short p = sm.ps[warp][hh][i0 + u];
#pragma unroll
                    for (int e = 0; e < E; ++e) o[hh][e] = fma_bf16(p, vf[u][e], o[hh][e]);
                }
            }
        }
#pragma unroll
        for (int hh = 0; hh < G; ++hh)
#pragma unroll
            for (int e = 0; e < E; ++e) sm.ho[warp][hh][lane * E + e] = o[hh][e];
    }
    __syncthreads();

    attn_finish<D, G>(A, sm, grp, g * G, t * Hk + g, t, first, last, &s_last_block);
}

// ---- q/k RMSNorm + RoPE + cache write (btb_kernels.cu:261-327) -----------------------------------------------------
// One warp per (head, row): lane l holds dims l*E .. l*E+E-1, so rotate_half's partner is lane ^ 16.
struct RopeArgs {
    const bf16* qkv;
    const bf16* wq;
    const bf16* wk;
    const bf16* cos_t;
    const bf16* sin_t;
    const int* n0p;
    const int* depth;
    const int* tbl;
    const int* rw;  // the rows layout (RowSeq), or null; with it n0p, depth and tbl are not read
    bf16* K;
    bf16* V;
    bf16* qo;
    float eps;
    int T, Hq, Hk, centered;
    long long hs, rs;
    int cap;  // cache rows: a slot at or past it is refused
};
// the E values lane `lane` owns of `head` for row t at position `pos`: q and k heads normalised and rotated, a v head
// as it stands - the bf16 values the cache and the query buffer hold
// E consecutive bf16 (E = 2, 4 or 8; the address a multiple of 2 E bytes) as one load
template <int E, bool COHERENT>
__device__ __forceinline__ void ld_run(const bf16* p, bf16* out) {
    if (E == 4) {
        const uint2 v = COHERENT ? __ldcg(reinterpret_cast<const uint2*>(p)) : *reinterpret_cast<const uint2*>(p);
        *reinterpret_cast<uint2*>(out) = v;
    } else if (E == 2) {
        const uint32_t v = COHERENT ? __ldcg(reinterpret_cast<const uint32_t*>(p)) : *reinterpret_cast<const uint32_t*>(p);
        *reinterpret_cast<uint32_t*>(out) = v;
    } else {
        const uint4 v = COHERENT ? __ldcg(reinterpret_cast<const uint4*>(p)) : *reinterpret_cast<const uint4*>(p);
        *reinterpret_cast<uint4*>(out) = v;
    }
}

template <int D, bool COHERENT>
__device__ __forceinline__ void rope_values(const RopeArgs& A, int head, int t, int lane, int pos, bf16* out) {
    constexpr int E = D / 32;
    const int Hq = A.Hq, Hk = A.Hk;
    const int width = (Hq + 2 * Hk) * D;
    const bf16* src = A.qkv + (size_t)t * width + (size_t)head * D + lane * E;
    __align__(16) bf16 raw[E];
    ld_run<E, COHERENT>(src, raw);
    if (head >= Hq + Hk) {
#pragma unroll
        for (int e = 0; e < E; ++e) out[e] = raw[e];
        return;
    }
    const bf16* wn = head < Hq ? A.wq : A.wk;
    // every load the head needs is issued before the first is used
    __align__(16) bf16 wr[E], cr[E], sr[E];
    if (wn != nullptr) ld_run<E, false>(wn + lane * E, wr);
    ld_run<E, false>(A.cos_t + (size_t)pos * D + lane * E, cr);
    ld_run<E, false>(A.sin_t + (size_t)pos * D + lane * E, sr);
    float v[E];
#pragma unroll
    for (int e = 0; e < E; ++e) v[e] = bf2f(raw[e]);
    if (wn != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) ss = fmaf(v[e], v[e], ss);
        ss = warp_sum(ss);
        const float rstd = rsqrtf(ss / (float)D + A.eps);
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const float wv = bf2f(wr[e]);
            v[e] = bfround(v[e] * rstd * (A.centered ? 1.f + wv : wv));
        }
    }
    const float sgn = lane < 16 ? -1.f : 1.f;
#pragma unroll
    for (int e = 0; e < E; ++e) {
        const float rot = __shfl_xor_sync(0xffffffffu, v[e], 16);
        const float qc = bfround(v[e] * bf2f(cr[e]));
        out[e] = f2bf(fmaf(sgn * rot, bf2f(sr[e]), qc));
    }
}

template <int D, bool COHERENT>
__device__ __forceinline__ void rope_item(const RopeArgs& A, int head, int t, int lane) {
    constexpr int E = D / 32;
    int slot, pos;
    if (A.rw != nullptr) {
        const RowSeq rp(A.rw, t);
        if (rp.len < 0) return;  // padding
        pos = rp.position();
        slot = rp.slot(pos);
    } else {
        const int n0 = COHERENT ? __ldcg(A.n0p) : *A.n0p;
        slot = n0 + t;
        pos = n0 + A.depth[t];
    }
    if (slot < 0 || slot >= A.cap || pos < 0 || pos >= A.cap) {
        if (lane == 0) b2_fail(B2_ERR_DOMAIN);
        return;
    }
    if (A.rw == nullptr && A.tbl != nullptr) slot = A.tbl[slot];
    const int Hq = A.Hq, Hk = A.Hk;
    bf16 o[E];
    rope_values<D, COHERENT>(A, head, t, lane, pos, o);
    bf16* dst = head >= Hq + Hk ? (A.V + (size_t)(head - Hq - Hk) * A.hs + (size_t)slot * A.rs + lane * E)
                : head < Hq     ? (A.qo + ((size_t)t * Hq + head) * D + lane * E)
                                : (A.K + (size_t)(head - Hq) * A.hs + (size_t)slot * A.rs + lane * E);
#pragma unroll
    for (int e = 0; e < E; ++e) dst[e] = o[e];
}

// ---- the step's row: q/k-norm + RoPE + cache write and the attention in one block -------------------------------------
// One row (T = 1) at slot n0. Every block of kv head g rotates the head's G queries itself (into shared memory); the
// block whose group holds slot n0 also makes the new key and value, writes them to the cache and keeps them in shared
// memory, since it is the only block that reads them. The old keys' loads are issued before any of that, so the two
// latencies overlap. The arithmetic is rope_values' and attn_item's: the row's bits are the two kernels' bits.
// G: the query heads this block takes, GQ the heads a kv head serves. G == GQ: the kv head's whole group (z = 0).
// G == 1: head z of the group - a short cache leaves most of the card idle and the per-key arithmetic is what takes
// the time, so the group's heads spread over GQ blocks (each reads the kv head's rows: they are few). Only block z = 0
// writes the cache.
// VSTAGE: every warp's 32 value rows are copied to shared memory asynchronously (cp.async) as soon as its keys' cache rows
// are known - they land while the scores are made, so the value products wait for no round trip of their own. The block's
// dynamic shared memory then holds, after AttnSmem, NWA x 32 rows of D bf16 (attn_vstage_bytes).
template <int D, int G>
__host__ __device__ constexpr size_t attn_vstage_offset() { return (sizeof(AttnSmem<D, G>) + 127) & ~(size_t)127; }
template <int D>
__host__ __device__ constexpr size_t attn_vstage_bytes() { return (size_t)NWA * 32 * D * 2; }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

template <int D, int G, int GQ, bool TRIGGER = true, bool VSTAGE = false>
__device__ __forceinline__ void attn_step_item(const AttnArgs& A, const RopeArgs& RA, int grp, int g, int z,
                                               uint8_t* dsm_raw) {
    const int hbase = g * GQ + z;
    constexpr int E = D / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = warp >> 1, half = warp & 1;
    const int Hq = A.Hq, Hk = A.Hk;
    __shared__ int s_last_block;
    __shared__ __align__(16) bf16 knew[D];
    __shared__ __align__(16) bf16 vnew[D];
    AttnSmem<D, G>& sm = *reinterpret_cast<AttnSmem<D, G>*>(dsm_raw);

    const int n0 = *A.n0p;
    const int pos = n0 + RA.depth[0];
    const int last = n0;
    const int first = A.win > 0 ? max(last + 1 - A.win, 0) : 0;
    const int lo = grp * GK, hi = lo + GK - 1;
    if (lo > last || hi < first) return;
    if (n0 < 0 || last >= A.cap || pos < 0 || pos >= A.cap) {
        if (threadIdx.x == 0) b2_fail(B2_ERR_DOMAIN);
        return;
    }
    const bool owner = lo <= n0 && n0 <= hi;  // this block's group holds the new row
    const bf16* Kg = A.K + (size_t)g * A.hs;
    const bf16* Vg = A.V + (size_t)g * A.hs;
    // ---- this lane's key ------------------------------------------------------------------------------------------
    const int wbase = lo + tile * BN + half * 32;
    const int j = wbase + lane;
    const int new_lane = owner ? n0 - wbase : -1;  // the lane of this warp that holds the new key (if in 0..31)
    int row = -1;
    if (j >= first && j <= last) row = A.tbl != nullptr ? A.tbl[j] : j;
    // a warp none of whose keys the row sees leaves its tile's half empty and stays out of the arithmetic
    const bool any = __ballot_sync(0xffffffffu, row >= 0) != 0u;
    // the warp's value rows on their way to shared memory: two keys an instruction, sixteen lanes a row (a row is D * 2
    // contiguous bytes on both sides: coalesced reads, conflict-free writes); the new key's row comes from `vnew` instead
    uint8_t* vst = dsm_raw + attn_vstage_offset<D, G>() + (size_t)warp * 32 * D * 2;
    if (VSTAGE && any) {
        constexpr int LPR = D * 2 / 16;   // lanes a row: 16-byte pieces
        constexpr int KPI = 32 / LPR;     // keys an instruction
        const int piece = lane % LPR, sub = lane / LPR;
#pragma unroll
        for (int u0 = 0; u0 < 32; u0 += KPI) {
            const int u = u0 + sub;
            const int rk = __shfl_sync(0xffffffffu, row, u);
            if (rk >= 0 && u != new_lane)
                cp_async16(smem_u32(vst + (size_t)u * D * 2 + piece * 16),
                           reinterpret_cast<const uint8_t*>(Vg + (size_t)rk * A.rs) + piece * 16);
        }
    }
    // ---- the head's queries (every block), the new key and value (the owner): the block's LAST warps take them, the
    // ones whose tiles a short cache leaves empty, and before their own keys - the rotation is what the block waits for
    const int rw = NWA - 1 - warp;
    if (rw < G) {
        bf16 o[E];
        rope_values<D, false>(RA, hbase + rw, 0, lane, pos, o);
#pragma unroll
        for (int e = 0; e < E; ++e) reinterpret_cast<bf16*>(&sm.qs[rw][0])[lane * E + e] = o[e];
        if (owner) {
            bf16* dst = RA.qo + (size_t)(hbase + rw) * D + lane * E;
#pragma unroll
            for (int e = 0; e < E; ++e) dst[e] = o[e];
        }
    } else if (rw < G + 2 && owner) {
        const bool is_k = rw == G;
        bf16 o[E];
        rope_values<D, false>(RA, is_k ? Hq + g : Hq + Hk + g, 0, lane, pos, o);
        const int slot = A.tbl != nullptr ? A.tbl[n0] : n0;
        bf16* dst = (is_k ? RA.K : RA.V) + (size_t)g * A.hs + (size_t)slot * A.rs + lane * E;
        bf16* keep = (is_k ? knew : vnew) + lane * E;
#pragma unroll
        for (int e = 0; e < E; ++e) keep[e] = o[e];
        if (z == 0) {
#pragma unroll
            for (int e = 0; e < E; ++e) dst[e] = o[e];
        }
    }
    // an old key's row: D/8 independent 16-byte loads in flight
    uint4 kv[D / 8];
    {
        const bool fetch = row >= 0 && lane != new_lane;
        const uint4* kr = reinterpret_cast<const uint4*>(Kg + (size_t)(fetch ? row : 0) * A.rs);
#pragma unroll
        for (int c = 0; c < D / 8; ++c) kv[c] = fetch ? __ldg(kr + c) : make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
    float s[G];
    if (any) {
        if (lane == new_lane && row >= 0) {
#pragma unroll
            for (int c = 0; c < D / 8; ++c) kv[c] = reinterpret_cast<const uint4*>(knew)[c];
        }
        const float scale2 = __fmul_rn(A.scale, LOG2E);
#pragma unroll
        for (int hh = 0; hh < G; ++hh) s[hh] = 0.f;
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
            // eight dims of the chain: the key's and the query's bf16 multiplied where they lie, the sum f32 (the bits
            // of fmaf over the widened values, in index order)
#pragma unroll
            for (int hh = 0; hh < G; ++hh) {
                const uint4 q4 = *reinterpret_cast<const uint4*>(&sm.qs[hh][c * 4]);
                float a = s[hh];
                a = fma2_bf16(kv[c].x, q4.x, a);
                a = fma2_bf16(kv[c].y, q4.y, a);
                a = fma2_bf16(kv[c].z, q4.z, a);
                a = fma2_bf16(kv[c].w, q4.w, a);
                s[hh] = a;
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
    } else {
        // what the arithmetic would have left for a half with no key: max -inf, sum 0, outputs 0
        if (lane < G) sm.hmax[tile][half][lane] = NEG_INF, sm.hsum[tile][half][lane] = 0.f;
        for (int i = lane; i < G * D; i += 32) sm.ho[warp][i / D][i % D] = 0.f;
    }
    __syncthreads();
    if (any) {
        float o[G][E];
#pragma unroll
        for (int hh = 0; hh < G; ++hh) {
            const float m = fmaxf(sm.hmax[tile][0][hh], sm.hmax[tile][1][hh]);
            const float p = (m == NEG_INF || row < 0) ? 0.f : ex2(__fsub_rn(s[hh], m));
            float l = p;
#pragma unroll
            for (int k = 16; k > 0; k >>= 1) l = __fadd_rn(l, __shfl_xor_sync(0xffffffffu, l, k));
            sm.ps[warp][hh][lane] = __bfloat16_as_ushort(f2bf(p));
            if (lane == 0) sm.hsum[tile][half][hh] = l;
#pragma unroll
            for (int e = 0; e < E; ++e) o[hh][e] = 0.f;
        }
        __syncwarp();
        // all thirty-two keys' value runs in flight at once (raw, in the registers the key row has left); a key the
        // row does not see has weight 0 over zeros
        uint32_t vraw[32][E / 2];
        if (VSTAGE) {
            cp_async_wait_all();  // this lane's copies have landed ...
            __syncwarp();         // ... and so have the other lanes'
        }
#pragma unroll
        for (int u = 0; u < 32; ++u) {
            const int rk = __shfl_sync(0xffffffffu, row, u);
            const bool from_smem = u == new_lane;
            const bf16* vr = from_smem ? vnew + lane * E
                             : VSTAGE  ? reinterpret_cast<const bf16*>(vst + (size_t)u * D * 2) + lane * E
                                       : Vg + (size_t)(rk >= 0 ? rk : 0) * A.rs + lane * E;
            if (E == 4) {
                const uint2 vv = rk < 0 ? make_uint2(0u, 0u)
                                 : (from_smem || VSTAGE) ? *reinterpret_cast<const uint2*>(vr)
                                                         : __ldg(reinterpret_cast<const uint2*>(vr));
                vraw[u][0] = vv.x, vraw[u][E / 2 - 1] = vv.y;
            } else {
                vraw[u][0] = rk < 0 ? 0u
                             : (from_smem || VSTAGE) ? *reinterpret_cast<const uint32_t*>(vr)
                                                     : __ldg(reinterpret_cast<const uint32_t*>(vr));
            }
        }
#pragma unroll
        for (int u = 0; u < 32; ++u) {
            unsigned short vf[E];
#pragma unroll
            for (int e = 0; e < E / 2; ++e) split_bf16(vraw[u][e], vf[2 * e], vf[2 * e + 1]);
#pragma unroll
            for (int hh = 0; hh < G; ++hh) {
                const unsigned short p = sm.ps[warp][hh][u];
#pragma unroll
                for (int e = 0; e < E; ++e) o[hh][e] = fma_bf16(p, vf[e], o[hh][e]);
            }
        }
#pragma unroll
        for (int hh = 0; hh < G; ++hh)
#pragma unroll
            for (int e = 0; e < E; ++e) sm.ho[warp][hh][lane * E + e] = o[hh][e];
    }
    __syncthreads();
    // The next kernel's blocks may come in now, not earlier: a GEMV's blocks open with a burst of weight copies into
    // every SM, and a key or value row of this block queued behind that burst arrives microseconds late.
    if (TRIGGER) pdl_launch_dependents();
    attn_finish<D, G>(A, sm, grp, hbase, G == GQ ? g : hbase, 0, first, last, &s_last_block);
}
