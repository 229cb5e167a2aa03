// The sampled pick: temperature, top-k, top-p and a hashed Gumbel-max draw over a row of logits, one launch.
//
// What it computes is btb's card sampler (native/cuda/btb_kernels.cu:1865-2124: btb_sample_max / _hist / _bin / _draw /
// _out / _keys) and, to the kept set, its CPU kernel (native/src/sample.rs:385-405): s = x / T; the top-k threshold is
// the k-th largest s found by a three-level radix select (11 + 11 + 10 of a float's 32 ordered bits) over integer
// counts; the top-p threshold the same select over masses exp(s - max) in 2^30 fixed point (exact u64 sums, so no
// order of summation changes it); the token is argmax(s + gumbel(key, i)) over the kept tokens, lowest index first.
//
// How it runs here: the reference spreads a row over the grid as up to fifteen launches with its histograms in global
// memory. Here a row belongs to one thread-block cluster of 8 CTAs. Each CTA keeps an eighth of the scaled row in its
// shared memory (read from global memory once), builds its private histogram there, and the eight histograms are
// summed through distributed shared memory after one cluster barrier a level; every CTA does the same scan of the same
// sums, so nothing is broadcast. Nine cluster barriers a pick, no global scratch, no atomics on global memory.
#include <cooperative_groups.h>

#include "btb_b200_internal.h"

namespace cg = cooperative_groups;

namespace {

constexpr int SMP_CTAS = 8;       // CTAs a cluster (the portable maximum)
constexpr int SMP_THREADS = 1024;
constexpr int SMP_BINS = 2048;
constexpr float SMP_MASS = 1073741824.0f;  // 2^30 a unit of mass
constexpr float SMP_FLOOR = -21.0f;        // this far under the top a token carries less than 2^-30

__device__ __forceinline__ unsigned smp_ordered(float f) {
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float smp_unordered(unsigned o) {
    return __uint_as_float((o & 0x80000000u) ? (o & 0x7FFFFFFFu) : ~o);
}
// exp(t), t <= 0: t = n ln2 + r with ln2 split in two, e^r a degree-7 series, 0 below -87 (sample.rs `fast_exp`).
// Every product and sum is rounded on its own (no contraction), as the host's scalar code rounds them.
__device__ __forceinline__ float smp_exp(float t) {
    if (t < -87.0f) return 0.0f;
    const float n = roundf(__fmul_rn(t, 1.4426950408889634f));
    const float r = __fsub_rn(__fsub_rn(t, __fmul_rn(n, 0.69314575f)), __fmul_rn(n, 1.4286068e-6f));
    float p = __fmul_rn(r, 0.0001984127f);
    p = __fmul_rn(r, __fadd_rn(0.001388889f, p));
    p = __fmul_rn(r, __fadd_rn(0.008333334f, p));
    p = __fmul_rn(r, __fadd_rn(0.041666668f, p));
    p = __fmul_rn(r, __fadd_rn(0.16666667f, p));
    p = __fmul_rn(r, __fadd_rn(0.5f, p));
    p = __fmul_rn(r, __fadd_rn(1.0f, p));
    p = __fadd_rn(1.0f, p);
    int e = (int)n + 127;
    e = e < 1 ? 1 : (e > 254 ? 254 : e);
    return __fmul_rn(__int_as_float((unsigned)e << 23), p);
}
__device__ __forceinline__ float smp_uniform(unsigned long long key, unsigned i) {
    unsigned long long h = key ^ ((unsigned long long)i * 0x9E3779B97F4A7C15ull);
    h ^= h >> 32;
    h *= 0xBF58476D1CE4E5B9ull;
    h ^= h >> 29;
    h *= 0x94D049BB133111EBull;
    h ^= h >> 32;
    return __fmul_rn(__fadd_rn((float)(unsigned)(h >> 41), 0.5f), 1.0f / 8388608.0f);  // 23 bits: never 1.0
}
__device__ __forceinline__ unsigned long long smp_mix_step(unsigned long long x, unsigned long long p) {
    x = (x ^ p) + 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    x ^= x >> 31;
    return x;
}
// btb/sampling.py `_mix` / `key_for`
__device__ __forceinline__ unsigned long long smp_key(unsigned long long seed, unsigned long long pos, unsigned salt) {
    unsigned long long x = smp_mix_step(smp_mix_step(0ull, seed), pos);
    if (salt) x = smp_mix_step(x, (unsigned long long)salt);
    return x & 0x7FFFFFFFFFFFFFFFull;
}
__device__ __forceinline__ unsigned long long smp_pack(float v, unsigned i) {
    return ((unsigned long long)smp_ordered(v) << 32) | (unsigned long long)(~i);
}

struct SampleArgs {
    const void* logits;
    long long ls;  // elements between rows
    int V, f32, top_k;
    unsigned salt;
    const float* fp;                 // [1/T, top_p] on the card
    const unsigned long long* keys;  // [R], or null: derived from seed and position
    const unsigned long long* seed;
    const int* n0p;
    const int* depth;
    long long* out;
    unsigned* floors;  // [R, 2] the top-k and top-p thresholds (ordered bits), or null
    unsigned long long* packed;  // [R] the winner as (ordered value << 32 | ~index), or null
    int per;           // a CTA's slice of the row
};

struct Shared {
    // this CTA's histogram of the level (two, so a level needs one barrier): a bin's 64-bit sum kept as two 32-bit words
    // - the masses' low 16 bits and the rest - because 32-bit shared atomics are native and 64-bit ones are not, and
    // a level's values crowd into a few bins (a CTA's eighth of a row cannot overflow either word)
    unsigned lo[2][SMP_BINS];
    unsigned hi[2][SMP_BINS];
    unsigned long long tot[SMP_BINS];      // the cluster's
    unsigned long long cs[64];
    unsigned long long best;
    unsigned long long carry;
    unsigned vmax, pre;
};

// One radix select over the cluster's row slices: mode 0 by count (target top_k), mode 1 by mass (target top_p of the
// mass at or above `floor`). Returns the threshold's ordered bits; every thread of every CTA returns the same value.
__device__ unsigned smp_select(cg::cluster_group& cl, Shared* S, const float* sv, int n, int mode, unsigned floor,
                               float M, unsigned top_k, float top_p, int& gen) {
    const unsigned tid = threadIdx.x;
    for (int level = 0; level < 3; ++level, ++gen) {
        unsigned* mine_lo = S->lo[gen & 1];
        unsigned* mine_hi = S->hi[gen & 1];
        const unsigned bits = level < 2 ? 11u : 10u;
        const unsigned shift = level == 0 ? 21u : (level == 1 ? 10u : 0u), hi = shift + bits;
        const unsigned prefix = level == 0 ? 0u : S->pre;
        for (unsigned b = tid; b < SMP_BINS; b += SMP_THREADS) mine_lo[b] = 0u, mine_hi[b] = 0u;
        __syncthreads();
        for (int i = tid; i < n; i += SMP_THREADS) {
            const float s = sv[i];
            const unsigned u = smp_ordered(s);
            if (u < floor) continue;
            if (hi < 32u && (u >> hi) != (prefix >> hi)) continue;
            const unsigned bin = (u >> shift) & (SMP_BINS - 1);
            if (mode == 0) {
                atomicAdd(&mine_lo[bin], 1u);
            } else if (s - M >= SMP_FLOOR) {
                const unsigned w = (unsigned)__fmul_rn(smp_exp(__fsub_rn(s, M)), SMP_MASS);  // at most 2^30
                if (w) {
                    atomicAdd(&mine_lo[bin], w & 0xFFFFu);
                    atomicAdd(&mine_hi[bin], w >> 16);
                }
            }
        }
        cl.sync();  // every CTA's histogram of this level is whole
        for (unsigned b = tid; b < SMP_BINS; b += SMP_THREADS) {
            unsigned long long a = 0ull;
#pragma unroll
            for (int c = 0; c < SMP_CTAS; ++c)
                a += (unsigned long long)cl.map_shared_rank(mine_lo, c)[b] + ((unsigned long long)cl.map_shared_rank(mine_hi, c)[b] << 16);
            S->tot[b] = a;
        }
        __syncthreads();
        if (tid < 64) {
            unsigned long long c = 0ull;
            for (unsigned j = 0; j < 32; ++j) c += S->tot[tid * 32 + j];
            S->cs[tid] = c;
        }
        __syncthreads();
        if (tid == 0) {
            unsigned long long target;
            if (level != 0) {
                target = S->carry;
            } else if (mode == 0) {
                target = (unsigned long long)top_k;
            } else {
                unsigned long long z = 0ull;
                for (int c = 0; c < 64; ++c) z += S->cs[c];
                target = (unsigned long long)__fmul_rn((float)z, top_p);
                if (!target) target = 1ull;  // at least the top token
            }
            // from the top: the chunk of 32 bins the running total first reaches the target in, then the bin
            unsigned long long acc = 0ull;
            int chunk = -1;
            for (int c = 63; c >= 0; --c) {
                acc += S->cs[c];
                if (acc >= target) {
                    chunk = c;
                    break;
                }
            }
            unsigned pick = 0;
            unsigned long long rem = target;
            if (chunk >= 0) {  // else fewer tokens (less mass) than asked for: the threshold stays at the bottom
                rem = target - (acc - S->cs[chunk]);
                unsigned long long a = 0ull;
                for (int b = chunk * 32 + 31; b >= chunk * 32; --b) {
                    const unsigned long long c = S->tot[b];
                    a += c;
                    if (a >= rem) {
                        pick = (unsigned)b;
                        rem -= a - c;
                        break;
                    }
                }
            }
            S->pre = prefix | (pick << shift);
            S->carry = rem;
        }
        __syncthreads();
    }
    return S->pre;
}

// What the pick and the verify share: the row's slice into shared memory, its max, the two thresholds, the key
struct RowFront {
    float M;
    unsigned floorK, floorP, floor;
    unsigned long long key;
    int lo, n;
};
__device__ __forceinline__ float smp_scaled(const SampleArgs& A, unsigned r, int i, float invT) {
    return A.f32 ? __fmul_rn(static_cast<const float*>(A.logits)[(size_t)r * A.ls + i], invT)
                 : __fmul_rn(bf2f(static_cast<const bf16*>(A.logits)[(size_t)r * A.ls + i]), invT);
}
__device__ RowFront smp_front(cg::cluster_group& cl, Shared* S, float* sv, const SampleArgs& A, unsigned r, unsigned rank) {
    const unsigned tid = threadIdx.x;
    RowFront F;
    F.lo = (int)rank * A.per;
    F.n = max(0, min(A.per, A.V - F.lo));
    const float invT = A.fp[0], top_p = A.fp[1];
    if (tid == 0) {
        S->vmax = 0u;
        S->best = 0ull;
    }
    __syncthreads();
    float m = NEG_INF;
    for (int i = tid; i < F.n; i += SMP_THREADS) {
        const float s = smp_scaled(A, r, F.lo + i, invT);
        sv[i] = s;
        m = fmaxf(m, s);
    }
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((tid & 31u) == 0) atomicMax(&S->vmax, smp_ordered(m));
    cl.sync();
    unsigned om = 0u;
    for (int c = 0; c < SMP_CTAS; ++c) om = max(om, *cl.map_shared_rank(&S->vmax, c));
    F.M = smp_unordered(om);
    int gen = 0;
    F.floorK = F.floorP = 0u;
    if (A.top_k > 0) F.floorK = smp_select(cl, S, sv, F.n, 0, 0u, F.M, (unsigned)A.top_k, top_p, gen);
    if (top_p < 1.0f) F.floorP = smp_select(cl, S, sv, F.n, 1, F.floorK, F.M, 0u, top_p, gen);
    F.floor = max(F.floorK, F.floorP);
    if (A.keys != nullptr) {
        F.key = A.keys[r];
    } else {
        const long long pos = (long long)*A.n0p + (A.depth != nullptr ? A.depth[r] : 0);
        F.key = smp_key(*A.seed, (unsigned long long)pos, A.salt);
    }
    return F;
}
// the Gumbel race over the kept tokens of this CTA's slice; after the cluster barrier every CTA's S->best is whole
__device__ __forceinline__ void smp_race(cg::cluster_group& cl, Shared* S, const float* sv, const RowFront& F) {
    const unsigned tid = threadIdx.x;
    unsigned long long best = 0ull;
    for (int i = tid; i < F.n; i += SMP_THREADS) {
        const float s = sv[i];
        if (smp_ordered(s) < F.floor || !(s - F.M >= SMP_FLOOR)) continue;
        const unsigned tok = (unsigned)(F.lo + i);
        const float v = __fsub_rn(s, logf(-logf(smp_uniform(F.key, tok))));
        if (v > NEG_INF) best = max(best, smp_pack(v, tok));
    }
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if ((tid & 31u) == 0 && best) atomicMax(&S->best, best);
    cl.sync();
}

__global__ void __cluster_dims__(SMP_CTAS, 1, 1) __launch_bounds__(SMP_THREADS) sample_pick(const SampleArgs A) {
    cg::cluster_group cl = cg::this_cluster();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Shared* S = reinterpret_cast<Shared*>(smem_raw);
    float* sv = reinterpret_cast<float*>(smem_raw + sizeof(Shared));
    const unsigned tid = threadIdx.x, rank = blockIdx.x, r = blockIdx.y;
    const RowFront F = smp_front(cl, S, sv, A, r, rank);
    smp_race(cl, S, sv, F);
    if (rank == 0 && tid == 0) {
        unsigned long long b = 0ull;
        for (int c = 0; c < SMP_CTAS; ++c) b = max(b, *cl.map_shared_rank(&S->best, c));
        // nothing in the race: token 0, as the host's
        if (A.out != nullptr) A.out[r] = b ? (long long)(~(unsigned)(b & 0xFFFFFFFFull)) : 0ll;
        if (A.packed != nullptr) A.packed[r] = b;
        if (A.floors != nullptr) {
            A.floors[2 * r] = F.floorK;
            A.floors[2 * r + 1] = F.floorP;
        }
    }
    cl.sync();  // no CTA leaves while a peer may still read its shared memory
}

// ---- the verify pass's pick: exact rejection sampling at a tree node (native/cuda/btb_kernels.cu:2126-2359
// btb_sample_verify; btb/sampling.py:272-372 `Verify`). A row is a node with up to 32 drafted children in draw order.
// Where the drafts are point masses (hasq 0) the node draws from the target and the child that equals the draw is
// accepted. Where the drafter gave a distribution q, child i is accepted when u_i * q_i(c) < p_i(c): p_0 the target
// over the kept tokens, p_{i+1} = norm(max(0, p_i - q_i)), q_i = q with the earlier children taken out; when no child
// is accepted the node draws from the last residual. Either way the emitted token is a draw from the target.
//
// The thresholds and the point-mass race are the pick's (the cluster of eight). The trials' sums are floating point,
// so their order is part of the result: they run on the cluster's first CTA alone as the reference's one block of 1024
// threads does - thread t adds tokens t, t + 1024, ... in order, a warp folds by halving strides, the 32 warps' sums
// are added in order - reading the row where it lies (it is in L2 by then).
constexpr int SMP_KIDS = 32;

struct VerifyArgs {
    SampleArgs P;
    const float* q;  // [R, Vd] the drafter's masses a node
    const int* kids;  // [R, C] children in draw order, -1 after the last
    const unsigned* hasq;
    unsigned* out;  // [R] (accepted slot + 1) << 24 | token; slot 0: none accepted
    int Vd, C;
};

struct VerifyShared {
    float red[SMP_THREADS / 32];
    float total;
    float zp[SMP_KIDS + 1], zq[SMP_KIDS + 1];
    int kid[SMP_KIDS];
    unsigned long long won;
};

// the sum of every thread's `part`, in the fixed order above; every thread returns it
__device__ __forceinline__ float smp_block_sum(VerifyShared* W, float part) {
    const unsigned tid = threadIdx.x;
    for (int o = 16; o > 0; o >>= 1) part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, o));
    if ((tid & 31u) == 0) W->red[tid >> 5] = part;
    __syncthreads();
    if (tid == 0) {
        float z = 0.0f;
        for (int w = 0; w < SMP_THREADS / 32; ++w) z = __fadd_rn(z, W->red[w]);
        W->total = z;
    }
    __syncthreads();
    const float z = W->total;
    __syncthreads();  // `total` and `red` are free again
    return z;
}

// token x's mass after `k` rejected trials: exp(s - M) if kept, then k times max(0, w / zp[j] - q'(x) / zq[j]) with q'
// losing x's mass once x was itself the tried child
__device__ __forceinline__ float smp_left(const VerifyArgs& A, const VerifyShared* W, unsigned r, const float* qrow,
                                          unsigned x, int k, float invT, float M, unsigned floor) {
    const float s = smp_scaled(A.P, r, (int)x, invT);
    float w = smp_ordered(s) >= floor ? smp_exp(__fsub_rn(s, M)) : 0.0f;
    float qx = x < (unsigned)A.Vd ? qrow[x] : 0.0f;
    for (int j = 0; j < k; ++j) {
        w = fmaxf(0.0f, __fsub_rn(__fdiv_rn(w, W->zp[j]), __fdiv_rn(qx, W->zq[j])));
        if (W->kid[j] == (int)x) qx = 0.0f;
    }
    return w;
}

__global__ void __cluster_dims__(SMP_CTAS, 1, 1) __launch_bounds__(SMP_THREADS) sample_verify(const VerifyArgs A) {
    cg::cluster_group cl = cg::this_cluster();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Shared* S = reinterpret_cast<Shared*>(smem_raw);
    float* sv = reinterpret_cast<float*>(smem_raw + sizeof(Shared));
    __shared__ VerifyShared W;
    const unsigned tid = threadIdx.x, rank = blockIdx.x, r = blockIdx.y;
    const RowFront F = smp_front(cl, S, sv, A.P, r, rank);
    const bool drawn = A.hasq[r] != 0u;  // the same for every CTA of the row
    if (!drawn) smp_race(cl, S, sv, F);
    if (rank == 0 && tid == 0) {
        unsigned long long b = 0ull;
        if (!drawn)
            for (int c = 0; c < SMP_CTAS; ++c) b = max(b, *cl.map_shared_rank(&S->best, c));
        W.won = b;
    }
    cl.sync();  // the peers' shared memory is not read after this: they may leave
    if (rank != 0) return;
    for (int c = tid; c < SMP_KIDS; c += SMP_THREADS) W.kid[c] = c < A.C ? A.kids[(size_t)r * A.C + c] : -1;
    __syncthreads();

    if (!drawn) {
        if (tid == 0) {
            const unsigned tok = W.won ? ~(unsigned)(W.won & 0xFFFFFFFFull) : 0u;
            unsigned slot = 0u;
            for (int c = 0; c < A.C; ++c)
                if (W.kid[c] >= 0 && (unsigned)W.kid[c] == tok) {
                    slot = (unsigned)c + 1u;
                    break;
                }
            A.out[r] = (slot << 24) | tok;
        }
        return;
    }

    const float invT = A.P.fp[0];
    const float* qrow = A.q + (size_t)r * A.Vd;
    const int V = A.P.V;
    // zp[0]: the target's mass over the kept tokens; zq[0]: the drafter's over its vocabulary
    float part = 0.0f;
    for (int i = tid; i < V; i += SMP_THREADS) {
        const float s = smp_scaled(A.P, r, i, invT);
        if (smp_ordered(s) >= F.floor) part = __fadd_rn(part, smp_exp(__fsub_rn(s, F.M)));
    }
    const float z0 = smp_block_sum(&W, part);
    part = 0.0f;
    for (int i = tid; i < A.Vd; i += SMP_THREADS) part = __fadd_rn(part, qrow[i]);
    const float q0 = smp_block_sum(&W, part);
    if (tid == 0) {
        W.zp[0] = z0;
        W.zq[0] = q0;
    }
    __syncthreads();

    // the trials, every thread deciding alike
    int tried = 0;
    unsigned accepted = 0u, token = 0u;
    for (int i = 0; i < A.C; ++i) {
        const int c = W.kid[i];
        if (c < 0) break;
        const float zqi = W.zq[i];
        const float qc = (c < A.Vd && zqi > 0.0f) ? fminf(__fdiv_rn(qrow[c], zqi), 1.0f) : 0.0f;
        if (!(qc > 0.0f)) break;  // a child the drafter gives no mass was no draw of its: the trials end
        const float pc = __fdiv_rn(smp_left(A, &W, r, qrow, (unsigned)c, i, invT, F.M, F.floor), W.zp[i]);
        const float u = smp_uniform(F.key, 0xF00000u + (unsigned)i);
        if (__fmul_rn(u, qc) < pc) {
            accepted = (unsigned)i + 1u, token = (unsigned)c;
            break;
        }
        part = 0.0f;
        for (int x = tid; x < V; x += SMP_THREADS)
            part = __fadd_rn(part, smp_left(A, &W, r, qrow, (unsigned)x, i + 1, invT, F.M, F.floor));
        // smp_left(.., i + 1, ..) reads zp[i] and zq[i] only: the entries this pass is about to add are not read yet
        const float z = smp_block_sum(&W, part);
        if (tid == 0) {
            W.zp[i + 1] = z;
            W.zq[i + 1] = __fsub_rn(zqi, qrow[c]);
        }
        __syncthreads();
        if (!(z > 0.0f)) {  // nothing left: the target was the drafter's distribution, the rejection was rounding
            accepted = (unsigned)i + 1u, token = (unsigned)c;
            break;
        }
        tried = i + 1;
    }
    if (accepted) {
        if (tid == 0) A.out[r] = (accepted << 24) | token;
        return;
    }
    // none accepted: a draw from what is left after every trial
    unsigned long long best = 0ull;
    for (int x = tid; x < V; x += SMP_THREADS) {
        const float w = smp_left(A, &W, r, qrow, (unsigned)x, tried, invT, F.M, F.floor);
        if (!(w > 0.0f)) continue;
        const float v = __fadd_rn(logf(w), -logf(-logf(smp_uniform(F.key, (unsigned)x))));
        if (v > NEG_INF) best = max(best, smp_pack(v, (unsigned)x));
    }
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if (tid == 0) W.won = 0ull;
    __syncthreads();
    if ((tid & 31u) == 0 && best) atomicMax(&W.won, best);
    __syncthreads();
    if (tid == 0) A.out[r] = W.won ? ~(unsigned)(W.won & 0xFFFFFFFFull) : 0u;
}

// btb_sample_out (native/cuda/btb_kernels.cu:2110-2114): the token of a packed winner
struct OutArgs {
    const unsigned long long* packed;
    unsigned* out;
    int R;
};
__global__ void sample_out_k(const OutArgs A) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < A.R) A.out[r] = ~(unsigned)(A.packed[r] & 0xFFFFFFFFull);
}

// btb_sample_keys (native/cuda/btb_kernels.cu:2116-2124): keys[0..1] = key_for(seed, pos[0], salt) as (lo, hi)
struct KeysArgs {
    const unsigned* seed;
    const int* pos;
    unsigned salt;
    unsigned* keys;
};
__global__ void sample_keys_k(const KeysArgs A) {
    if (blockIdx.x || threadIdx.x) return;
    const unsigned long long sd = ((unsigned long long)A.seed[1] << 32) | (unsigned long long)A.seed[0];
    const unsigned long long k = smp_key(sd, (unsigned long long)(unsigned)A.pos[0], A.salt);
    A.keys[0] = (unsigned)(k & 0xFFFFFFFFull);
    A.keys[1] = (unsigned)(k >> 32);
}

}  // namespace

B2_DEFINE_STATUS(sample)

extern "C" int btb_b200_sample_keys(const void* seed, const void* pos, unsigned salt, void* keys, void* stream) {
    if (!seed || !pos || !keys) return B2_ERR_NULL;
    KeysArgs a{static_cast<const unsigned*>(seed), static_cast<const int*>(pos), salt, static_cast<unsigned*>(keys)};
    return b2_launch((const void*)sample_keys_k, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), a, 0);
}

extern "C" int btb_b200_sample_out(const void* packed, void* out, int R, void* stream) {
    if (!packed || !out) return B2_ERR_NULL;
    if (R <= 0) return B2_ERR_DOMAIN;
    OutArgs a{static_cast<const unsigned long long*>(packed), static_cast<unsigned*>(out), R};
    return b2_launch((const void*)sample_out_k, dim3((R + 255) / 256), dim3(256), 0, static_cast<cudaStream_t>(stream), a, 0);
}

extern "C" int btb_b200_sample_pick(const void* logits, int f32_logits, int R, int V, long long ls, const void* fp,
                                    int top_k, const void* keys, const void* seed, const void* n0p, const void* depth,
                                    unsigned salt, void* out, void* floors, void* packed, void* stream) {
    if (!logits || !fp || (!out && !packed)) return B2_ERR_NULL;
    if (!keys && (!seed || !n0p)) return B2_ERR_NULL;
    if (R <= 0 || R > 65535 || V <= 0 || ls < V || top_k < 0) return B2_ERR_DOMAIN;
    const int per = (V + SMP_CTAS - 1) / SMP_CTAS;
    const size_t smem = sizeof(Shared) + (size_t)per * sizeof(float);
    if (smem > 227 * 1024) return B2_ERR_DOMAIN;  // a row's eighth must fit a CTA's shared memory
    static bool allowed[64] = {};
    if (const int rc = b2_allow_smem((const void*)sample_pick, allowed)) return rc;
    SampleArgs a{logits, ls, V, f32_logits, top_k, salt, static_cast<const float*>(fp),
                 static_cast<const unsigned long long*>(keys), static_cast<const unsigned long long*>(seed),
                 static_cast<const int*>(n0p), static_cast<const int*>(depth), static_cast<long long*>(out),
                 static_cast<unsigned*>(floors), static_cast<unsigned long long*>(packed), per};
    // the cluster shape is the kernel's own (__cluster_dims__); the grid is whole clusters
    return b2_launch((const void*)sample_pick, dim3(SMP_CTAS, R), dim3(SMP_THREADS), smem, static_cast<cudaStream_t>(stream), a, 0);
}

extern "C" int btb_b200_sample_verify(const void* logits, int f32_logits, int R, int V, long long ls, const void* q, int Vd,
                                      const void* kids, int C, const void* hasq, const void* keys, int top_k,
                                      const void* fp, void* out, void* stream) {
    if (!logits || !q || !hasq || !keys || !fp || !out || (C > 0 && !kids)) return B2_ERR_NULL;
    if (R <= 0 || R > 65535 || V <= 0 || V > 0xFFFFFF || ls < V || Vd < 0 || C < 0 || C > SMP_KIDS || top_k < 0) return B2_ERR_DOMAIN;
    const int per = (V + SMP_CTAS - 1) / SMP_CTAS;
    const size_t smem = sizeof(Shared) + (size_t)per * sizeof(float);
    if (smem + sizeof(VerifyShared) > 227 * 1024) return B2_ERR_DOMAIN;
    static bool allowed[64] = {};
    if (const int rc = b2_allow_smem((const void*)sample_verify, allowed)) return rc;
    VerifyArgs a{};
    a.P = SampleArgs{logits, ls, V, f32_logits, top_k, 0u, static_cast<const float*>(fp),
                     static_cast<const unsigned long long*>(keys), nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, per};
    a.q = static_cast<const float*>(q);
    a.kids = static_cast<const int*>(kids);
    a.hasq = static_cast<const unsigned*>(hasq);
    a.out = static_cast<unsigned*>(out);
    a.Vd = Vd, a.C = C;
    return b2_launch((const void*)sample_verify, dim3(SMP_CTAS, R), dim3(SMP_THREADS), smem, static_cast<cudaStream_t>(stream), a, 0);
}
