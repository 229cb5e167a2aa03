// The tensor-core matvec for passes of up to 32 rows (verify trees, prefill chunks, small batches):
// y[m][r] = bf16(sum_c w[r][c] x[m][c]) on the 5th-generation tensor cores.
//
// What it stands in for is btb's btb_gemv_mma_bf16 (native/cuda/btb_gemv_mma.cuh:123-315): one kernel for every pass
// width, x padded to 32 rows, each output one accumulation over all of k, so that a row's bits do not depend on how
// many rows share the pass. Like the reference's, its summation order is its own: results agree with the fp32-chain
// GEMV to rounding, not to the bit (neither did the reference's two families), and a caller keeps ONE family for the
// passes whose rows it compares bit for bit.
//
// How it runs on sm_100a: the pass is the GEMM y^T[R, 32] = W[R, C] x^T[C, 32]. A CTA owns a tile of 128 weight rows
// (the MMA's M) over a range of K. TMA tensor maps bring a [128 x 64] tile of W and the [32 x 64] tile of x (rows past
// the pass's M read as zeros, columns past C too) into shared memory under the 128-byte swizzle, one elected thread
// issues tcgen05.mma (M 128, N 32, K 16, bf16 in, f32 accumulate) four times a stage with the accumulator in tensor
// memory, tcgen05.commit hands the stage back to the producer through an mbarrier, and the epilogue reads the 128 x 32
// accumulator with tcgen05.ld (a weight row a thread) and writes bf16. Matrices of few tiles (2560 rows: 20) split K
// over gridDim.y; the partial sums meet in a second, ordered pass (the same order every launch). No cluster
// multicast; every wait is bounded and a CTA that gives up still frees its tensor memory.
#include <cuda.h>

#include <mutex>
#include <unordered_map>
#include <utility>

#include "btb_b200_internal.h"
#include "gemv_core.cuh"

B2_DEFINE_STATUS(tc)

namespace {

constexpr int TC_BM = 128;  // weight rows a tile (the MMA's M)
constexpr int TC_BN = 32;   // x rows a tile of the matvec, padded (the MMA's N); the prefill GEMM takes up to 256
constexpr int TC_BK = 64;   // columns a stage: one 128-byte swizzle span of bf16
constexpr int TC_STAGES_MAX = 10;  // ring depth at most; the launch picks (four stages let two CTAs share an SM)
constexpr int A_BYTES = TC_BM * TC_BK * 2;
template <int BN>
struct TcTile {
    static constexpr int B_BYTES = BN * TC_BK * 2, ST_BYTES = A_BYTES + B_BYTES;
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(tm), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
// a K-major operand tile in shared memory: rows of 128 bytes under the 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);  // start address, in 16-byte units
    d |= (uint64_t)1 << 16;                    // leading byte offset (not used by a swizzled K-major tile)
    d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset: the next 8-row group
    d |= (uint64_t)1 << 46;                    // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                    // layout: 128-byte swizzle
    return d;
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
        "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

struct TcArgs {
    bf16* y;      // [M, R]
    float* part;  // [splits, 32, R] partial sums when splits > 1
    int R, C, M, kblocks_per_split, splits, stages;
    // the gate/up form: the matrix is [2 * glu_I, C] (gate rows, then up rows); a tile takes 64 gate rows and, glu_I rows
    // on, their 64 up rows, and writes m [M, glu_I] = bf16(bf16(silu(bf16 g)) * bf16 u). 0: the plain matvec.
    int glu_I;
    // the plain matvec cut over K: a counter a tile (zero between launches); the CTA that finds the others' partial sums
    // all written adds them, in range order, itself
    int* cnt;
};

// BN: the x rows a CTA's tile holds. GEMM false: the matvec - one accumulator of 32 columns, gridDim.y cuts K into
// ranges whose partial sums a second launch adds in range order. GEMM true: the prefill GEMM - gridDim.y walks the x
// rows BN at a time and the CTA takes its tile's whole K, but in the matvec's own ranges: range s accumulates into its
// own BN columns of tensor memory and the epilogue adds the ranges in order, so an output element is the matvec's sum
// to the bit whatever the chunk's size and wherever in the chunk the row stands.
__device__ __forceinline__ float tc_silu(float g) { return g / (1.f + expf(-g)); }

constexpr int TC_WS_HEAD = 1024;  // the workspace's first bytes: the tiles' counters (a split matrix has at most 148 tiles)

// The end of a matvec CTA whose tile is cut over K (every thread of the CTA calls it, after its partial sums are
// written): the CTA that arrives last on the tile's counter adds the ranges' partial sums in range order - the same sum
// every launch, rounded to bf16 once - and leaves the counter at zero for the next launch. A CTA that gave up counts
// too (the status word already says so), so that a failed launch does not leave a counter standing. NT threads: thread
// t takes row t % 128 and the x rows t / 128, + NT / 128, ..; two x rows' loads (up to 32) are in flight at once - summed
// one load after the other, the job took longer than a second launch.
template <int NT>
__device__ __forceinline__ void tc_finish_split(const TcArgs& A, int row0, int* s_last) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) *s_last = atomicAdd(A.cnt + blockIdx.x, 1) == A.splits - 1;
    __syncthreads();
    if (!*s_last) return;
    __threadfence();
    constexpr int NG = NT / TC_BM;  // x rows in work at once
    const int row = row0 + ((int)threadIdx.x & (TC_BM - 1)), g = (int)threadIdx.x / TC_BM;
    if (g < NG && row < A.R) {
        for (int n = g; n < A.M; n += 2 * NG) {
            float v[2][16];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int k = 0; k < 16; ++k)
                    v[j][k] = (k < A.splits && n + j * NG < A.M) ? __ldcg(A.part + ((size_t)k * 32 + n + j * NG) * A.R + row) : 0.f;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                if (n + j * NG >= A.M) break;
                float s = 0.f;
#pragma unroll
                for (int k = 0; k < 16; ++k)
                    if (k < A.splits) s += v[j][k];
                A.y[(size_t)(n + j * NG) * A.R + row] = f2bf(s);
            }
        }
    }
    if (threadIdx.x == 0) A.cnt[blockIdx.x] = 0;
}

template <int BN, bool GEMM>
__global__ void __launch_bounds__(128, GEMM ? 1 : 2) gemv_tc(const __grid_constant__ CUtensorMap tmW,
                                                             const __grid_constant__ CUtensorMap tmX, const TcArgs A) {
    constexpr int ST_BYTES = TcTile<BN>::ST_BYTES;
    __shared__ float s_up[GEMM ? 1 : 64][GEMM ? 1 : 33];  // the gate/up form: a tile's up outputs on their way to the gate rows' threads
    const bool glu = !GEMM && A.glu_I > 0;
    const int ranges = GEMM ? A.splits : 1;  // accumulators in tensor memory
    const uint32_t tmem_cols = GEMM ? 512u : 32u;
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t full[TC_STAGES_MAX], empty[TC_STAGES_MAX], done;
    const int TC_STAGES = A.stages;
    __shared__ uint32_t tmem_slot;
    __shared__ int s_fail;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~(uintptr_t)1023);
    const int row0 = glu ? blockIdx.x * 64 : blockIdx.x * TC_BM;  // (the gate/up form: the tile's first gate row)
    const int total_kb = (A.C + TC_BK - 1) / TC_BK;
    const int kb0 = GEMM ? 0 : blockIdx.y * A.kblocks_per_split;
    const int nkb = GEMM ? total_kb : max(0, min(A.kblocks_per_split, total_kb - kb0));
    const int n0 = GEMM ? blockIdx.y * BN : 0;  // the tile's first x row

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        mbar_init(smem_u32(&done), 1);
        s_fail = 0;
        mbar_fence_init();
    }
    if (warp == 0) {  // the accumulators' columns of tensor memory (the GEMM takes the SM's whole 512: one CTA an SM)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    pdl_launch_dependents();
    pdl_wait();  // x is the kernel's before this one

    // (The two loops below are single threads: what a K block costs them is their instruction count times the issue
    // latency of a lone thread, so nothing is recomputed a block - the stage and its phase are running counters, not a
    // division by the ring's depth, and addresses, coordinates and descriptors advance by additions.)
    if (warp == 0 && lane == 0) {
        // the producer: the weights' tile and x's tile of every K block of this CTA's range
        const uint32_t tiles0 = smem_u32(tiles), full0 = smem_u32(&full[0]), empty0 = smem_u32(&empty[0]);
        int s = 0, wrapped = 0;
        uint32_t ph = 0;
        int xk = kb0 * TC_BK;  // the K block's first column
        for (int kb = 0; kb < nkb; ++kb, xk += TC_BK) {
            if (wrapped && !mbar_wait_bounded(empty0 + s * 8, ph ^ 1)) {
                *(volatile int*)&s_fail = 1;
                break;
            }
            const uint32_t bar = full0 + s * 8, at = tiles0 + s * ST_BYTES;
            mbar_expect_tx(bar, ST_BYTES);
            if (glu) {  // two boxes of 64 rows: the gate rows into the tile's upper half, their up rows into its lower half
                tma_load_2d(at, &tmW, xk, row0, bar);
                tma_load_2d(at + A_BYTES / 2, &tmW, xk, A.glu_I + row0, bar);
            } else {
                tma_load_2d(at, &tmW, xk, row0, bar);
            }
            tma_load_2d(at + A_BYTES, &tmX, xk, n0, bar);
            if (++s == TC_STAGES) s = 0, ph ^= 1, wrapped = 1;
        }
    } else if (warp == 1 && lane == 0) {
        // the issuer: four K = 16 instructions a stage; D f32, A and B bf16, both K-major, N = 32, M = 128
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
        // a stage's descriptors are the first stage's plus the stage's offset in the address field (16-byte units; the
        // ring lies below 256 KB, so the field never carries), a K = 16 step 32 bytes further
        const uint64_t da0 = umma_desc_sw128(smem_u32(tiles)), db0 = umma_desc_sw128(smem_u32(tiles) + A_BYTES);
        const uint32_t full0 = smem_u32(&full[0]), empty0 = smem_u32(&empty[0]);
        int s = 0;
        uint32_t ph = 0;
        int rs = 0, first = 0;  // the GEMM's K block kb belongs to range kb / kps: its own accumulator, started afresh at the range's first block
        for (int kb = 0; kb < nkb; ++kb) {
            if (!mbar_wait_bounded(full0 + s * 8, ph)) {
                *(volatile int*)&s_fail = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t da = da0 + (uint64_t)(s * (ST_BYTES >> 4)), db = db0 + (uint64_t)(s * (ST_BYTES >> 4));
#pragma unroll
            for (int k = 0; k < TC_BK / 16; ++k)
                umma_bf16(tmem + (uint32_t)(rs * BN), da + 2 * k, db + 2 * k, idesc, (first | k) != 0);
            umma_commit(empty0 + s * 8);  // the stage is free once these have read it
            if (++s == TC_STAGES) s = 0, ph ^= 1;
            if (GEMM) {
                if (++first == A.kblocks_per_split) first = 0, ++rs;
            } else {
                first = 1;
            }
        }
        umma_commit(smem_u32(&done));
    }
    __syncwarp();
    // the epilogue: warp w reads lanes 32 w .. 32 w + 31 (a weight row a thread); the 32 columns are the x rows
    bool ok = true;
    if (nkb > 0) ok = mbar_wait_bounded(smem_u32(&done), 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok && nkb > 0 && !*(volatile int*)&s_fail) {
        const int row = row0 + warp * 32 + lane;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
            if (GEMM && n0 + c0 >= A.M) break;  // x rows past the pass
            uint32_t r[32];
            float tot[32];
#pragma unroll
            for (int n = 0; n < 32; ++n) tot[n] = 0.f;
#pragma unroll 1
            for (int rs = 0; rs < ranges; ++rs) {
            const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(rs * BN + c0);
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, "
                "%24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                  "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
                  "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
                  "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                : "r"(taddr));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int n = 0; n < 32; ++n) tot[n] += __uint_as_float(r[n]);  // the ranges in order, from zero
            }
            if (!GEMM && glu) {
                // thread l < 64 holds gate row row0 + l, thread 64 + l its up row
                const int l = warp * 32 + lane;
                if (A.splits == 1) {
                    if (l >= 64) {
#pragma unroll
                        for (int n = 0; n < 32; ++n) s_up[GEMM ? 0 : l - 64][GEMM ? 0 : n] = tot[n];
                    }
                    __syncthreads();
                    if (l < 64 && row0 + l < A.glu_I) {
#pragma unroll
                        for (int n = 0; n < 32; ++n)
                            if (n < A.M) {
                                const float g = bfround(tot[n]), u = bfround(s_up[GEMM ? 0 : l][GEMM ? 0 : n]);
                                A.y[(size_t)n * A.glu_I + row0 + l] = f2bf(bfround(tc_silu(g)) * u);
                            }
                    }
                } else {  // partial sums by tile position: [split][n][tile * 128 + l]
                    const size_t Rv = (size_t)gridDim.x * TC_BM;
#pragma unroll
                    for (int n = 0; n < 32; ++n)
                        if (n < A.M) A.part[((size_t)blockIdx.y * 32 + n) * Rv + (size_t)blockIdx.x * TC_BM + l] = __uint_as_float(r[n]);
                }
            } else if (row < A.R) {
                if (GEMM || A.splits == 1) {
#pragma unroll
                    for (int n = 0; n < 32; ++n)
                        if (n0 + c0 + n < A.M) A.y[(size_t)(n0 + c0 + n) * A.R + row] = f2bf(tot[n]);
                } else {
#pragma unroll
                    for (int n = 0; n < 32; ++n)
                        if (n < A.M) A.part[((size_t)blockIdx.y * 32 + n) * A.R + row] = __uint_as_float(r[n]);
                }
            }
        }
    } else if (threadIdx.x == 0 && nkb > 0) {
        b2_fail(B2_ERR_TIMEOUT);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
    if (!GEMM && !glu && A.splits > 1 && A.cnt != nullptr) tc_finish_split<128>(A, row0, &s_fail);  // (the flag's word is free by now)
}

// ---- the same matvec over pack12 weights read as stored ----------------------------------------------------------------------
// The weights' tile cannot be copied into the MMA's operand layout by TMA: it does not exist as bf16 anywhere. Here TMA
// brings the tile's stored parts - 128 rows x 64 low bytes and 128 rows x 32 bytes of codes - into a staging area, eight
// more warps (a 16-byte piece of a row a thread) widen them in registers (p12_chunk: the GEMV's own widen, escapes from the row's
// list) and write the bf16 tile into shared memory in the 128-byte-swizzled layout the MMA reads (16-byte piece c of row
// d at piece c ^ (d & 7)), make it visible to the async proxy, meet on a named barrier and one of them counts the tile
// in on the stage's second mbarrier; the issuer waits for that one. No widened copy is ever in global memory, and the
// sums are btb_b200_gemv_tc_bf16's over the widened matrix to the bit (the operands are the same bits in the same places).
//
// What bounds it is not memory: with the loads, the widening and the MMAs all taken out, a K block still cost about
// half a microsecond of barrier hand-offs (wait, named barrier, arrive, the issuer's wait and commit, the producer's
// wait), whatever the ring's depth, and the widening's own dependent chain added as much again in series. Hence one
// arrival a tile instead of one a thread, and two groups of wideners on alternate K blocks, so that one group's
// hand-offs run under the other's arithmetic.
constexpr int P12_LO = TC_BM * TC_BK;          // a stage's low bytes
constexpr int P12_HI = TC_BM * TC_BK / 2;      // ... and codes
constexpr int P12_B = TC_BN * TC_BK * 2;       // x's tile
constexpr int P12_ST = A_BYTES + P12_B + P12_LO + P12_HI;
struct TcP12Args {
    TcArgs t;
    uint32_t table[4];
    const int32_t* esc_idx;
    const uint8_t* esc_val;
    const int32_t* esc_row;  // [R + 1] or null: no escapes anywhere
};

// one 16-byte piece of the operand tile from its stored parts, row I * RG on from the thread's first: the offsets are
// immediates of the shared-space loads and the store (one address each a stage, not one a row)
template <int I, int RG>
__device__ __forceinline__ void p12_widen_row(uint32_t a_lo, uint32_t a_hi, uint32_t a_out, const uint32_t (&table)[4]) {
    uint32_t l0, l1, codes;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2+%3];" : "=r"(l0), "=r"(l1) : "r"(a_lo), "n"(I * RG * TC_BK) : "memory");
    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(codes) : "r"(a_hi), "n"(I * RG * (TC_BK / 2)) : "memory");
    uint32_t wp[4];
    p12_chunk(l0, l1, codes, table, wp);
    asm volatile("st.shared.v4.u32 [%0+%1], {%2, %3, %4, %5};" ::"r"(a_out), "n"(I * RG * 128), "r"(wp[0]), "r"(wp[1]), "r"(wp[2]),
                 "r"(wp[3])
                 : "memory");
}
template <int RG, int... Is>
__device__ __forceinline__ void p12_widen_rows(uint32_t a_lo, uint32_t a_hi, uint32_t a_out, const uint32_t (&table)[4],
                                               std::integer_sequence<int, Is...>) {
    (p12_widen_row<Is, RG>(a_lo, a_hi, a_out, table), ...);
}

// one group's named barrier (ids 1 ..): true if any of its `GT` threads came with `bad`
template <int ID, int GT>
__device__ __forceinline__ int p12_group_bar(bool bad) {
    int any_bad;
    asm volatile("{\n.reg .pred q, r;\nsetp.ne.b32 q, %1, 0;\nbar.red.or.pred r, %3, %2, q;\nselp.b32 %0, 1, 0, r;\n}\n"
                 : "=r"(any_bad)
                 : "r"((int)bad), "n"(GT), "n"(ID)
                 : "memory");
    return any_bad;
}

template <int NW, int NG>
__global__ void __launch_bounds__(128 + 32 * NW, 2) gemv_tc_p12(const __grid_constant__ CUtensorMap tmLo,
                                                      const __grid_constant__ CUtensorMap tmHi,
                                                      const __grid_constant__ CUtensorMap tmX, const TcP12Args P) {
    const TcArgs& A = P.t;
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_p[TC_STAGES_MAX], full_a[TC_STAGES_MAX], empty[TC_STAGES_MAX], done;
    __shared__ uint32_t tmem_slot;
    __shared__ int s_fail;
    const int TC_STAGES = A.stages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~(uintptr_t)1023);
    const int row0 = blockIdx.x * TC_BM;
    const int total_kb = A.C / TC_BK;  // (whole K blocks: the host checks)
    const int kb0 = blockIdx.y * A.kblocks_per_split;
    const int nkb = max(0, min(A.kblocks_per_split, total_kb - kb0));
    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(smem_u32(&full_p[s]), 1);
            mbar_init(smem_u32(&full_a[s]), 1);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        mbar_init(smem_u32(&done), 1);
        s_fail = 0;
        mbar_fence_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(32u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    pdl_launch_dependents();
    pdl_wait();

    // (single-thread loops: running counters and additions, as in gemv_tc)
    if (warp == 0 && lane == 0) {
        // the producer: the stored parts of the weights' tile and x's tile
        const uint32_t tiles0 = smem_u32(tiles), full0 = smem_u32(&full_p[0]), empty0 = smem_u32(&empty[0]);
        int s = 0, wrapped = 0;
        uint32_t ph = 0;
        int xk = kb0 * TC_BK;
        for (int kb = 0; kb < nkb; ++kb, xk += TC_BK) {
            if (wrapped && !mbar_wait_bounded(empty0 + s * 8, ph ^ 1)) {
                *(volatile int*)&s_fail = 1;
                break;
            }
            const uint32_t bar = full0 + s * 8, at = tiles0 + s * P12_ST;
            mbar_expect_tx(bar, P12_B + P12_LO + P12_HI);
            tma_load_2d(at + A_BYTES + P12_B, &tmLo, xk, row0, bar);
            tma_load_2d(at + A_BYTES + P12_B + P12_LO, &tmHi, xk >> 1, row0, bar);
            tma_load_2d(at + A_BYTES, &tmX, xk, 0, bar);
            if (++s == TC_STAGES) s = 0, ph ^= 1, wrapped = 1;
        }
    } else if (warp == 1 && lane == 0) {
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
        const uint64_t da0 = umma_desc_sw128(smem_u32(tiles)), db0 = umma_desc_sw128(smem_u32(tiles) + A_BYTES);
        const uint32_t full0 = smem_u32(&full_a[0]), empty0 = smem_u32(&empty[0]);
        int s = 0;
        uint32_t ph = 0;
        for (int kb = 0; kb < nkb; ++kb) {
            if (!mbar_wait_bounded(full0 + s * 8, ph)) {  // every row of the tile widened (and x landed before that)
                *(volatile int*)&s_fail = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t da = da0 + (uint64_t)(s * (P12_ST >> 4)), db = db0 + (uint64_t)(s * (P12_ST >> 4));
#pragma unroll
            for (int k = 0; k < TC_BK / 16; ++k) umma_bf16(tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
            umma_commit(empty0 + s * 8);
            if (++s == TC_STAGES) s = 0, ph ^= 1;
        }
        umma_commit(smem_u32(&done));
    } else if (warp >= 4) {
        // the wideners: NG groups of NW / NG warps that take the tile's K blocks in turn (group g the blocks kb = g, g + NG,
        // ...), so that one group's barrier round trips run under the other's arithmetic. A thread takes 16-byte piece
        // c of rows (tg >> 3) + RG i: a warp's lanes read four consecutive rows' stored bytes (256 and 128 contiguous bytes)
        // and write four whole rows of the operand tile - no bank conflicts anywhere.
        constexpr int GT = NW * 32 / NG;  // threads a group
        const int t = threadIdx.x - 128, grp = t / GT, tg = t - grp * GT, c = tg & 7;
        constexpr int RG = GT / 8;       // rows in work at once: eight lanes a row
        constexpr int RPT = TC_BM / RG;  // rows a thread
        // Escapes (a code of 15: the high byte comes from the matrix's ascending list) are not looked up a weight: row d of
        // a tile has an owner among the eight lanes that write it, which walks the row's run of the list forwards - the
        // group's K blocks come in ascending order; the entries of the other group's blocks are passed over - and patches
        // the high bytes in once the warp has written the row.
        const int own = c < RPT ? (tg >> 3) + RG * c : -1;  // the tile row this thread owns, if any
        int cur = 0, end = 0, peek = 0x7fffffff;
        if (own >= 0 && P.esc_row != nullptr && row0 + own < A.R) {
            cur = __ldg(P.esc_row + row0 + own), end = __ldg(P.esc_row + row0 + own + 1);
            // (a K range that does not start at column 0: skip the entries before it)
            const int from = (int)((size_t)(row0 + own) * A.C + (size_t)kb0 * TC_BK);
            int a = cur, b = kb0 > 0 ? end : cur;
            while (a < b) {
                const int mid = (a + b) >> 1;
                if (__ldg(P.esc_idx + mid) < from) a = mid + 1;
                else b = mid;
            }
            cur = a;
            if (cur < end) peek = __ldg(P.esc_idx + cur);
        }
        const uint32_t fullp0 = smem_u32(&full_p[0]), fulla0 = smem_u32(&full_a[0]), tiles0 = smem_u32(tiles);
        static_assert(RG % 8 == 0, "a thread's rows share their swizzle");
        const uint32_t off_lo = (uint32_t)((tg >> 3) * TC_BK + c * 8), off_hi = (uint32_t)((tg >> 3) * (TC_BK / 2) + c * 4);
        const uint32_t off_out = (uint32_t)((tg >> 3) * 128 + ((c ^ ((tg >> 3) & 7)) << 4));
        int s = grp;  // (NG <= the ring's depth: the host keeps at least two stages)
        uint32_t ph = 0;
        int base = own >= 0 ? (int)((size_t)(row0 + own) * A.C + (size_t)(kb0 + grp) * TC_BK) : 0;  // the owned row's first element of the K block
        for (int kb = grp; kb < nkb; kb += NG, base += NG * TC_BK) {
            bool bad = !mbar_wait_bounded(fullp0 + s * 8, ph);
            if (bad) *(volatile int*)&s_fail = 1;
            bad = __any_sync(0xffffffffu, bad);  // (one answer a warp: it syncs below; another agent's failure shows as this wait's own)
            const uint32_t st = tiles0 + (uint32_t)s * P12_ST;  // (shared-space addresses: 32-bit arithmetic, no generic loads)
            if (!bad) {
                // (RG is a multiple of 8: a thread's rows all have its first row's swizzle; row i lies a constant on)
                const uint32_t a_lo = st + A_BYTES + P12_B + off_lo, a_hi = st + A_BYTES + P12_B + P12_LO + off_hi, a_out = st + off_out;
                p12_widen_rows<RG>(a_lo, a_hi, a_out, P.table, std::make_integer_sequence<int, RPT>{});
                __syncwarp();  // a row's eight writers are lanes of one warp, its owner among them
                if (own >= 0) {
                    // (prefetching a window of the row's next entries every stage was measured slower: most rows have none)
                    while (peek < base + TC_BK) {  // the row's entries up to the end of this K block
                        const int col = peek - base;
                        if (col >= 0)
                            asm volatile("st.shared.u8 [%0], %1;" ::"r"(st + own * 128 + (((col >> 3) ^ (own & 7)) << 4) + (col & 7) * 2 + 1),
                                         "r"((uint32_t)__ldg(P.esc_val + cur))
                                         : "memory");
                        ++cur;
                        peek = cur < end ? __ldg(P.esc_idx + cur) : 0x7fffffff;
                    }
                }
            }
            fence_proxy_async();  // the tile's bytes, written by ordinary stores, are the MMA's (an async-proxy reader) to see
            // the tile is written: the group's own barrier, which also carries the one answer every one of its threads acts
            // on (a thread leaving the loop alone would leave the others at the next barrier for good); one of them then
            // counts the tile in for the issuer (an arrival a thread on one barrier word was most of a stage's time)
            const int any_bad = grp == 0   ? p12_group_bar<1, GT>(bad)
                                : grp == 1 ? p12_group_bar<2, GT>(bad)
                                : grp == 2 ? p12_group_bar<3, GT>(bad)
                                           : p12_group_bar<4, GT>(bad);
            if (any_bad) break;
            if (tg == 0) mbar_arrive(fulla0 + s * 8);
            s += NG;
            if (s >= TC_STAGES) s -= TC_STAGES, ph ^= 1;
        }
    }
    __syncwarp();
    if (warp < 4) {
        bool ok = true;
        if (nkb > 0) ok = mbar_wait_bounded(smem_u32(&done), 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok && nkb > 0 && !*(volatile int*)&s_fail) {
            const int row = row0 + warp * 32 + lane;
            // (eight columns at a time keeps the kernel's registers at the wideners' need)
            for (int n0 = 0; n0 < A.M; n0 += 8) {
                uint32_t r[8];
                const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)n0;
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                             : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < A.R) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int n = n0 + j;
                        if (n < A.M) {
                            if (A.splits == 1) A.y[(size_t)n * A.R + row] = f2bf(0.f + __uint_as_float(r[j]));  // (the bf16 kernel's "from zero")
                            else A.part[((size_t)blockIdx.y * 32 + n) * A.R + row] = __uint_as_float(r[j]);
                        }
                    }
                }
            }
        } else if (threadIdx.x == 0 && nkb > 0) {
            b2_fail(B2_ERR_TIMEOUT);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(32u) : "memory");
    if (A.splits > 1 && A.cnt != nullptr) tc_finish_split<128 + 32 * NW>(A, row0, &s_fail);  // (the flag's word is free by now)
}

struct TcReduceArgs {
    const float* part;
    bf16* y;
    int R, M, splits;
    int glu_I, Rv;  // the gate/up form: y is m [M, glu_I]; the partial sums lie by tile position, Rv a range's row extent
};
// the K ranges' partial sums added in range order (the same sum every launch), rounded to bf16 once
__global__ void __launch_bounds__(256) gemv_tc_reduce(const TcReduceArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (A.glu_I > 0) {
        if (i >= A.M * A.glu_I) return;
        const int n = i / A.glu_I, c = i - n * A.glu_I;
        const size_t at = (size_t)(c >> 6) * TC_BM + (c & 63);  // the gate row's place in its tile; its up row 64 on
        float g = 0.f, u = 0.f;
        for (int k = 0; k < A.splits; ++k) {
            g += __ldcg(A.part + ((size_t)k * 32 + n) * A.Rv + at);
            u += __ldcg(A.part + ((size_t)k * 32 + n) * A.Rv + at + 64);
        }
        A.y[i] = f2bf(bfround(tc_silu(bfround(g))) * bfround(u));
        return;
    }
    if (i >= A.M * A.R) return;
    const int n = i / A.R, r = i - n * A.R;
    float s = 0.f;
    for (int k = 0; k < A.splits; ++k) s += __ldcg(A.part + ((size_t)k * 32 + n) * A.R + r);
    A.y[i] = f2bf(s);
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// A 2-D tensor map of a row-major matrix, made once a (matrix, box) and kept: a weight matrix is encoded the first
// time it is used, an activation buffer likewise (an engine reuses its buffers), so an eager launch does not pay the
// driver's encode every time. The map depends on nothing but its key - the address, the extents, the box and the element
// kind - so an entry never goes stale; the table is emptied when it has grown to 4096 entries.
struct MapKey {
    const void* base;
    uint64_t rows, cols;
    uint32_t box_cols, box_rows, kind;
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && box_cols == o.box_cols && box_rows == o.box_rows && kind == o.kind;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
        h ^= (k.rows + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
        h ^= (k.cols + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
        h ^= (((uint64_t)k.box_cols << 40) ^ ((uint64_t)k.box_rows << 8) ^ k.kind) + (h << 6) + (h >> 2);
        return (size_t)h;
    }
};
// kind 0: bf16 elements, boxes of box_rows x 64 columns under the 128-byte swizzle; kind 1: bytes, boxes of
// box_rows x box_cols, no swizzle. Zeros outside the matrix either way.
int make_map_kind(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t cols, uint32_t box_cols, uint32_t box_rows, uint32_t kind) {
    static EncodeFn fn = nullptr;
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> kept;
    const MapKey key{base, rows, cols, box_cols, box_rows, kind};
    std::lock_guard<std::mutex> lock(mu);
    if (fn == nullptr) {
        cudaDriverEntryPointQueryResult q;
        void* p = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || p == nullptr) {
            (void)cudaGetLastError();
            return B2_ERR_CUDA;
        }
        fn = reinterpret_cast<EncodeFn>(p);
    }
    const auto it = kept.find(key);
    if (it != kept.end()) {
        *tm = it->second;
        return B2_OK;
    }
    const uint64_t es_bytes = kind == 0 ? 2 : 1;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * es_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t es[2] = {1, 1};
    const CUresult rc = fn(tm, kind == 0 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base),
                           dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           kind == 0 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return B2_ERR_CUDA;
    if (kept.size() >= 4096) kept.clear();
    kept.emplace(key, *tm);
    return B2_OK;
}
// a [rows, cols] bf16 row-major matrix: boxes of box_rows x 64 columns, 128-byte swizzle
int make_map(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    return make_map_kind(tm, base, rows, cols, (uint32_t)TC_BK, box_rows, 0);
}

// K ranges a matrix is cut into: enough CTAs for two an SM, a whole number of K blocks each; a function of the
// matrix's shape alone, so every pass width sums in the same order
// `kps`: the K blocks a range holds. The count is recomputed from the rounded-up range length, so the last range is
// never empty (14 wanted ranges over 64 blocks are 5 blocks each, which 13 ranges already cover): every slice of the
// workspace that the ordered sum reads has been written by this launch.
int tc_splits(int R, int C, int* kps = nullptr) {
    const int tiles = (R + TC_BM - 1) / TC_BM, kb = (C + TC_BK - 1) / TC_BK;
    const int per_sm = b2_tuning().tc_ctas > 0 ? b2_tuning().tc_ctas : 2;
    const int want = max(1, (per_sm * b2_sm_count()) / tiles);
    const int aim = max(1, min(min(want, 16), kb / 4));
    const int per = (kb + aim - 1) / aim;
    if (kps != nullptr) *kps = per;
    return (kb + per - 1) / per;
}

// three parameters (two tensor maps by value and the argument block): launched through the runtime's own form
template <int BN, bool GEMM>
int launch_tc(CUtensorMap& tw, CUtensorMap& tx, TcArgs& a, dim3 grid, int stages, cudaStream_t s) {
    constexpr int ST = TcTile<BN>::ST_BYTES;
    const int max_stages = min(TC_STAGES_MAX, (224 * 1024 - 1024) / ST);
    stages = min(stages, max_stages);
    a.stages = stages;
    static bool allowed[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B2_ERR_CUDA;
    if (!allowed[dev]) {
        if (cudaFuncSetAttribute(gemv_tc<BN, GEMM>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_stages * ST + 1024) != cudaSuccess) {
            (void)cudaGetLastError();
            return B2_ERR_CUDA;
        }
        allowed[dev] = true;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = grid;
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = stages * ST + 1024;
    cfg.stream = s;
    void* params[3] = {&tw, &tx, &a};
    if (cudaLaunchKernelExC(&cfg, reinterpret_cast<const void*>(gemv_tc<BN, GEMM>), params) != cudaSuccess) {
        (void)cudaGetLastError();
        return B2_ERR_CUDA;
    }
    return B2_OK;
}

}  // namespace

extern "C" size_t btb_b200_gemv_tc_workspace_bytes(int R, int C) {
    if (R <= 0 || C <= 0) return 0;
    const int s = tc_splits(R, C);
    return s > 1 ? TC_WS_HEAD + (size_t)s * 32 * R * sizeof(float) : 0;
}

extern "C" int btb_b200_gemv_tc_bf16(const void* w, const void* x, void* y, int M, int R, int C, void* workspace,
                                     void* stream) {
    if (!w || !x || !y) return B2_ERR_NULL;
    if (M < 1 || M > 32 || R <= 0 || C <= 0 || (C & 7)) return B2_ERR_DOMAIN;
    if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(x) & 15)) return B2_ERR_DOMAIN;
    int kps = 0;
    const int splits = tc_splits(R, C, &kps);
    if (splits > 1 && (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 15))) return B2_ERR_NULL;
    CUtensorMap tw, tx;
    if (make_map(&tw, w, (uint64_t)R, (uint64_t)C, TC_BM) || make_map(&tx, x, (uint64_t)M, (uint64_t)C, TC_BN)) return B2_ERR_CUDA;
    const int stages = b2_tuning().tc_stages > 0 ? min(TC_STAGES_MAX, b2_tuning().tc_stages) : 4;
    float* part = splits > 1 ? reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + TC_WS_HEAD) : nullptr;
    const int tiles = (R + TC_BM - 1) / TC_BM;
    // the `tc_fold` tunable: the last CTA of a tile adds the ranges itself instead of the second launch. Measured equal
    // (its fences, counter round trip and loads cost what the launch does), so the second launch stays the default.
    const bool in_kernel = splits > 1 && splits <= 16 && tiles * (int)sizeof(int) <= TC_WS_HEAD && b2_tuning().tc_fold;
    TcArgs a{static_cast<bf16*>(y), part, R, C, M, kps, splits, stages, 0, in_kernel ? static_cast<int*>(workspace) : nullptr};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (const int rc = launch_tc<TC_BN, false>(tw, tx, a, dim3(tiles, splits), stages, s)) return rc;
    if (splits > 1 && !in_kernel) {
        TcReduceArgs ra{part, static_cast<bf16*>(y), R, M, splits};
        return b2_launch((const void*)gemv_tc_reduce, dim3((M * R + 255) / 256), dim3(256), 0, s, ra);
    }
    return B2_OK;
}

// a [rows, cols] byte matrix: boxes of box_rows x box_cols bytes, no swizzle
static int make_map_u8(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t cols, uint32_t box_cols, uint32_t box_rows) {
    return make_map_kind(tm, base, rows, cols, box_cols, box_rows, 1);
}

// btb_b200_gemv_tc_bf16 over pack12 weights read as stored (parts as btb_b200_gemv_p12's; `table` a HOST pointer to the 16
// high bytes): the sums of the bf16 kernel over the widened matrix, to the bit. C a multiple of 64. workspace as
// btb_b200_gemv_tc_workspace_bytes(R, C).
extern "C" int btb_b200_gemv_tc_p12(const void* lo, const void* hi4, const void* table, const void* esc_idx,
                                    const void* esc_val, const void* esc_row, const void* x, void* y, int M, int R, int C,
                                    void* workspace, void* stream) {
    if (!lo || !hi4 || !table || !x || !y) return B2_ERR_NULL;
    if (esc_row != nullptr && (!esc_idx || !esc_val)) return B2_ERR_NULL;
    if (M < 1 || M > 32 || R <= 0 || C <= 0 || (C & 63)) return B2_ERR_DOMAIN;
    if ((reinterpret_cast<uintptr_t>(lo) & 15) || (reinterpret_cast<uintptr_t>(hi4) & 15) || (reinterpret_cast<uintptr_t>(x) & 15))
        return B2_ERR_DOMAIN;
    int kps = 0;
    const int splits = tc_splits(R, C, &kps);
    if (splits > 1 && (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 15))) return B2_ERR_NULL;
    CUtensorMap tl, th, tx;
    if (make_map_u8(&tl, lo, (uint64_t)R, (uint64_t)C, TC_BK, TC_BM) || make_map_u8(&th, hi4, (uint64_t)R, (uint64_t)C / 2, TC_BK / 2, TC_BM) ||
        make_map(&tx, x, (uint64_t)M, (uint64_t)C, TC_BN))
        return B2_ERR_CUDA;
    int stages = b2_tuning().tc_stages > 0 ? b2_tuning().tc_stages : 3;
    stages = max(2, min(min(stages, TC_STAGES_MAX), (224 * 1024 - 1024) / P12_ST));
    TcP12Args a{};
    float* part = splits > 1 ? reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + TC_WS_HEAD) : nullptr;
    const int tiles = (R + TC_BM - 1) / TC_BM;
    const bool in_kernel = splits > 1 && splits <= 16 && tiles * (int)sizeof(int) <= TC_WS_HEAD && b2_tuning().tc_fold;
    a.t = TcArgs{static_cast<bf16*>(y), part, R, C, M, kps, splits, stages, 0, in_kernel ? static_cast<int*>(workspace) : nullptr};
    memcpy(a.table, table, 16);
    a.esc_idx = static_cast<const int32_t*>(esc_idx), a.esc_val = static_cast<const uint8_t*>(esc_val);
    a.esc_row = static_cast<const int32_t*>(esc_row);
    static bool allowed[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B2_ERR_CUDA;
    const int max_smem = ((224 * 1024 - 1024) / P12_ST) * P12_ST + 1024;
    if (!allowed[dev]) {
        if (cudaFuncSetAttribute(gemv_tc_p12<8, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess) {
            (void)cudaGetLastError();
            return B2_ERR_CUDA;
        }
        allowed[dev] = true;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(tiles, splits);
    // (eight widener warps in two groups: twelve in three and sixteen in two or four were measured slower)
    cfg.blockDim = dim3(128 + 32 * 8);
    cfg.dynamicSmemBytes = stages * P12_ST + 1024;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    if (b2_tuning().pdl & 1) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr, cfg.numAttrs = 1;
    }
    void* params[4] = {&tl, &th, &tx, &a};
    const void* kern = reinterpret_cast<const void*>(gemv_tc_p12<8, 2>);
    if (cudaLaunchKernelExC(&cfg, kern, params) != cudaSuccess) {
        (void)cudaGetLastError();
        return B2_ERR_CUDA;
    }
    if (splits > 1 && !in_kernel) {
        TcReduceArgs ra{part, static_cast<bf16*>(y), R, M, splits};
        return b2_launch((const void*)gemv_tc_reduce, dim3((M * R + 255) / 256), dim3(256), 0, s, ra);
    }
    return B2_OK;
}

// ---- the gate/up form ---------------------------------------------------------------------------------------------------
// m [M, I] = bf16(bf16(silu(g)) * u) with g, u the tensor-core matvec's bf16 outputs at rows i and I + i of the merged
// [2I, C] gate/up block: btb_b200_gemv_tc_bf16 followed by btb_b200_silu_mul, their bits, without the [M, 2I] buffer
// between them. It stands in for btb's btb_gemv_mma_glu_silu (native/cuda/btb_gemv_mma.cuh:216-315). workspace:
// btb_b200_gemv_tc_glu_workspace_bytes(I, C) bytes (0 where the matrix has tiles enough for the card).
static int glu_splits(int I, int C, int* kps) {
    const int tiles = (I + 63) / 64, kb = (C + TC_BK - 1) / TC_BK;
    const int per_sm = b2_tuning().tc_ctas > 0 ? b2_tuning().tc_ctas : 2;
    const int aim = max(1, min(min(max(1, (per_sm * b2_sm_count()) / tiles), 16), kb / 4));
    const int per = (kb + aim - 1) / aim;
    if (kps != nullptr) *kps = per;
    return (kb + per - 1) / per;
}
extern "C" size_t btb_b200_gemv_tc_glu_workspace_bytes(int I, int C) {
    if (I <= 0 || C <= 0) return 0;
    const int s = glu_splits(I, C, nullptr);
    return s > 1 ? TC_WS_HEAD + (size_t)s * 32 * ((I + 63) / 64) * TC_BM * sizeof(float) : 0;  // (the head is the plain matvec's: a caller may share one workspace)
}
extern "C" int btb_b200_gemv_tc_glu_bf16(const void* w, const void* x, void* m, int M, int I, int C, void* workspace,
                                         void* stream) {
    if (!w || !x || !m) return B2_ERR_NULL;
    if (M < 1 || M > 32 || I <= 0 || C <= 0 || (C & 7)) return B2_ERR_DOMAIN;
    if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(x) & 15)) return B2_ERR_DOMAIN;
    int kps = 0;
    const int splits = glu_splits(I, C, &kps);
    if (splits > 1 && (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 15))) return B2_ERR_NULL;
    CUtensorMap tw, tx;
    if (make_map(&tw, w, (uint64_t)2 * I, (uint64_t)C, 64) || make_map(&tx, x, (uint64_t)M, (uint64_t)C, TC_BN)) return B2_ERR_CUDA;
    const int stages = b2_tuning().tc_stages > 0 ? min(TC_STAGES_MAX, b2_tuning().tc_stages) : 4;
    const int tiles = (I + 63) / 64;
    float* part = splits > 1 ? reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + TC_WS_HEAD) : nullptr;
    TcArgs a{static_cast<bf16*>(m), part, 2 * I, C, M, kps, splits, stages, I, nullptr};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (const int rc = launch_tc<TC_BN, false>(tw, tx, a, dim3(tiles, splits), stages, s)) return rc;
    if (splits > 1) {
        TcReduceArgs ra{part, static_cast<bf16*>(m), 2 * I, M, splits, I, tiles * TC_BM};
        return b2_launch((const void*)gemv_tc_reduce, dim3((M * I + 255) / 256), dim3(256), 0, s, ra);
    }
    return B2_OK;
}

// ---- the prefill GEMM ------------------------------------------------------------------------------------------------
// y [T, R] = bf16(x [T, C] W^T) for a prompt chunk of T rows, T in the hundreds or thousands: the same kernel with tiles
// of 128 weight rows by up to 256 x rows, every tile its whole K, no second launch. What it stands in for is btb's
// btb_gemm_mma_bf16 (native/cuda/btb_gemm.cuh:154), whose rows are the tensor-core matvec's rows: here too an output
// element is summed exactly as btb_b200_gemv_tc_bf16 sums it - the matrix's K ranges each in an accumulator of its own,
// added in range order - so row t of a chunk carries the bits the matvec gives that row alone (tested): a prompt
// prefilled in chunks of any size leaves the cache rows that 32-row tensor-core passes would have.
extern "C" int btb_b200_gemm_tc_bf16(const void* w, const void* x, void* y, int T, int R, int C, void* stream) {
    if (!w || !x || !y) return B2_ERR_NULL;
    if (T < 1 || R <= 0 || C <= 0 || (C & 7)) return B2_ERR_DOMAIN;
    if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(x) & 15)) return B2_ERR_DOMAIN;
    // the matvec's K ranges for this matrix, an accumulator each: ranges * BN columns of the SM's 512
    int kps = 0;
    const int ranges = tc_splits(R, C, &kps);
    int BN = ranges <= 2 ? 256 : ranges <= 4 ? 128 : ranges <= 8 ? 64 : 32;
    while (BN > 32 && BN / 2 >= T) BN /= 2;  // a short chunk does not need the wide tile
    CUtensorMap tw, tx;
    if (make_map(&tw, w, (uint64_t)R, (uint64_t)C, TC_BM) || make_map(&tx, x, (uint64_t)T, (uint64_t)C, BN)) return B2_ERR_CUDA;
    const int ytiles = (T + BN - 1) / BN;
    if (ytiles > 65535) return B2_ERR_DOMAIN;
    TcArgs a{static_cast<bf16*>(y), nullptr, R, C, T, kps, ranges, 4};
    const dim3 grid((R + TC_BM - 1) / TC_BM, ytiles);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int stages = b2_tuning().tc_stages > 0 ? b2_tuning().tc_stages : 4;
    switch (BN) {
        case 32: return launch_tc<32, true>(tw, tx, a, grid, stages, s);
        case 64: return launch_tc<64, true>(tw, tx, a, grid, stages, s);
        case 128: return launch_tc<128, true>(tw, tx, a, grid, stages, s);
        default: return launch_tc<256, true>(tw, tx, a, grid, stages, s);
    }
}
