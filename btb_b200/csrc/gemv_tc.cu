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

#include "btb_b200_internal.h"

B2_DEFINE_STATUS(tc)

namespace {

constexpr int TC_BM = 128;  // weight rows a tile (the MMA's M)
constexpr int TC_BN = 32;   // x rows, padded (the MMA's N)
constexpr int TC_BK = 64;   // columns a stage: one 128-byte swizzle span of bf16
constexpr int TC_STAGES_MAX = 10;  // ring depth at most; the launch picks (four stages let two CTAs share an SM)
constexpr int A_BYTES = TC_BM * TC_BK * 2, B_BYTES = TC_BN * TC_BK * 2, ST_BYTES = A_BYTES + B_BYTES;

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
};

__global__ void __launch_bounds__(128, 2) gemv_tc(const __grid_constant__ CUtensorMap tmW,
                                                  const __grid_constant__ CUtensorMap tmX, const TcArgs A) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t full[TC_STAGES_MAX], empty[TC_STAGES_MAX], done;
    const int TC_STAGES = A.stages;
    __shared__ uint32_t tmem_slot;
    __shared__ int s_fail;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~(uintptr_t)1023);
    const int row0 = blockIdx.x * TC_BM;
    const int kb0 = blockIdx.y * A.kblocks_per_split;
    const int total_kb = (A.C + TC_BK - 1) / TC_BK;
    const int nkb = max(0, min(A.kblocks_per_split, total_kb - kb0));

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        mbar_init(smem_u32(&done), 1);
        s_fail = 0;
        mbar_fence_init();
    }
    if (warp == 0) {  // the accumulator's 32 columns of tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(32)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    pdl_launch_dependents();
    pdl_wait();  // x is the kernel's before this one

    if (warp == 0 && lane == 0) {
        // the producer: the weights' tile and x's tile of every K block of this CTA's range
        for (int kb = 0; kb < nkb; ++kb) {
            const int s = kb % TC_STAGES, ph = (kb / TC_STAGES) & 1;
            if (kb >= TC_STAGES && !mbar_wait_bounded(smem_u32(&empty[s]), ph ^ 1)) {
                *(volatile int*)&s_fail = 1;
                break;
            }
            const uint32_t bar = smem_u32(&full[s]);
            mbar_expect_tx(bar, ST_BYTES);
            tma_load_2d(smem_u32(tiles + s * ST_BYTES), &tmW, (kb0 + kb) * TC_BK, row0, bar);
            tma_load_2d(smem_u32(tiles + s * ST_BYTES + A_BYTES), &tmX, (kb0 + kb) * TC_BK, 0, bar);
        }
    } else if (warp == 1 && lane == 0) {
        // the issuer: four K = 16 instructions a stage; D f32, A and B bf16, both K-major, N = 32, M = 128
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
        for (int kb = 0; kb < nkb; ++kb) {
            const int s = kb % TC_STAGES, ph = (kb / TC_STAGES) & 1;
            if (!mbar_wait_bounded(smem_u32(&full[s]), ph)) {
                *(volatile int*)&s_fail = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a0 = smem_u32(tiles + s * ST_BYTES), b0 = a0 + A_BYTES;
#pragma unroll
            for (int k = 0; k < TC_BK / 16; ++k)
                umma_bf16(tmem, umma_desc_sw128(a0 + k * 32), umma_desc_sw128(b0 + k * 32), idesc, (kb | k) != 0);
            umma_commit(smem_u32(&empty[s]));  // the stage is free once these have read it
        }
        umma_commit(smem_u32(&done));
    }
    __syncwarp();
    // the epilogue: warp w reads lanes 32 w .. 32 w + 31 (a weight row a thread); the 32 columns are the x rows
    bool ok = true;
    if (nkb > 0) ok = mbar_wait_bounded(smem_u32(&done), 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok && nkb > 0 && !*(volatile int*)&s_fail) {
        uint32_t r[32];
        const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16);
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
        const int row = row0 + warp * 32 + lane;
        if (row < A.R) {
            if (A.splits == 1) {
#pragma unroll
                for (int n = 0; n < 32; ++n)
                    if (n < A.M) A.y[(size_t)n * A.R + row] = f2bf(__uint_as_float(r[n]));
            } else {
#pragma unroll
                for (int n = 0; n < 32; ++n)
                    if (n < A.M) A.part[((size_t)blockIdx.y * 32 + n) * A.R + row] = __uint_as_float(r[n]);
            }
        }
    } else if (threadIdx.x == 0 && nkb > 0) {
        b2_fail(B2_ERR_TIMEOUT);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(32) : "memory");
}

struct TcReduceArgs {
    const float* part;
    bf16* y;
    int R, M, splits;
};
// the K ranges' partial sums added in range order (the same sum every launch), rounded to bf16 once
__global__ void __launch_bounds__(256) gemv_tc_reduce(const TcReduceArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= A.M * A.R) return;
    const int n = i / A.R, r = i - n * A.R;
    float s = 0.f;
    for (int k = 0; k < A.splits; ++k) s += __ldcg(A.part + ((size_t)k * 32 + n) * A.R + r);
    A.y[i] = f2bf(s);
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// a [rows, cols] bf16 row-major matrix as a 2-D tensor map with boxes of box_rows x 64 columns, 128-byte swizzle,
// zeros outside the matrix
int make_map(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    static EncodeFn fn = nullptr;
    if (fn == nullptr) {
        cudaDriverEntryPointQueryResult q;
        void* p = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || p == nullptr) {
            (void)cudaGetLastError();
            return B2_ERR_CUDA;
        }
        fn = reinterpret_cast<EncodeFn>(p);
    }
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)TC_BK, box_rows};
    cuuint32_t es[2] = {1, 1};
    const CUresult rc = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS ? B2_OK : B2_ERR_CUDA;
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

}  // namespace

extern "C" size_t btb_b200_gemv_tc_workspace_bytes(int R, int C) {
    if (R <= 0 || C <= 0) return 0;
    const int s = tc_splits(R, C);
    return s > 1 ? (size_t)s * 32 * R * sizeof(float) : 0;
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
    TcArgs a{static_cast<bf16*>(y), static_cast<float*>(workspace), R, C, M, kps, splits, stages};
    const int smem = stages * ST_BYTES + 1024;
    static bool allowed[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B2_ERR_CUDA;
    if (!allowed[dev]) {
        if (cudaFuncSetAttribute(gemv_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_STAGES_MAX * ST_BYTES + 1024) != cudaSuccess) {
            (void)cudaGetLastError();
            return B2_ERR_CUDA;
        }
        allowed[dev] = true;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // three parameters (two tensor maps by value and the argument block): launched through the runtime's own form
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3((R + TC_BM - 1) / TC_BM, splits);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    void* params[3] = {&tw, &tx, &a};
    if (cudaLaunchKernelExC(&cfg, reinterpret_cast<const void*>(gemv_tc), params) != cudaSuccess) {
        (void)cudaGetLastError();
        return B2_ERR_CUDA;
    }
    if (splits > 1) {
        TcReduceArgs ra{static_cast<const float*>(workspace), static_cast<bf16*>(y), R, M, splits};
        return b2_launch((const void*)gemv_tc_reduce, dim3((M * R + 255) / 256), dim3(256), 0, s, ra);
    }
    return B2_OK;
}
