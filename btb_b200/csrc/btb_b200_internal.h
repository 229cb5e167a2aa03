// Host-side plumbing shared by the kernels' translation units: tunables, the device's SM count, and the one launch
// path (cudaLaunchKernelEx with the programmatic-dependent-launch attribute when it is switched on).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "common.cuh"

struct B2Tuning {
    int ring_bytes;   // shared memory a GEMV CTA spends on its warps' rings
    int seg_bytes;    // a ring stage holds at most this many weight bytes of a row
    int x_smem_max;   // x is staged in shared memory when M * C * 2 is at most this
    int ctas_per_sm;  // GEMV CTAs an SM (the grid is persistent)
    int evict_first;  // weight copies carry an L2 evict-first hint
    int pdl;          // programmatic stream serialization: bit 0 the GEMV launches, bit 1 the step's small kernels,
                      // bit 2 the MoE block's kernels (router, picked experts, activation, sum)
    int warps;        // warps a GEMV CTA for passes of one or two rows: 8 or 16
    int solo;         // under PDL a GEMV CTA claims an SM's shared memory for itself
    int moe_stream;   // the picked experts' matvecs through the streaming kernel (0: the plain 16-lane kernel)
    int ms_tpr;       // threads that share an expert row: 4, 8 or 16
    int ms_ctas;      // CTAs of the expert kernel an SM holds (0: one for four threads a row, else two)
    int ms_seg, ms_warps;  // the expert kernel's columns a stage and warps a CTA (0: its own choice)
    int tc_stages, tc_ctas;  // the tensor-core matvec's ring depth and CTAs an SM its K split aims at (0: 4 and 2)
    int balance;      // pick the GEMV grid and warps a CTA so that the rows divide evenly over the warps
    int x_direct;     // a one-row plain GEMV reads x where it lies (L1/L2) instead of staging it in shared memory first
    int l2_warm_kb;   // the step's attention launch pulls at most this much of the next kernels' weights into L2 (0: off)
    int l2_warm_ctas; // blocks that do it (0: every SM the attention's own blocks leave idle)
    int warps_packed; // warps a GEMV CTA prefers over rows widened in registers (pack12, FP8); 0: the bf16 preference
    int tc_fold;      // the tensor-core matvec adds its K ranges' partial sums in the launch itself (0: a second launch)
};
B2Tuning& b2_tuning();
int b2_sm_count();

// one launch: `args` is the kernel's single by-value parameter struct
// `kind`: 1 a GEMV, 2 one of the step's small kernels, 4 one of the MoE block's - the `pdl` tunable is a mask over the
// kinds (0 never launches early)
template <typename Args>
static inline int b2_launch(const void* kern, dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            const Args& args, int kind = 2) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    if (b2_tuning().pdl & kind) {
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
    }
    void* params[1] = {const_cast<Args*>(&args)};
    const cudaError_t e = cudaLaunchKernelExC(&cfg, kern, params);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return B2_ERR_CUDA;
    }
    return B2_OK;
}

// opt a kernel in to large dynamic shared memory once a device
static inline int b2_allow_smem(const void* kern, bool* done_for_device) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B2_ERR_CUDA;
    if (!done_for_device[dev]) {
        // the opt-in ceiling (227 KB a block) covers static and dynamic shared memory together
        cudaFuncAttributes fa;
        if (cudaFuncGetAttributes(&fa, kern) != cudaSuccess) {
            (void)cudaGetLastError();
            return B2_ERR_CUDA;
        }
        const int room = 227 * 1024 - (int)fa.sharedSizeBytes;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, room) != cudaSuccess) {
            (void)cudaGetLastError();
            return B2_ERR_CUDA;
        }
        done_for_device[dev] = true;
    }
    return B2_OK;
}
