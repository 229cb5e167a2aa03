// The picked experts' matvecs as one streaming launch: stored-format expert rows (bf16, MXFP4 blocks, FP8 with block
// scales) pulled through shared memory by TMA bulk copies and multiplied in the CPU tier's order.
//
// The order is btb's host kernels' (native/src/gemv.rs:46-58, 85-123; the on-card twins btb_gemv_lane16{,_mx4}_f32,
// native/cuda/btb_kernels.cu:1635-1766): column c of a row belongs to chain c mod 16, a chain takes its columns in
// increasing order with one fmaf each, and the sixteen sums fold pairwise (1, 2, 4, 8 apart). A chain is sequential,
// so a row offers sixteen-way parallelism and no more. Here four threads share a row, each running four adjacent
// chains: a warp takes eight rows at a time, a thread reads its four consecutive weights of every sixteen columns
// from shared memory as one word, and the fold is two adds in the thread and two shuffles. The rows arrive by one
// bulk copy a row segment into a per-warp ring (rows padded by 16 bytes, so the eight rows' words fall in distinct
// banks); x is staged once a CTA as f32. Every weight byte is read from DRAM once, in large transfers - the
// per-column byte loads of the plain 16-lane kernel ran at a twentieth of the memory's rate.
#include <cuda_fp16.h>
#include <type_traits>
#include <cuda_fp8.h>

#include "btb_b200_internal.h"
#include "moe_widen.cuh"
#include "tp.cuh"

B2_DEFINE_STATUS(moes)

namespace {

enum { S_BF16 = 0, S_MX4 = 1, S_FP8 = 2 };
// f(0), f(1), ... f(N - 1) with the index a compile-time constant (offsets and shifts become immediates)
template <int N>
struct Unrolled {
    template <class F>
    static __device__ __forceinline__ void run(F&& f) {
        Unrolled<N - 1>::run(f);
        f(std::integral_constant<int, N - 1>{});
    }
};
template <>
struct Unrolled<0> {
    template <class F>
    static __device__ __forceinline__ void run(F&&) {}
};

constexpr int PAD = 16;     // bytes between the rows of a stage
constexpr int MAXW = 16;    // warps a CTA at most

struct MSArgs {
    const uint8_t* w;       // expert 0's weights
    const uint8_t* scales;  // MX4: e8m0 bytes [R, C/32]; FP8: f32 grid [sr, sc]
    long long w_stride, s_stride;  // bytes from an expert to the next
    const int* idx;         // [n_tasks] the task's expert, or null (expert 0 for all)
    const float* x;         // [rows_x, C] f32
    int x_div;              // task i reads x row i / x_div
    float* y;               // [n_tasks, R] f32
    int R, C, sr, sc, E;
    int ep_rank, ep_size;
    int seg;                // columns a stage holds of each row (a multiple of 32)
    int stages;
    // x made on the way in from the gate/up outputs (btb/engine/host.py:439-450): x row of task i is the gated
    // activation of gu row i [2C]. act_kind -1: x as given; 0: silu(gate) * up over halves; 1: gpt-oss's clamped GLU
    // over interleaved lanes - every bf16 rounding of the host's torch ops kept
    int act_kind;
    float alpha, limit;
    // the gated activation made on the way OUT of the gate/up matvecs (the same operations): glu_kind 0 pairs gate row j
    // with up row R/2 + j (a warp takes four of each), 1 pairs rows 2j and 2j + 1; the task's activated row [R/2] goes to
    // glu_out and y is not written. -1: plain outputs
    int glu_kind;
    float* glu_out;
    // experts cut over ranks (tp.cuh): with send.n > 0 a finished output of an expert this rank holds goes to every
    // rank's copy of the [n_tasks, R] vector as a marked word carrying bf16(sum) - the rounding the ordered sum applies
    // to a product first thing - and another rank's experts' rows are left to their owner
    B2Send send;
};

__device__ __forceinline__ float moe_act_value(const float* gu, int c, int I, int kind, float alpha, float limit) {
    const int gi = kind == 0 ? c : 2 * c, ui = kind == 0 ? I + c : 2 * c + 1;
    float g = bfround(__ldcg(gu + gi)), u = bfround(__ldcg(gu + ui));
    if (kind == 0) return bfround(bfround(g / (1.f + expf(-g))) * u);
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    const float t1 = bfround(g * alpha);
    const float t2 = bfround(1.f / (1.f + expf(-t1)));
    const float glu = bfround(g * t2);
    return bfround(bfround(u + 1.f) * glu);
}

// the gated activation of one (gate, up) pair of f32 outputs: moe_act_value's operations
__device__ __forceinline__ float moe_act_pair(float g, float u, int kind, float alpha, float limit) {
    g = bfround(g), u = bfround(u);
    if (kind == 0) return bfround(bfround(g / (1.f + expf(-g))) * u);
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    const float t1 = bfround(g * alpha);
    const float t2 = bfround(1.f / (1.f + expf(-t1)));
    const float glu = bfround(g * t2);
    return bfround(bfround(u + 1.f) * glu);
}

// Four e4m3 weights (the bytes of wb, lowest first) under one block scale against four bf16 x (two packed pairs), each
// product into its own chain: e4m3 -> f16 (exact) -> f32 through the fma pipe -> times the scale -> the nearest bf16 (the
// weight btb holds) -> bf16 x bf16 + f32 with one rounding. One block of PTX, so that every 16-bit half is named where
// it lies.
__device__ __forceinline__ void fp8_step4(uint32_t wb, uint32_t x01, uint32_t x23, float sc, float& a0, float& a1,
                                          float& a2, float& a3) {
    asm("{\n"
        ".reg .b16 w0, w1, a, b, c, d, one, pa, pb, pc, pd, xa, xb, xc, xd;\n"
        ".reg .b32 h01, h23, p01, p23;\n"
        ".reg .f32 f0, f1, f2, f3;\n"
        "mov.b32 {w0, w1}, %4;\n"
        "cvt.rn.f16x2.e4m3x2 h01, w0;\n"
        "cvt.rn.f16x2.e4m3x2 h23, w1;\n"
        "mov.b32 {a, b}, h01;\n"
        "mov.b32 {c, d}, h23;\n"
        "mov.b16 one, 0x3C00;\n"
        "fma.rn.f32.f16 f0, a, one, %8;\n"
        "fma.rn.f32.f16 f1, b, one, %8;\n"
        "fma.rn.f32.f16 f2, c, one, %8;\n"
        "fma.rn.f32.f16 f3, d, one, %8;\n"
        "mul.rn.f32 f0, f0, %7;\n"
        "mul.rn.f32 f1, f1, %7;\n"
        "mul.rn.f32 f2, f2, %7;\n"
        "mul.rn.f32 f3, f3, %7;\n"
        "cvt.rn.bf16x2.f32 p01, f1, f0;\n"
        "cvt.rn.bf16x2.f32 p23, f3, f2;\n"
        "mov.b32 {pa, pb}, p01;\n"
        "mov.b32 {pc, pd}, p23;\n"
        "mov.b32 {xa, xb}, %5;\n"
        "mov.b32 {xc, xd}, %6;\n"
        "fma.rn.f32.bf16 %0, pa, xa, %0;\n"
        "fma.rn.f32.bf16 %1, pb, xb, %1;\n"
        "fma.rn.f32.bf16 %2, pc, xc, %2;\n"
        "fma.rn.f32.bf16 %3, pd, xd, %3;\n"
        "}\n"
        : "+f"(a0), "+f"(a1), "+f"(a2), "+f"(a3)
        : "r"(wb), "r"(x01), "r"(x23), "f"(sc), "f"(-0.0f));
}

// two bytes of e2m1 codes (four codes, the lowest nibble first) as two f16 pairs through the conversion unit
__device__ __forceinline__ void e2m1x4_f16x2(uint32_t two_bytes, uint32_t& h01, uint32_t& h23) {
    asm("{\n.reg .b8 b0, b1;\n.reg .b16 t;\ncvt.u16.u32 t, %2;\nmov.b16 {b0, b1}, t;\ncvt.rn.f16x2.e2m1x2 %0, b0;\n"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n}"
        : "=r"(h01), "=r"(h23)
        : "r"(two_bytes));
}
// four bytes of e2m1 codes (eight codes, the lowest nibble first) as four f16 pairs
__device__ __forceinline__ void e2m1x8_f16x2(uint32_t four_bytes, uint32_t& h01, uint32_t& h23, uint32_t& h45, uint32_t& h67) {
    asm("{\n.reg .b8 b0, b1, b2, b3;\nmov.b32 {b0, b1, b2, b3}, %4;\ncvt.rn.f16x2.e2m1x2 %0, b0;\n"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\ncvt.rn.f16x2.e2m1x2 %2, b2;\ncvt.rn.f16x2.e2m1x2 %3, b3;\n}"
        : "=r"(h01), "=r"(h23), "=r"(h45), "=r"(h67)
        : "r"(four_bytes));
}
// an f16 pair times the f16 value p, as two f32 (exact: the mixed-precision fma's product is not rounded before the sum,
// and the addend is -0, which keeps a zero's sign)
__device__ __forceinline__ void f16x2_times(uint32_t h, unsigned short p, float& f0, float& f1) {
    asm("{\n.reg .b16 lo, hi;\nmov.b32 {lo, hi}, %2;\nfma.rn.f32.f16 %0, lo, %3, %4;\nfma.rn.f32.f16 %1, hi, %3, %4;\n}"
        : "=f"(f0), "=f"(f1)
        : "r"(h), "h"(p), "f"(-0.0f));
}
// One MXFP4 block's share of a thread: its CPT columns of the block's first sixteen and of its last sixteen. The weight is
// code x 2^(s - 127). FAST: the scale is an f16 value (2^-24 .. 2^15, subnormals included), so the widen f16 -> f32 and
// the scale are ONE mixed-precision fma, exact; else the widen multiplies by 1 and an f32 multiply (exact too, or
// overflowing as the reference's does) follows.
template <int CPT, bool FAST>
__device__ __forceinline__ void mx4_block(const uint8_t* bp, int q, const float* xa, unsigned short ph, float pf, float* acc) {
    const unsigned short mul = FAST ? ph : (unsigned short)0x3C00;
    if (CPT == 4) {
        const uint32_t lo = *reinterpret_cast<const unsigned short*>(bp + q * 2);
        const uint32_t hi = *reinterpret_cast<const unsigned short*>(bp + 8 + q * 2);
        const float4 va = *reinterpret_cast<const float4*>(xa), vb = *reinterpret_cast<const float4*>(xa + 16);
        uint32_t a01, a23, b01, b23;
        e2m1x8_f16x2(__byte_perm(lo, hi, 0x5410), a01, a23, b01, b23);
        float w[8];
        f16x2_times(a01, mul, w[0], w[1]);
        f16x2_times(a23, mul, w[2], w[3]);
        f16x2_times(b01, mul, w[4], w[5]);
        f16x2_times(b23, mul, w[6], w[7]);
        if (!FAST) {
#pragma unroll
            for (int u = 0; u < 8; ++u) w[u] = __fmul_rn(w[u], pf);
        }
        acc[0] = fmaf(w[0], va.x, acc[0]);
        acc[1 % CPT] = fmaf(w[1], va.y, acc[1 % CPT]);
        acc[2 % CPT] = fmaf(w[2], va.z, acc[2 % CPT]);
        acc[3 % CPT] = fmaf(w[3], va.w, acc[3 % CPT]);
        acc[0] = fmaf(w[4], vb.x, acc[0]);
        acc[1 % CPT] = fmaf(w[5], vb.y, acc[1 % CPT]);
        acc[2 % CPT] = fmaf(w[6], vb.z, acc[2 % CPT]);
        acc[3 % CPT] = fmaf(w[7], vb.w, acc[3 % CPT]);
    } else {
        const uint32_t codes = (uint32_t)bp[q] | ((uint32_t)bp[8 + q] << 8);
        const float2 va = *reinterpret_cast<const float2*>(xa), vb = *reinterpret_cast<const float2*>(xa + 16);
        uint32_t a01, b01;
        e2m1x4_f16x2(codes, a01, b01);  // the first half's two columns, then the second half's
        float w[4];
        f16x2_times(a01, mul, w[0], w[1]);
        f16x2_times(b01, mul, w[2], w[3]);
        if (!FAST) {
#pragma unroll
            for (int u = 0; u < 4; ++u) w[u] = __fmul_rn(w[u], pf);
        }
        acc[0] = fmaf(w[0], va.x, acc[0]);
        acc[1 % CPT] = fmaf(w[1], va.y, acc[1 % CPT]);
        acc[0] = fmaf(w[2], vb.x, acc[0]);
        acc[1 % CPT] = fmaf(w[3], vb.y, acc[1 % CPT]);
    }
}

// x in shared memory: f32 [C], then bf16 [C] (C is a multiple of 32, so both start on 128 bytes)
__host__ __device__ constexpr int x_smem_bytes(int C) { return (C * 6 + 127) & ~127; }

template <int FMT>
__host__ __device__ constexpr int col_bytes2() { return FMT == S_BF16 ? 4 : FMT == S_FP8 ? 2 : 1; }  // twice a column's bytes

// TPR threads share a row, each running CPT = 16 / TPR adjacent chains; a warp takes RB = 32 / TPR rows at a time
template <int FMT, int TPR>
__global__ void __launch_bounds__(MAXW * 32, TPR == 4 ? 1 : 2) moe_gemv_stream(const MSArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int CPT = 16 / TPR, RB = 32 / TPR;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int ri = lane / TPR, q = lane % TPR;  // the thread's row of the warp's RB, its chains q CPT .. q CPT + CPT - 1
    const int task = blockIdx.y;
    const int R = A.R, C = A.C, seg = A.seg, S = A.stages;
    // the row a group's slot holds: eight consecutive rows, or (glu_kind 0, four threads a row) four gate rows and the four
    // up rows they pair with
    const bool halves = TPR == 4 && A.glu_kind == 0;
    auto row_of = [&](int grp, int slot) { return halves ? (slot < 4 ? grp * 4 + slot : (R >> 1) + grp * 4 + slot - 4) : grp * RB + slot; };
    constexpr int CB2 = col_bytes2<FMT>();
    const int row_bytes = C * CB2 / 2;
    const int stride = seg * CB2 / 2 + PAD;  // a stage row
    const int sbytes = RB * stride;
    const int nseg = (C + seg - 1) / seg;
    float* xs = reinterpret_cast<float*>(smem);
    unsigned short* xh = reinterpret_cast<unsigned short*>(smem + (size_t)C * 4);  // x again as bf16, when it is bf16-valued
    const int xbytes = x_smem_bytes(C);
    uint8_t* ring = smem + xbytes + (size_t)warp * S * sbytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + xbytes + (size_t)nw * S * sbytes) + warp * S;

    if (lane == 0) {
        for (int s = 0; s < S; ++s) mbar_init(smem_u32(bars + s), 1);
        mbar_fence_init();
    }
    __syncwarp();
    pdl_launch_dependents();
    pdl_wait();  // the picks and x are the kernels' before this one

    int e = 0;
    if (A.idx != nullptr) {
        e = __ldcg(A.idx + task);
        if (e < 0 || e >= A.E) {  // never read outside the experts: record and skip
            if (threadIdx.x == 0 && blockIdx.x == 0) b2_fail(B2_ERR_DOMAIN);
            e = -1;
        }
    }
    bool mine = e >= 0;
    if (mine && A.ep_size > 1) {
        mine = e % A.ep_size == A.ep_rank;
        e = e / A.ep_size;
    }
    // this CTA's groups of eight rows: an even split of the task's groups over the CTAs that share it
    const int groups = (R + RB - 1) / RB;
    const int base = groups / gridDim.x, rem = groups % gridDim.x;
    const int g0 = blockIdx.x * base + min((int)blockIdx.x, rem);
    const int gc = base + ((int)blockIdx.x < rem ? 1 : 0);
    const int my_groups = gc > warp ? (gc - warp + nw - 1) / nw : 0;
    if (!mine) {  // another rank's expert (or a refused pick): zeros, so that the ranks' sum is the whole
        if (A.send.n != 0) return;  // (under the exchange the owner writes the row into every rank's copy)
        for (int g = g0 + warp; g < g0 + gc; g += nw) {
            const int r = row_of(g, ri);
            if (r < R && q == 0) {
                if (A.glu_kind < 0) A.y[(size_t)task * R + r] = 0.f;
                else if (A.glu_kind == 0 ? r < (R >> 1) : !(r & 1)) A.glu_out[(size_t)task * (R >> 1) + (A.glu_kind == 0 ? r : r >> 1)] = 0.f;
            }
        }
        return;
    }
    const uint8_t* wbase = A.w + (size_t)e * A.w_stride;
    const uint64_t pol = l2_evict_first_policy();
    const int n_items = my_groups * nseg;
    int p_grp = g0 + warp, p_seg = 0, p_st = 0, issued = 0;
    auto issue_next = [&]() {
        const int c0 = p_seg * seg;
        const int n = min(seg, C - c0);
        const int rows = halves ? RB : min(RB, R - p_grp * RB);  // (halves: R/2 a multiple of four, every group whole)
        const uint32_t nb = (uint32_t)(n * CB2 / 2);
        const uint32_t bar = smem_u32(bars + p_st);
        if (lane == 0) mbar_expect_tx(bar, nb * rows);
        __syncwarp();
        // (a copy a lane: one lane issuing the group's copies in a straight line was measured at more instructions)
        if (lane < rows) {
            const uint8_t* src = wbase + (size_t)row_of(p_grp, lane) * row_bytes + (size_t)c0 * CB2 / 2;
            bulk_g2s_hint(smem_u32(ring + (size_t)p_st * sbytes + (size_t)lane * stride), src, nb, bar, pol);
        }
        ++issued;
        if (++p_st == S) p_st = 0;
        if (++p_seg == nseg) {
            p_seg = 0;
            p_grp += nw;
        }
    };
    {
        const int first = min(S, n_items);
        for (int i = 0; i < first; ++i) issue_next();
    }
    // x as f32 in shared memory, once a CTA - and, when every element is a bf16 value (the rows btb's experts are given
    // are: the normed row widened, the gated activation rounded by its last torch op), as bf16 too: then the chains run
    // on the mixed-precision fma (bf16 x bf16 + f32, one rounding: fmaf's bits) over half the shared-memory traffic
    int inexact = 0;
    if (A.act_kind < 0) {
        const float4* xg = reinterpret_cast<const float4*>(A.x + (size_t)(task / A.x_div) * C);
        for (int i = threadIdx.x; i < C / 4; i += blockDim.x) {
            const float4 v = __ldcg(xg + i);
            reinterpret_cast<float4*>(xs)[i] = v;
            const uint32_t a = __float_as_uint(v.x), b = __float_as_uint(v.y), c = __float_as_uint(v.z), d = __float_as_uint(v.w);
            inexact |= (int)((a | b | c | d) & 0xffffu);
            reinterpret_cast<uint2*>(xh)[i] = make_uint2((a >> 16) | (b & 0xffff0000u), (c >> 16) | (d & 0xffff0000u));
        }
    } else {
        const float* gu = A.x + (size_t)task * 2 * C;
        for (int i = threadIdx.x; i < C; i += blockDim.x) {
            const float v = moe_act_value(gu, i, C, A.act_kind, A.alpha, A.limit);
            xs[i] = v;
            xh[i] = (unsigned short)(__float_as_uint(v) >> 16);
        }
    }
    // (MXFP4 rows run on f32 x either way: their widen and scale are one exact fma, nothing more to save)
    const bool xbf = CPT > 1 && FMT != S_MX4 && __syncthreads_or(inexact) == 0;
    if (CPT == 1 || FMT == S_MX4) __syncthreads();

    float acc[CPT];
#pragma unroll
    for (int u = 0; u < CPT; ++u) acc[u] = 0.f;
    // FP8: rows a scale block holds, columns a scale block holds (the divisions made once, not a stage)
    const int bm = FMT == S_FP8 ? R / A.sr : 1, bn = FMT == S_FP8 ? C / A.sc : 1;
    const bool bn128 = bn == 128 && (seg & 127) == 0 && seg <= 512;  // a stage starts on a block, holds four at most
    const float* srow_cur = nullptr;  // the scale row of the group's rows (a warp's rows share it: bm is a multiple of 8 or the rows differ)
    int c_grp = g0 + warp, c_seg = 0, c_st = 0;
    uint32_t c_par = 0;
    bool ok = true;
    int i = 0;
    for (; i < n_items; ++i) {
        const int r = row_of(c_grp, ri);
        const bool live = r < R;
        const int c0 = c_seg * seg;
        const int n = min(seg, C - c0);
        // the stage's scales are on their way while the weights land
        float fsc[4] = {1.f, 1.f, 1.f, 1.f};
        unsigned mxs = 0u;
        if (FMT == S_FP8) {
            if (c_seg == 0)
                srow_cur = reinterpret_cast<const float*>(A.scales + (size_t)e * A.s_stride) + (size_t)((live ? r : 0) / bm) * A.sc;
            if (bn128) {
                const int cb0 = c0 >> 7;
#pragma unroll
                for (int u = 0; u < 4; ++u) fsc[u] = cb0 + u < A.sc ? __ldg(srow_cur + cb0 + u) : 1.f;
            }
        } else if (FMT == S_MX4) {
            // a row's scale bytes of this stage (one a block of 32 columns): four a thread, shared by shuffle below
            const uint8_t* sr = A.scales + (size_t)e * A.s_stride + (size_t)(live ? r : 0) * (C >> 5) + (c0 >> 5);
            const int nb = n >> 5;
            constexpr int SPT = TPR >= 16 ? 1 : 16 / TPR >= 4 ? 4 : 16 / TPR;  // scale bytes a thread fetches: 4, 2 or 1
#pragma unroll
            for (int u = 0; u < SPT; ++u) {
                const int b = q * SPT + u;
                mxs |= (b < nb ? (unsigned)__ldg(sr + b) : 127u) << (8 * u);
            }
        }
        if (!mbar_wait_bounded(smem_u32(bars + c_st), c_par)) {
            ok = false;
            break;
        }
        const uint8_t* srowp = ring + (size_t)c_st * sbytes + (size_t)ri * stride;
        const float* xp = xs + c0;
        if (xbf) {
            const unsigned short* xb = xh + c0 + q * CPT;
            if (FMT == S_FP8) {
                const uint8_t* wq = srowp + q * CPT;
                auto step16 = [&](int off, float sc) {  // the 16 columns at `off` of the stage
                    if (CPT == 4) {
                        const uint32_t wb = *reinterpret_cast<const uint32_t*>(wq + off);
                        const uint2 xv = *reinterpret_cast<const uint2*>(xb + off);
                        fp8_step4(wb, xv.x, xv.y, sc, acc[0], acc[1 % CPT], acc[2 % CPT], acc[3 % CPT]);
                    } else {
                        const uint32_t w01 = e4m3x2_held_pair(*reinterpret_cast<const unsigned short*>(wq + off), sc);
                        const uint32_t xv = *reinterpret_cast<const uint32_t*>(xb + off);
                        acc[0] = fma1_bf16<0, 0>(w01, xv, acc[0]);
                        acc[1 % CPT] = fma1_bf16<1, 1>(w01, xv, acc[1 % CPT]);
                    }
                };
                if (bn128) {
                    // one scale for each run of 128 columns (eight steps); every offset a constant
                    Unrolled<4>::run([&](auto KB) {
                        constexpr int kb = decltype(KB)::value;
                        if (kb * 128 < n) {
                            const float sc = fsc[kb];
                            Unrolled<8>::run([&](auto U) { step16(kb * 128 + decltype(U)::value * 16, sc); });
                        }
                    });
                } else {
                    const int steps = n >> 4;
#pragma unroll 4
                    for (int s = 0; s < steps; ++s) step16(s * 16, __ldg(srow_cur + (c0 + s * 16) / bn));
                }
            } else {
                const int steps = n >> 4;
#pragma unroll 4
                for (int s = 0; s < steps; ++s) {
                    const uint8_t* wp = srowp + s * 32 + q * CPT * 2;
                    if (CPT == 4) {
                        const uint2 wb = *reinterpret_cast<const uint2*>(wp);
                        const uint2 xv = *reinterpret_cast<const uint2*>(xb + s * 16);
                        acc[0] = fma1_bf16<0, 0>(wb.x, xv.x, acc[0]);
                        acc[1 % CPT] = fma1_bf16<1, 1>(wb.x, xv.x, acc[1 % CPT]);
                        acc[2 % CPT] = fma1_bf16<0, 0>(wb.y, xv.y, acc[2 % CPT]);
                        acc[3 % CPT] = fma1_bf16<1, 1>(wb.y, xv.y, acc[3 % CPT]);
                    } else {
                        const uint32_t wb = *reinterpret_cast<const uint32_t*>(wp);
                        const uint32_t xv = *reinterpret_cast<const uint32_t*>(xb + s * 16);
                        acc[0] = fma1_bf16<0, 0>(wb, xv, acc[0]);
                        acc[1 % CPT] = fma1_bf16<1, 1>(wb, xv, acc[1 % CPT]);
                    }
                }
            }
        } else if (FMT == S_FP8) {
            const uint8_t* wq = srowp + q * CPT;
            const float* xq = xp + q * CPT;
            auto step16 = [&](int off, float sc) {
                if (CPT == 4) {
                    const uint32_t wb = *reinterpret_cast<const uint32_t*>(wq + off);
                    const float4 xv = *reinterpret_cast<const float4*>(xq + off);
                    const uint32_t w01 = e4m3x2_held_pair(wb, sc), w23 = e4m3x2_held_pair(wb >> 16, sc);
                    acc[0] = fmaf(bf_lo(w01), xv.x, acc[0]);
                    acc[1 % CPT] = fmaf(bf_hi(w01), xv.y, acc[1 % CPT]);
                    acc[2 % CPT] = fmaf(bf_lo(w23), xv.z, acc[2 % CPT]);
                    acc[3 % CPT] = fmaf(bf_hi(w23), xv.w, acc[3 % CPT]);
                } else if (CPT == 2) {
                    const uint32_t w01 = e4m3x2_held_pair(*reinterpret_cast<const unsigned short*>(wq + off), sc);
                    const float2 xv = *reinterpret_cast<const float2*>(xq + off);
                    acc[0] = fmaf(bf_lo(w01), xv.x, acc[0]);
                    acc[1 % CPT] = fmaf(bf_hi(w01), xv.y, acc[1 % CPT]);
                } else {
                    acc[0] = fmaf(bf_lo(e4m3x2_held_pair(wq[off], sc)), xq[off], acc[0]);
                }
            };
            if (bn128) {
                Unrolled<4>::run([&](auto KB) {
                    constexpr int kb = decltype(KB)::value;
                    if (kb * 128 < n) {
                        const float sc = fsc[kb];
                        Unrolled<8>::run([&](auto U) { step16(kb * 128 + decltype(U)::value * 16, sc); });
                    }
                });
            } else {
                const int steps = n >> 4;
#pragma unroll 4
                for (int s = 0; s < steps; ++s) step16(s * 16, __ldg(srow_cur + (c0 + s * 16) / bn));
            }
        } else if (FMT == S_MX4) {
            const int nb = n >> 5;
            constexpr int SPT = TPR >= 16 ? 1 : 16 / TPR >= 4 ? 4 : 16 / TPR;
            // the block's 16 bytes: byte i holds columns 2i (low nibble) and 2i + 1 of its first 16 columns, byte 8 + i
            // the same of its last 16. 2^(s - 127) is a normal f16 for s in 113..142 (every sane checkpoint's scales):
            // where all of the warp's scales of this stage are, the widen f16 -> f32 and the scale are one exact fma,
            // the multiplier's f16 bits (s - 112) << 10 made by a shift of the byte
            const bool stage_f16 = CPT > 1 && __all_sync(0xffffffffu, __vminu4(mxs, 0x71717171u) == 0x71717171u &&
                                                                          __vmaxu4(mxs, 0x8E8E8E8Eu) == 0x8E8E8E8Eu);
            if (stage_f16) {
                const unsigned rel = mxs - 0x70707070u;  // every byte s - 112, 1..30: no borrow
                const int row_lane = (lane / TPR) * TPR;
                // the row's scale bytes of the whole stage, from the threads that fetched them (outside any condition:
                // a shuffle under one costs a divergence check each)
                unsigned pks[16 / SPT];
#pragma unroll
                for (int j = 0; j < 16 / SPT; ++j) pks[j] = __shfl_sync(0xffffffffu, rel, row_lane + (j % TPR));
                const uint8_t* bq = srowp + q * (CPT / 2);  // CPT codes = CPT / 2 bytes of each half of a block
                const float* xq = xp + q * CPT;
                auto block = [&](auto B) {
                    constexpr int b = decltype(B)::value;
                    constexpr int sh = (b % SPT) * 8;
                    const unsigned pk = pks[b / SPT];
                    // (s - 112) << 10: the f16 bits of 2^(s - 127)
                    const unsigned short ph = (unsigned short)(sh >= 10 ? (pk >> (sh - 10)) & 0x7C00u : (pk << (10 - sh)) & 0x7C00u);
                    mx4_block<CPT == 1 ? 2 : CPT, true>(bq + b * 16, 0, xq + b * 32, ph, 1.f, acc);
                };
                // (a stage holds sixteen blocks at most: seg <= 512)
                if (nb == 16) {
                    Unrolled<16>::run(block);
                } else {
                    Unrolled<16>::run([&](auto B) {
                        if (int(decltype(B)::value) < nb) block(B);
                    });
                }
            } else {
#pragma unroll 2
                for (int b = 0; b < nb; ++b) {
                    const unsigned pk = __shfl_sync(0xffffffffu, mxs, (lane / TPR) * TPR + b / SPT);
                    const float sc = e8m0_to_f32((pk >> ((b % SPT) * 8)) & 255u);
                    const uint8_t* bp = srowp + b * 16;
                    const float* xa = xp + b * 32 + q * CPT;
                    if (CPT > 1) {
                        mx4_block<CPT == 1 ? 2 : CPT, false>(bp, q, xa, 0, sc, acc);
                    } else {
                        const int sh = (q & 1) << 2;
                        acc[0] = fmaf(__fmul_rn(fp4_to_f32((bp[q >> 1] >> sh) & 15u), sc), *xa, acc[0]);
                        acc[0] = fmaf(__fmul_rn(fp4_to_f32((bp[8 + (q >> 1)] >> sh) & 15u), sc), *(xa + 16), acc[0]);
                    }
                }
            }
        } else {
            const int steps = n >> 4;
#pragma unroll 4
            for (int s = 0; s < steps; ++s) {
                const uint8_t* wp = srowp + s * 32 + q * CPT * 2;
                const float* xq = xp + s * 16 + q * CPT;
                if (CPT == 4) {
                    const uint2 wb = *reinterpret_cast<const uint2*>(wp);
                    const float4 xv = *reinterpret_cast<const float4*>(xq);
                    acc[0] = fmaf(bf_lo(wb.x), xv.x, acc[0]);
                    acc[1 % CPT] = fmaf(bf_hi(wb.x), xv.y, acc[1 % CPT]);
                    acc[2 % CPT] = fmaf(bf_lo(wb.y), xv.z, acc[2 % CPT]);
                    acc[3 % CPT] = fmaf(bf_hi(wb.y), xv.w, acc[3 % CPT]);
                } else if (CPT == 2) {
                    const uint32_t wb = *reinterpret_cast<const uint32_t*>(wp);
                    const float2 xv = *reinterpret_cast<const float2*>(xq);
                    acc[0] = fmaf(bf_lo(wb), xv.x, acc[0]);
                    acc[1 % CPT] = fmaf(bf_hi(wb), xv.y, acc[1 % CPT]);
                } else {
                    acc[0] = fmaf(__uint_as_float((uint32_t)*reinterpret_cast<const unsigned short*>(wp) << 16), *xq, acc[0]);
                }
            }
        }
        __syncwarp();
        if (issued < n_items) issue_next();
        if (c_seg == nseg - 1) {
            // reduce16's pairwise fold: chains 1 apart, 2 apart (both in this thread), 4 and 8 apart (the row's threads)
            float s = CPT == 4 ? (acc[0] + acc[1 % CPT]) + (acc[2 % CPT] + acc[3 % CPT]) : CPT == 2 ? acc[0] + acc[1 % CPT] : acc[0];
#pragma unroll
            for (int o = 1; o < TPR; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (A.glu_kind >= 0) {
                // the row's partner (its up row, or its gate row) sits TPR lanes away (rows 2j, 2j + 1) or four rows away
                const float other = __shfl_xor_sync(0xffffffffu, s, A.glu_kind == 0 ? 4 * TPR : TPR);
                const bool gate = A.glu_kind == 0 ? ri < 4 : !(ri & 1);
                if (live && q == 0 && gate)
                    A.glu_out[(size_t)task * (R >> 1) + (A.glu_kind == 0 ? r : r >> 1)] = moe_act_pair(s, other, A.glu_kind, A.alpha, A.limit);
            } else if (live && q == 0) {
                if (A.send.n == 0) {
                    A.y[(size_t)task * R + r] = s;
                } else {
                    const uint32_t word = b2_word(f2bf(s), b2_hop_mark(A.send.pass, A.send.per_pass, A.send.base));
                    const size_t at = (size_t)task * A.send.stride + A.send.offset + r;
#pragma unroll 1
                    for (int p = 0; p < A.send.n; ++p) A.send.out[p][at] = word;
                }
            }
#pragma unroll
            for (int u = 0; u < CPT; ++u) acc[u] = 0.f;
            c_seg = 0;
            c_grp += nw;
        } else {
            ++c_seg;
        }
        if (++c_st == S) {
            c_st = 0;
            c_par ^= 1u;
        }
    }
    if (!ok) {
        // a copy never landed: say so, then let the copies still in flight land (bounded) before the shared memory goes
        if (lane == 0) b2_fail(B2_ERR_TIMEOUT);
        for (int j = i + 1; j < issued; ++j) {
            if (++c_st == S) {
                c_st = 0;
                c_par ^= 1u;
            }
            mbar_wait_bounded(smem_u32(bars + c_st), c_par);
        }
    }
}

struct MSPlan {
    int ctas, warps, seg, stages, smem;
};

template <int FMT, int TPR>
bool plan_stream(int n_tasks, int R, int C, MSPlan& p) {
    constexpr int RB = 32 / TPR;
    // CTAs an SM holds: two measured best for MXFP4 rows (half the bytes a column, so twice the arithmetic a byte), one
    // for FP8 and bf16 rows at four threads a row
    const int per_sm = b2_tuning().ms_ctas > 0 ? b2_tuning().ms_ctas : (TPR == 4 && FMT != S_MX4 ? 1 : 2);
    const int sms = b2_sm_count();
    const int groups = (R + RB - 1) / RB;
    p.ctas = max(1, min(groups, per_sm * sms / max(1, n_tasks)));  // CTAs that share a task
    const int per_cta = (groups + p.ctas - 1) / p.ctas;
    p.warps = max(4, min(MAXW, per_cta));
    // even the rows out: with per_cta groups over the warps, fewer warps may idle less (the last round is fuller)
    {
        const int rounds = (per_cta + p.warps - 1) / p.warps;
        p.warps = max(4, (per_cta + rounds - 1) / rounds);
    }
    const int xbytes = x_smem_bytes(C);
    const int budget = (per_sm == 1 ? 200 : 104) * 1024 - xbytes;
    const B2Tuning& t = b2_tuning();
    if (t.ms_warps > 0) p.warps = min(MAXW, t.ms_warps);
    // (an MXFP4 stage holds at most 16 blocks of a row: the scale bytes its threads fetch ahead)
    for (p.seg = min(t.ms_seg > 0 && (FMT != S_MX4 || t.ms_seg <= 512) ? t.ms_seg : 512, (C + 31) & ~31);; p.seg = max(32, (p.seg / 2) & ~31)) {
        const int stride = p.seg * col_bytes2<FMT>() / 2 + PAD;
        const int sbytes = RB * stride;
        p.stages = max(2, min(6, budget / (p.warps * (sbytes + 8))));
        p.smem = xbytes + p.warps * p.stages * (sbytes + 8);
        if (p.smem <= (per_sm == 1 ? 220 : 110) * 1024 || p.seg == 32) break;  // two stages must fit: a narrower segment
    }
    return p.smem <= (per_sm == 1 ? 220 : 110) * 1024;
}

template <int FMT, int TPR>
int launch_stream_t(const MSArgs& a0, int n_tasks, cudaStream_t s) {
    MSPlan p;
    MSArgs a = a0;
    if (!plan_stream<FMT, TPR>(n_tasks, a.R, a.C, p)) return B2_ERR_DOMAIN;
    a.seg = p.seg, a.stages = p.stages;
    auto kern = moe_gemv_stream<FMT, TPR>;
    static bool allowed[64];
    int rc = b2_allow_smem(reinterpret_cast<const void*>(kern), allowed);
    if (rc) return rc;
    return b2_launch(reinterpret_cast<const void*>(kern), dim3(p.ctas, n_tasks), dim3(p.warps * 32), p.smem, s, a, 4);
}

template <int FMT>
int launch_stream(const MSArgs& a, int n_tasks, cudaStream_t s) {
    // threads a row: four measured best for every format (the conversion units bound the kernel, not latency)
    int tpr = b2_tuning().ms_tpr;
    if (tpr != 4 && tpr != 8 && tpr != 16) tpr = 4;
    switch (tpr) {
        case 4: return launch_stream_t<FMT, 4>(a, n_tasks, s);
        case 16: return launch_stream_t<FMT, 16>(a, n_tasks, s);
        default: return launch_stream_t<FMT, 8>(a, n_tasks, s);
    }
}

}  // namespace

// whether the streaming kernel takes the shape: rows and row segments must start on 16 bytes, x rows on 16
bool b2_moe_stream_ok(int fmt, const void* w, const void* scales, long long w_stride, long long s_stride, const void* x,
                      int R, int C, int sr, int sc) {
    if (reinterpret_cast<uintptr_t>(w) & 15 || reinterpret_cast<uintptr_t>(x) & 15 || (w_stride & 15) || (C & 31)) return false;
    if (fmt == S_FP8 && ((reinterpret_cast<uintptr_t>(scales) & 3) || (s_stride & 3) || R % sr || C % sc)) return false;
    return fmt == S_BF16 || fmt == S_MX4 || fmt == S_FP8;
}

int b2_moe_stream_launch(int fmt, const void* w, const void* scales, long long w_stride, long long s_stride, int sr, int sc,
                         const void* idx, int n_tasks, int E, const void* x, int x_div, void* y, int R, int C, int ep_rank,
                         int ep_size, int act_kind, float alpha, float limit, cudaStream_t s, const B2Send* send,
                         int glu_kind, void* glu_out) {
    MSArgs a{static_cast<const uint8_t*>(w), static_cast<const uint8_t*>(scales), w_stride, s_stride,
             static_cast<const int*>(idx), static_cast<const float*>(x), x_div, static_cast<float*>(y), R, C,
             sr > 0 ? sr : 1, sc > 0 ? sc : 1, E, ep_rank, ep_size, 0, 0, act_kind, alpha, limit, glu_kind,
             static_cast<float*>(glu_out), B2Send{}};
    if (send != nullptr) a.send = *send;
    if (glu_kind >= 0) {
        // pairs live in one warp: four threads a row (eight rows a warp), whole groups
        if (glu_out == nullptr || send != nullptr || act_kind >= 0 || (R & 7) || (glu_kind == 0 && ((R >> 1) & 3))) return B2_ERR_DOMAIN;
        switch (fmt) {
            case S_BF16: return launch_stream_t<S_BF16, 4>(a, n_tasks, s);
            case S_MX4: return launch_stream_t<S_MX4, 4>(a, n_tasks, s);
            case S_FP8: return launch_stream_t<S_FP8, 4>(a, n_tasks, s);
            default: return B2_ERR_DOMAIN;
        }
    }
    switch (fmt) {
        case S_BF16: return launch_stream<S_BF16>(a, n_tasks, s);
        case S_MX4: return launch_stream<S_MX4>(a, n_tasks, s);
        case S_FP8: return launch_stream<S_FP8>(a, n_tasks, s);
        default: return B2_ERR_DOMAIN;
    }
}
