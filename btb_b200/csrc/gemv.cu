// The decode GEMV family for sm_100a: y[m][r] = bf16(sum_c w[r][c] * x[m][c]), bf16 in, f32 accumulate.
//
// Arithmetic (what makes a row's bits): the reference's card order (native/cuda/btb_kernels.cu:83-142 of btb) - a
// row's K-sum is 32 independent f32 chains, chain l taking the 8-element chunks l, l+32, l+64, .. in order and a
// chunk's elements in index order, one fmaf each; the chains are folded by the butterfly xor 16, 8, 4, 2, 1 and the
// sum is rounded to bf16 once. Nothing here depends on M, R, the grid or the order the bytes arrive in, so row r of
// a 32-row verify pass is the one-row step's row r to the bit.
//
// Data movement (what makes it fast on B200): persistent CTAs, one per SM, each owning a contiguous range of rows.
// Every warp runs its own ring of shared-memory stages filled by the TMA unit's 1-D bulk copies
// (cp.async.bulk ... mbarrier::complete_tx) - one elected lane issues, the copy completes on the stage's mbarrier,
// the 32 lanes consume the stage with conflict-free 16-byte shared loads. A CTA keeps ring bytes (~100 KB) in
// flight whatever its register budget, which is what an 8 TB/s part needs (about 40 KB a SM by Little's law). The
// weight copies are issued BEFORE the grid-dependency wait, so under programmatic dependent launch the ring fills
// while the previous kernel of the step is still draining; x (the previous kernel's output) is staged into shared
// memory after the wait. Packed formats are widened to bf16 bit patterns in registers on the way from the stage to
// the FMA: no widened copy exists anywhere.
#include "common.cuh"
#include "btb_b200_internal.h"
#include "gemv_core.cuh"
#include "../../include/btb_b200.h"

B2_DEFINE_STATUS(gemv)

namespace {

// warps a CTA, a ring each: 8 or 16 (the tunable `warps`)

enum XMode { X_SMEM = 0, X_SMEM_SILU = 1, X_GLOBAL = 2, X_SMEM_NORM = 3 };

struct GemvArgs {
    const uint8_t* w;    // bf16: [R, C] bf16; p12: lo bytes [R*C]
    const uint8_t* hi4;  // p12: codes, two a byte
    const int32_t* esc_idx;
    const uint8_t* esc_val;
    const int32_t* esc_row;  // p12: [R+1] first escape at or past each row's start (a derived index)
    uint32_t table[4];       // p12: the 16 high bytes
    const bf16* x;           // [M, C], or gu [M, 2C] for the SwiGLU fold
    bf16* y;                 // [M, R]
    int R, C;
    int seg;     // elements a stage holds (a multiple of 256)
    int stages;  // ring depth
    int evict_first;
    // the residual + RMSNorm prologue (X_SMEM_NORM): x = rmsnorm(h_in + y) * w computed by every CTA on the way in,
    // h_out = h_in + y written by CTA 0 (h_in is never written here, so no CTA reads a half-updated row)
    const bf16* h_in;
    const bf16* y_add;   // null: no add
    const bf16* norm_w;
    bf16* h_out;         // null when y_add is null
    float eps;
    int centered;
    int T;               // live rows (rows T..M-1 of x are zeros)
    const float* fscales;  // FP8: the [sr, sc] f32 grid
    int fsc, fbm, fbn;     // its columns, a block's rows and columns
    // SwiGLU epilogue: w is [2 * pair, C] (gate rows, then up rows); a warp takes gate row p and up row p + pair one
    // after the other and writes y[m][p] = bf16(bf16(silu(bf16 g)) * bf16 u) - what btb_silu_mul makes of the two
    // outputs. 0: off. R counts pairs then.
    int pair;
    // a model cut over ranks by output rows (tp.cuh): with `recv.pass` set, x (or y_add under the norm prologue) is this
    // rank's copy of an exchanged vector, read word by word as the words arrive; with `send.n > 0` every output element
    // goes, marked, to each rank's copy of the full vector at [m][send.offset + row] instead of y
    B2Recv recv;
    B2Send send;
};

// NWT: the most warps a CTA of this instance is launched with (its register budget); the launch picks how many
// XCHG: the instance built for a model cut over ranks (marked words in, marked words out); the one-GPU instance carries
// none of that code
template <int M, int FMT, int XM, int NWT, bool XCHG>
__global__ void __launch_bounds__(NWT * 32, 1) gemv_stream(const GemvArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int NT = 0;  // the staging loops stride by the block's own width
    const int nw = blockDim.x >> 5;
    const int R = A.R, C = A.C, seg = A.seg, S = A.stages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nseg = (C + seg - 1) / seg;
    constexpr bool XS = XM != X_GLOBAL;

    // shared memory: [norm scratch][x: M*C bf16 when staged][rings: NWT * S stages][barriers: NWT * S]
    // (the norm prologue adds one f32 row of h and the 256 partial sums in front)
    const int nbytes = XM == X_SMEM_NORM ? ((C * 4 + 256 * 4 + 127) & ~127) : 0;
    const int xbytes = (XS ? ((M * C * 2 + 127) & ~127) : 0) + nbytes;
    const int sbytes = (stage_bytes<FMT>(seg) + 127) & ~127;
    bf16* xs = reinterpret_cast<bf16*>(smem + nbytes);
    uint8_t* ring = smem + xbytes + (size_t)warp * S * sbytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + xbytes + (size_t)nw * S * sbytes) + warp * S;

    // this CTA's rows [r0, r0 + cnt): an even split, the remainder one extra row to the first CTAs
    const int base = R / gridDim.x, rem = R % gridDim.x;
    const int r0 = blockIdx.x * base + min((int)blockIdx.x, rem);
    const int cnt = base + ((int)blockIdx.x < rem ? 1 : 0);
    // this warp's rows: r0 + warp, + nw, ..; its items are (row, segment) pairs in order
    const int my_rows = cnt > warp ? (cnt - warp + nw - 1) / nw : 0;
    const int n_items = my_rows * nseg * (A.pair != 0 ? 2 : 1);

    if (lane == 0) {
        for (int s = 0; s < S; ++s) mbar_init(smem_u32(bars + s), 1);
        mbar_fence_init();
    }
    __syncwarp();

    const uint64_t pol = A.evict_first ? l2_evict_first_policy() : 0;
    // the producer's cursor: the next item to copy (kept by every lane, issued by lane 0); no division on the way
    int p_row = r0 + warp, p_seg = 0, p_st = 0, issued = 0, p_sub = 0;
    const int pair = A.pair;
    auto issue_next = [&]() {
        const int c0 = p_seg * seg;
        const int n = min(seg, C - c0);
        if (lane == 0) {
            const uint32_t bar = smem_u32(bars + p_st);
            const uint32_t dst = smem_u32(ring + (size_t)p_st * sbytes);
            const size_t e0 = (size_t)(p_row + p_sub * pair) * C + c0;
            if (FMT == F_BF16 || FMT == F_FP8) {
                const uint32_t nb = FMT == F_BF16 ? n * 2 : n;
                mbar_expect_tx(bar, nb);
                if (A.evict_first) bulk_g2s_hint(dst, A.w + e0 * (FMT == F_BF16 ? 2 : 1), nb, bar, pol);
                else bulk_g2s(dst, A.w + e0 * (FMT == F_BF16 ? 2 : 1), nb, bar);
            } else {
                mbar_expect_tx(bar, n + n / 2);
                if (A.evict_first) {
                    bulk_g2s_hint(dst, A.w + e0, n, bar, pol);
                    bulk_g2s_hint(dst + seg, A.hi4 + e0 / 2, n / 2, bar, pol);
                } else {
                    bulk_g2s(dst, A.w + e0, n, bar);
                    bulk_g2s(dst + seg, A.hi4 + e0 / 2, n / 2, bar);
                }
            }
        }
        ++issued;
        if (++p_st == S) p_st = 0;
        if (++p_seg == nseg) {
            p_seg = 0;
            if (pair != 0 && p_sub == 0) {
                p_sub = 1;  // the pair's up row next
            } else {
                p_sub = 0;
                p_row += nw;
            }
        }
    };
    // fill the ring: weights do not depend on the grids before this one
    {
        const int first = min(S, n_items);
        for (int i = 0; i < first; ++i) issue_next();
    }

    pdl_launch_dependents();
    pdl_wait();  // x is the previous kernel's output
    // ... or, in a model cut over ranks, every rank's: the words are taken as they arrive
    const bool marked = XCHG && A.recv.pass != nullptr;
    const uint32_t mark_in = marked ? b2_hop_mark(A.recv.pass, A.recv.per_pass, A.recv.base) : 0u;
    const uint32_t mark_out = XCHG && A.send.n != 0 ? b2_hop_mark(A.send.pass, A.send.per_pass, A.send.base) : 0u;

    if (XS) {
        if (XM == X_SMEM) stage_x_copy<M, NT>(xs, A.x, C, marked, mark_in, A.T);
        else if (XM == X_SMEM_SILU) stage_x_silu<M, NT>(xs, A.x, C);
        else
            stage_x_norm<M, NT>(xs, reinterpret_cast<float*>(smem), A.h_in, nullptr, A.y_add, A.norm_w, A.h_out, A.eps,
                                A.centered, A.T, C, blockIdx.x == 0, marked, mark_in);
        __syncthreads();
    }

    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    bool ok = true;
    // the consumer's cursor
    int c_row = r0 + warp, c_seg = 0, c_st = 0, c_sub = 0;
    uint32_t c_par = 0;
    float gate[M];  // a pair's gate outputs (bf16 values) while its up row streams
    int i = 0;
    for (; i < n_items; ++i) {
        if (!mbar_wait_bounded(smem_u32(bars + c_st), c_par)) {
            ok = false;
            break;
        }
        const int row = c_row + c_sub * pair;
        const int c0 = c_seg * seg;
        const int nch = min(seg, C - c0) >> 3;  // the segment's chunks; its first chunk is global chunk c0 / 8
        const uint8_t* stg = ring + (size_t)c_st * sbytes;
        WidenCtx wc;
        wc.esc_idx = A.esc_idx, wc.esc_val = A.esc_val, wc.e0 = 0, wc.e1 = 0, wc.srow = nullptr, wc.bn = 8;
        wc.table[0] = A.table[0], wc.table[1] = A.table[1], wc.table[2] = A.table[2], wc.table[3] = A.table[3];
        if (FMT == F_P12 && A.esc_row != nullptr) {
            wc.e0 = __ldg(A.esc_row + row);
            wc.e1 = __ldg(A.esc_row + row + 1);
        }
        if (FMT == F_FP8) wc.srow = A.fscales + (size_t)(row / A.fbm) * A.fsc, wc.bn = A.fbn;
        consume_stage<M, FMT, XS>(acc, stg, seg, nch, c0, row, C, XS ? xs : A.x, wc, lane);
        // the stage is free once every lane has read it (the warp barrier orders their shared loads before the
        // elected lane's copy, as a consumer's release orders them in any TMA pipeline): refill it with the next item
        __syncwarp();
        if (issued < n_items) issue_next();
        if (c_seg == nseg - 1) {
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const float s = warp_sum(acc[m]);
                if (pair != 0 && c_sub == 0) {
                    gate[m] = bfround(s);
                } else if (lane == 0) {
                    const bf16 v = pair == 0 ? f2bf(s) : f2bf(bfround(act_silu(gate[m])) * bfround(s));
                    if (!XCHG || A.send.n == 0) {
                        A.y[(size_t)m * R + c_row] = v;
                    } else {
                        const size_t at = (size_t)m * A.send.stride + A.send.offset + c_row;
                        const uint32_t word = b2_word(v, mark_out);
#pragma unroll 1
                        for (int p = 0; p < A.send.n; ++p) A.send.out[p][at] = word;
                    }
                }
                acc[m] = 0.f;
            }
            c_seg = 0;
            if (pair != 0 && c_sub == 0) {
                c_sub = 1;
            } else {
                c_sub = 0;
                c_row += nw;
            }
        } else {
            ++c_seg;
        }
        if (++c_st == S) {
            c_st = 0;
            c_par ^= 1u;
        }
    }
    if (!ok) {
        // a copy never landed: say so, then let the copies still in flight land (bounded) before the CTA's shared
        // memory goes away
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

// ---- host side -----------------------------------------------------------------------------------------------------

struct Plan {
    int grid, seg, stages, smem, nw;
    bool xs;
};

// ring geometry: split a row into equal segments of at most `max_seg_bytes`, each a multiple of 256 elements (so a
// lane's chunk l + 32 j of the row is chunk l + 32 j' of its segment), as many stages as the per-warp budget holds
template <int FMT>
Plan make_plan(int M, int R, int C, bool want_xs, bool norm = false) {
    const B2Tuning& t = b2_tuning();
    Plan p;
    const int sms = b2_sm_count();
    // The unit of work is a row on a warp (the chain order allows no finer cut), so the pass takes as long as the
    // warp with the most rows: pick the grid and the CTA's warps so that the rows divide evenly. R = 2560 over 148
    // CTAs of 16 warps leaves most warps one row and some two - half the card idles through the second; 128 CTAs of
    // 20 warps take one row each. Wide passes keep 8 warps (their accumulators fill the register file).
    const int w_max = M <= 2 ? 32 : (M <= 8 ? 16 : 8);
    int NW = (M <= 2 && t.warps >= 16) ? 16 : 8;
    p.grid = max(1, min(sms * t.ctas_per_sm, (R + 1) / 2));
    // the warps a CTA is given when the rows divide as evenly either way: 16 for bf16 rows (memory-bound: more warps only
    // thin the rings), `warps_packed` for rows widened in registers (bound by instruction issue: more warps fill more slots)
    const int pref = FMT == F_BF16 || t.warps_packed <= 0 ? 16 : min(w_max, t.warps_packed);
    if (t.balance && t.ctas_per_sm == 1 && R >= sms) {
        double best = 0.0;
        for (int g = sms; g >= (sms * 3) / 4; --g) {
            const int per_cta = (R + g - 1) / g;
            for (int w = 8; w <= w_max; ++w) {
                const int per_warp = (per_cta + w - 1) / w;
                // rows done a unit of time, with a mild preference for more SMs and for the usual 16 warps
                const double eff = (double)R / ((double)per_warp * g * w) * (0.9 + 0.1 * g / sms) - 0.002 * abs(w - pref);
                if (eff > best + 1e-9) best = eff, p.grid = g, NW = w;
            }
        }
    }
    p.nw = NW;
    const int xbytes = ((M * C * 2 + 127) & ~127) + (norm ? ((C * 4 + 256 * 4 + 127) & ~127) : 0);
    p.xs = want_xs && (M * C * 2) <= t.x_smem_max;
    const int ring = t.ring_bytes;
    int per_warp = ring / NW;
    int max_seg_el = t.seg_bytes / (FMT == F_BF16 ? 2 : 1);  // elements (pack12 and FP8: a byte and a bit each)
    max_seg_el = max(256, max_seg_el & ~255);
    int sb = 0;
    auto total = [&](int st) { return (p.xs ? xbytes : 0) + NW * st * sb + NW * st * 8; };
    for (;;) {
        const int nseg = (C + max_seg_el - 1) / max_seg_el;
        int seg = (C + nseg - 1) / nseg;
        seg = (seg + 255) & ~255;
        p.seg = seg;
        sb = (stage_bytes<FMT>(seg) + 127) & ~127;
        p.stages = max(2, min(8, per_warp / sb));
        while (p.stages > 2 && total(p.stages) > 224 * 1024) --p.stages;
        if (total(p.stages) <= 224 * 1024) break;
        if (max_seg_el > 256) {
            max_seg_el = max(256, (max_seg_el / 2) & ~255);  // two stages of this size do not fit: halve the segment
        } else if (p.xs) {
            p.xs = false;  // a very wide x gives its shared memory back to the ring
        } else {
            break;
        }
    }
    p.smem = total(p.stages);
    // Under programmatic dependent launch the next GEMV's CTAs arrive while this one's are still resident. Two CTAs
    // of one grid on an SM would make that SM the pass's slowest, so a CTA claims more than half an SM's shared memory.
    if ((t.pdl & 1) && t.solo) p.smem = max(p.smem, 116 * 1024);
    return p;
}

template <int M, int FMT, int XM, int NWT, bool XCHG>
int launch_x(const GemvArgs& a, const Plan& p, cudaStream_t stream) {
    auto kern = gemv_stream<M, FMT, XM, NWT, XCHG>;
    static bool allowed[64];  // the opt-in past 48 KB of dynamic shared memory, once a device
    int rc = b2_allow_smem(reinterpret_cast<const void*>(kern), allowed);
    if (rc) return rc;
    if (p.nw > NWT) return B2_ERR_DOMAIN;
    return b2_launch(reinterpret_cast<const void*>(kern), dim3(p.grid), dim3(p.nw * 32), p.smem, stream, a, 1);
}
template <int M, int FMT, int XM, int NWT>
int launch_nw(const GemvArgs& a, const Plan& p, cudaStream_t stream) {
    // the exchange is built for bf16 weights with x staged plainly or under the norm prologue, and for wide passes' sends
    constexpr bool CAN = FMT == F_BF16 && XM != X_SMEM_SILU;
    if (a.recv.pass != nullptr || a.send.n != 0) {
        if (!CAN) return B2_ERR_DOMAIN;
        return launch_x<M, FMT, XM, NWT, CAN>(a, p, stream);
    }
    return launch_x<M, FMT, XM, NWT, false>(a, p, stream);
}
template <int M, int FMT, int XM>
int launch_one(const GemvArgs& a, const Plan& p, cudaStream_t stream) {
    // one instance a register budget: up to 16 warps (128 registers a thread) and, for one- and two-row passes, up to 32
    if (M <= 2 && p.nw > 24) return launch_nw<M, FMT, XM, (M <= 2 ? 32 : 8)>(a, p, stream);
    // (24 warps leave a thread 80 registers: the packed formats' decode tables stay in them)
    if (M <= 2 && p.nw > 16) return launch_nw<M, FMT, XM, (M <= 2 ? 24 : 8)>(a, p, stream);
    if (M <= 8 && p.nw > 8) return launch_nw<M, FMT, XM, (M <= 8 ? 16 : 8)>(a, p, stream);
    return launch_nw<M, FMT, XM, 8>(a, p, stream);
}

template <int FMT, int XM>
int launch_m(int M, const GemvArgs& a, const Plan& p, cudaStream_t s) {
    switch (M) {
        case 1: return launch_one<1, FMT, XM>(a, p, s);
        case 2: return launch_one<2, FMT, XM>(a, p, s);
        case 4: return launch_one<4, FMT, XM>(a, p, s);
        case 8: return launch_one<8, FMT, XM>(a, p, s);
        default: return B2_ERR_DOMAIN;
    }
}
template <int FMT>
int launch_m_global(int M, const GemvArgs& a, const Plan& p, cudaStream_t s) {
    switch (M) {
        case 1: return launch_one<1, FMT, X_GLOBAL>(a, p, s);
        case 2: return launch_one<2, FMT, X_GLOBAL>(a, p, s);
        case 4: return launch_one<4, FMT, X_GLOBAL>(a, p, s);
        case 8: return launch_one<8, FMT, X_GLOBAL>(a, p, s);
        case 16: return launch_one<16, FMT, X_GLOBAL>(a, p, s);
        case 32: return launch_one<32, FMT, X_GLOBAL>(a, p, s);
        default: return B2_ERR_DOMAIN;
    }
}

int check_dims(const void* w, const void* x, const void* y, int M, int R, int C) {
    if (w == nullptr || x == nullptr || y == nullptr) return B2_ERR_NULL;
    if (R <= 0 || C <= 0 || (C & 7) != 0) return B2_ERR_DOMAIN;
    if (M != 1 && M != 2 && M != 4 && M != 8 && M != 16 && M != 32) return B2_ERR_DOMAIN;
    if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(x) & 15)) return B2_ERR_DOMAIN;
    return B2_OK;
}

}  // namespace

// esc_row[r] = the first escape at or past row r's first element (r = 0..R): the CPU kernel's per-row cursor
// (native/src/gemv.rs:720-735 of btb) computed once when the weights are loaded
namespace {
struct P12RowsArgs {
    const int32_t* esc_idx;
    int32_t* esc_row;
    int n_esc, R, C;
};
__global__ void __launch_bounds__(256) p12_rows(const P12RowsArgs A) {
    const int r = blockIdx.x * 256 + threadIdx.x;
    if (r > A.R) return;
    const long long start = (long long)r * A.C;
    int a = 0, b = A.n_esc;
    while (a < b) {
        const int mid = (a + b) >> 1;
        if ((long long)A.esc_idx[mid] < start) a = mid + 1;
        else b = mid;
    }
    A.esc_row[r] = a;
}
}  // namespace

extern "C" int btb_b200_p12_rows(const void* esc_idx, int n_esc, int R, int C, void* esc_row, void* stream) {
    if (esc_row == nullptr || (n_esc > 0 && esc_idx == nullptr)) return B2_ERR_NULL;
    if (n_esc < 0 || R <= 0 || C <= 0) return B2_ERR_DOMAIN;
    P12RowsArgs a{static_cast<const int32_t*>(esc_idx), static_cast<int32_t*>(esc_row), n_esc, R, C};
    return b2_launch((const void*)p12_rows, dim3((R + 1 + 255) / 256), dim3(256), 0, static_cast<cudaStream_t>(stream),
                     a);
}

// the exchange descriptors of the C-ABI (include/btb_b200.h) into the kernels' own; refuses what a kernel could fault on
static int take_exchange(const btb_b200_recv* recv, const btb_b200_send* send, GemvArgs& a) {
    if (recv != nullptr && recv->pass != nullptr)
        a.recv = B2Recv{static_cast<const unsigned*>(recv->pass), recv->per_pass, recv->base};
    if (send != nullptr && send->n != 0) {
        if (send->n < 0 || send->n > B2_MAX_RANKS || send->stride <= 0 || send->offset < 0 ||
            send->offset + a.R > send->stride)
            return B2_ERR_DOMAIN;
        if (send->pass == nullptr) return B2_ERR_NULL;
        a.send.n = send->n, a.send.stride = send->stride, a.send.offset = send->offset;
        a.send.pass = static_cast<const unsigned*>(send->pass), a.send.per_pass = send->per_pass, a.send.base = send->base;
        for (int p = 0; p < send->n; ++p) {
            if (send->out[p] == nullptr || (reinterpret_cast<uintptr_t>(send->out[p]) & 15)) return B2_ERR_NULL;
            a.send.out[p] = static_cast<uint32_t*>(send->out[p]);
        }
    }
    return B2_OK;
}

static int gemv_bf16_impl(const void* w, const void* x, void* y, int T, int M, int R, int C, const btb_b200_recv* recv,
                          const btb_b200_send* send, void* stream) {
    const bool sends = send != nullptr && send->n != 0;
    int rc = check_dims(w, x, sends ? w : y, M, R, C);  // a sending launch has no local y
    if (rc) return rc;
    GemvArgs a{};
    a.w = static_cast<const uint8_t*>(w);
    a.x = static_cast<const bf16*>(x);
    a.y = static_cast<bf16*>(y);
    a.R = R, a.C = C, a.T = T;
    if (T < 1 || T > M) return B2_ERR_DOMAIN;
    if ((rc = take_exchange(recv, send, a)) != B2_OK) return rc;
    Plan p = make_plan<F_BF16>(M, R, C, M <= 8 && !(M == 1 && b2_tuning().x_direct && a.recv.pass == nullptr));
    // an exchanged x is decoded on its way into shared memory: a pass too wide to stage x takes btb_b200_xchg_unpack first
    if (a.recv.pass != nullptr && !p.xs) return B2_ERR_DOMAIN;
    a.seg = p.seg, a.stages = p.stages, a.evict_first = b2_tuning().evict_first;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return p.xs ? launch_m<F_BF16, X_SMEM>(M, a, p, s) : launch_m_global<F_BF16>(M, a, p, s);
}

extern "C" int btb_b200_gemv_bf16(const void* w, const void* x, void* y, int M, int R, int C, void* stream) {
    return gemv_bf16_impl(w, x, y, M, M, R, C, nullptr, nullptr, stream);
}

extern "C" int btb_b200_gemv_bf16_x(const void* w, const void* x, void* y, int T, int M, int R, int C,
                                    const btb_b200_recv* recv, const btb_b200_send* send, void* stream) {
    return gemv_bf16_impl(w, x, y, T, M, R, C, recv, send, stream);
}

// x = rmsnorm(h_in + y) * w computed inside the GEMV (bf16 weights, or pack12 when hi4 is not null); swiglu: the rows are
// gate then up and the output is the activated product of each pair
static int gemv_norm_impl(const void* w, const void* hi4, const void* table, const void* esc_idx, const void* esc_val,
                          const void* esc_row, const void* h_in, const void* y_add, const void* norm_w, float eps,
                          int centered, void* h_out, void* y, int T, int M, int R, int C, bool swiglu, void* stream,
                          const btb_b200_recv* recv = nullptr, const btb_b200_send* send = nullptr,
                          const void* fp8_scales = nullptr, int sr = 0, int sc = 0) {
    const bool sends = send != nullptr && send->n != 0;
    int rc = check_dims(w, h_in, sends ? w : y, M, R, C);
    if (rc) return rc;
    if (norm_w == nullptr || (y_add != nullptr && h_out == nullptr)) return B2_ERR_NULL;
    if (T <= 0 || T > M || M > 8 || !(eps == eps) || h_out == h_in) return B2_ERR_DOMAIN;
    if (swiglu && (R & 1)) return B2_ERR_DOMAIN;
    if (reinterpret_cast<uintptr_t>(norm_w) & 15) return B2_ERR_DOMAIN;  // read as 16-byte vectors
    const bool p12 = hi4 != nullptr;
    if (p12 && (table == nullptr || (C & 31) != 0 || (reinterpret_cast<uintptr_t>(hi4) & 15))) return B2_ERR_DOMAIN;
    if (p12 && esc_row != nullptr && (esc_idx == nullptr || esc_val == nullptr)) return B2_ERR_NULL;
    GemvArgs a{};
    a.w = static_cast<const uint8_t*>(w);
    a.hi4 = static_cast<const uint8_t*>(hi4);
    a.esc_idx = static_cast<const int32_t*>(esc_idx);
    a.esc_val = static_cast<const uint8_t*>(esc_val);
    a.esc_row = static_cast<const int32_t*>(esc_row);
    if (p12) memcpy(a.table, table, 16);
    a.y = static_cast<bf16*>(y);
    a.R = swiglu ? R / 2 : R, a.C = C;
    a.pair = swiglu ? R / 2 : 0;
    a.h_in = static_cast<const bf16*>(h_in), a.y_add = static_cast<const bf16*>(y_add);
    a.norm_w = static_cast<const bf16*>(norm_w), a.h_out = static_cast<bf16*>(h_out);
    a.eps = eps, a.centered = centered, a.T = T;
    if ((rc = take_exchange(recv, send, a)) != B2_OK) return rc;
    if (a.recv.pass != nullptr && y_add == nullptr) return B2_ERR_NULL;  // the exchanged input of this form is y_add
    const bool fp8 = fp8_scales != nullptr;
    if (fp8) {
        if (p12 || swiglu || sr <= 0 || sc <= 0 || R % sr || C % sc || (C & 15) || ((C / sc) & 7)) return B2_ERR_DOMAIN;
        a.fscales = static_cast<const float*>(fp8_scales);
        a.fsc = sc, a.fbm = R / sr, a.fbn = C / sc;
    }
    Plan p = fp8 ? make_plan<F_FP8>(M, a.R, C, true, true)
                 : p12 ? make_plan<F_P12>(M, a.R, C, true, true) : make_plan<F_BF16>(M, a.R, C, true, true);
    if (!p.xs) return B2_ERR_DOMAIN;  // too wide to stage: the caller runs btb_b200_add_rmsnorm and the plain GEMV
    a.seg = p.seg, a.stages = p.stages, a.evict_first = b2_tuning().evict_first;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (fp8) return launch_m<F_FP8, X_SMEM_NORM>(M, a, p, s);
    return p12 ? launch_m<F_P12, X_SMEM_NORM>(M, a, p, s) : launch_m<F_BF16, X_SMEM_NORM>(M, a, p, s);
}

extern "C" int btb_b200_gemv_norm(const void* w, const void* hi4, const void* table, const void* esc_idx,
                                  const void* esc_val, const void* esc_row, const void* h_in, const void* y_add,
                                  const void* norm_w, float eps, int centered, void* h_out, void* y, int T, int M, int R,
                                  int C, void* stream) {
    return gemv_norm_impl(w, hi4, table, esc_idx, esc_val, esc_row, h_in, y_add, norm_w, eps, centered, h_out, y, T, M, R,
                          C, false, stream);
}

extern "C" int btb_b200_gemv_norm_swiglu(const void* w, const void* hi4, const void* table, const void* esc_idx,
                                         const void* esc_val, const void* esc_row, const void* h_in, const void* y_add,
                                         const void* norm_w, float eps, int centered, void* h_out, void* m_out, int T,
                                         int M, int R, int C, void* stream) {
    return gemv_norm_impl(w, hi4, table, esc_idx, esc_val, esc_row, h_in, y_add, norm_w, eps, centered, h_out, m_out, T, M,
                          R, C, true, stream);
}

// btb_b200_gemv_norm / _norm_swiglu over bf16 weights in a model cut over ranks: with `recv`, y_add is this rank's copy
// of the previous block's exchanged output (marked words); with `send`, the outputs go to every rank's copy of the next
extern "C" int btb_b200_gemv_norm_x(const void* w, const void* h_in, const void* y_add, const void* norm_w, float eps,
                                    int centered, void* h_out, void* y, int T, int M, int R, int C, int swiglu,
                                    const btb_b200_recv* recv, const btb_b200_send* send, void* stream) {
    return gemv_norm_impl(w, nullptr, nullptr, nullptr, nullptr, nullptr, h_in, y_add, norm_w, eps, centered, h_out, y, T, M,
                          R, C, swiglu != 0, stream, recv, send);
}

// btb_b200_gemv_norm over FP8 weights (the widen of btb_b200_gemv_fp8)
extern "C" int btb_b200_gemv_norm_fp8(const void* w, const void* scales, int sr, int sc, const void* h_in, const void* y_add,
                                      const void* norm_w, float eps, int centered, void* h_out, void* y, int T, int M, int R,
                                      int C, void* stream) {
    if (scales == nullptr) return B2_ERR_NULL;
    return gemv_norm_impl(w, nullptr, nullptr, nullptr, nullptr, nullptr, h_in, y_add, norm_w, eps, centered, h_out, y, T, M,
                          R, C, false, stream, nullptr, nullptr, scales, sr, sc);
}

// FP8 e4m3 weights with an f32 [sr, sc] block-scale grid, each weight the bf16 btb holds for it, widened in registers
extern "C" int btb_b200_gemv_fp8(const void* w, const void* scales, int sr, int sc, const void* x, void* y, int M, int R,
                                 int C, void* stream) {
    int rc = check_dims(w, x, y, M, R, C);
    if (rc) return rc;
    if (scales == nullptr) return B2_ERR_NULL;
    // a row's bytes are bulk-copied from its own offset (16-byte aligned: C a multiple of 16) and a chunk of eight
    // columns lies in one scale block
    if (sr <= 0 || sc <= 0 || R % sr || C % sc || (C & 15) || ((C / sc) & 7)) return B2_ERR_DOMAIN;
    GemvArgs a{};
    a.w = static_cast<const uint8_t*>(w);
    a.fscales = static_cast<const float*>(scales);
    a.fsc = sc, a.fbm = R / sr, a.fbn = C / sc;
    a.x = static_cast<const bf16*>(x);
    a.y = static_cast<bf16*>(y);
    a.R = R, a.C = C;
    Plan p = make_plan<F_FP8>(M, R, C, M <= 8);
    a.seg = p.seg, a.stages = p.stages, a.evict_first = b2_tuning().evict_first;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return p.xs ? launch_m<F_FP8, X_SMEM>(M, a, p, s) : launch_m_global<F_FP8>(M, a, p, s);
}

extern "C" int btb_b200_gemv_silu_bf16(const void* w, const void* gu, void* y, int M, int R, int C, void* stream) {
    int rc = check_dims(w, gu, y, M, R, C);
    if (rc) return rc;
    GemvArgs a{};
    a.w = static_cast<const uint8_t*>(w);
    a.x = static_cast<const bf16*>(gu);
    a.y = static_cast<bf16*>(y);
    a.R = R, a.C = C;
    Plan p = make_plan<F_BF16>(M, R, C, true);
    // the fold stages the activated x in shared memory; a pass too wide for that takes btb_b200_silu_mul and the
    // plain GEMV (the same bits)
    if (!p.xs || M > 8) return B2_ERR_DOMAIN;
    a.seg = p.seg, a.stages = p.stages, a.evict_first = b2_tuning().evict_first;
    return launch_m<F_BF16, X_SMEM_SILU>(M, a, p, static_cast<cudaStream_t>(stream));
}

// the SwiGLU fold over pack12 weights
extern "C" int btb_b200_gemv_silu_p12(const void* lo, const void* hi4, const void* table, const void* esc_idx,
                                      const void* esc_val, const void* esc_row, const void* gu, void* y, int M, int R,
                                      int C, void* stream) {
    int rc = check_dims(lo, gu, y, M, R, C);
    if (rc) return rc;
    if (hi4 == nullptr || table == nullptr) return B2_ERR_NULL;
    if ((C & 31) != 0 || (reinterpret_cast<uintptr_t>(hi4) & 15)) return B2_ERR_DOMAIN;
    GemvArgs a{};
    a.w = static_cast<const uint8_t*>(lo);
    a.hi4 = static_cast<const uint8_t*>(hi4);
    a.esc_idx = static_cast<const int32_t*>(esc_idx);
    a.esc_val = static_cast<const uint8_t*>(esc_val);
    a.esc_row = static_cast<const int32_t*>(esc_row);
    if (a.esc_row != nullptr && (a.esc_idx == nullptr || a.esc_val == nullptr)) return B2_ERR_NULL;
    memcpy(a.table, table, 16);
    a.x = static_cast<const bf16*>(gu);
    a.y = static_cast<bf16*>(y);
    a.R = R, a.C = C;
    Plan p = make_plan<F_P12>(M, R, C, true);
    if (!p.xs || M > 8) return B2_ERR_DOMAIN;
    a.seg = p.seg, a.stages = p.stages, a.evict_first = b2_tuning().evict_first;
    return launch_m<F_P12, X_SMEM_SILU>(M, a, p, static_cast<cudaStream_t>(stream));
}

extern "C" int btb_b200_gemv_p12(const void* lo, const void* hi4, const void* table, const void* esc_idx,
                                 const void* esc_val, const void* esc_row, const void* x, void* y, int M, int R, int C,
                                 void* stream) {
    int rc = check_dims(lo, x, y, M, R, C);
    if (rc) return rc;
    if (hi4 == nullptr || table == nullptr) return B2_ERR_NULL;
    // a row's low bytes and codes are bulk-copied from their own offsets: both must start on 16 bytes
    if ((C & 31) != 0 || (reinterpret_cast<uintptr_t>(hi4) & 15)) return B2_ERR_DOMAIN;
    GemvArgs a{};
    a.w = static_cast<const uint8_t*>(lo);
    a.hi4 = static_cast<const uint8_t*>(hi4);
    a.esc_idx = static_cast<const int32_t*>(esc_idx);
    a.esc_val = static_cast<const uint8_t*>(esc_val);
    a.esc_row = static_cast<const int32_t*>(esc_row);
    if (a.esc_row != nullptr && (a.esc_idx == nullptr || a.esc_val == nullptr)) return B2_ERR_NULL;
    memcpy(a.table, table, 16);  // host pointer: the 16-byte table travels in the launch's arguments
    a.x = static_cast<const bf16*>(x);
    a.y = static_cast<bf16*>(y);
    a.R = R, a.C = C;
    Plan p = make_plan<F_P12>(M, R, C, M <= 8);
    a.seg = p.seg, a.stages = p.stages, a.evict_first = b2_tuning().evict_first;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return p.xs ? launch_m<F_P12, X_SMEM>(M, a, p, s) : launch_m_global<F_P12>(M, a, p, s);
}
