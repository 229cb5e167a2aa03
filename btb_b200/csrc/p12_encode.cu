// pack12 encoding on the card: a bf16 tensor into the parts the fused-widen GEMV reads (btb_b200_gemv_p12), without the
// tensor leaving HBM.
//
// The format is btb's (btb/pack12.py:1-14, 48-68 of btb): an element is its low byte and a 4-bit code into a table of
// the 15 most frequent high bytes (by count descending, ties by byte value ascending); code 15 marks an escape, listed
// by ascending element index with its high byte; codes are packed two a byte, the even element in the low nibble. The
// parts written here are byte-identical to that encoder's.
//
// How it runs: (1) a 256-bin histogram of the high bytes, per-CTA in shared memory, merged with global atomics (integer
// counts: the order of the adds does not matter); (2) the table chosen on the host from the 256 counts; (3) one pass
// that writes the low bytes and the packed codes and counts each 2048-element tile's escapes, a one-CTA exclusive scan
// of the tile counts, and (4) a pass that writes each tile's escapes at its offset in ascending index order (a warp
// takes 32 consecutive elements: ballot + popcount give the position inside the tile). Load-time work, bound by HBM.
#include "btb_b200_internal.h"

namespace {

constexpr int TILE = 2048;  // elements a CTA of 256 threads encodes: 8 a thread

struct HistArgs {
    const uint16_t* src;
    long long n;
    unsigned* hist;
};
__global__ void __launch_bounds__(256) p12_hist(const HistArgs A) {
    __shared__ unsigned h[256];
    h[threadIdx.x] = 0u;
    __syncthreads();
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < A.n; i += (long long)gridDim.x * 256)
        atomicAdd(&h[A.src[i] >> 8], 1u);
    __syncthreads();
    if (h[threadIdx.x] != 0u) atomicAdd(A.hist + threadIdx.x, h[threadIdx.x]);
}

struct EncArgs {
    const uint16_t* src;
    long long n;
    uint8_t code_of[256];  // high byte -> code (15: not in the table)
    uint8_t* lo;
    uint8_t* hi4;
    int* tile_esc;  // [tiles + 1]
};
// a thread takes 8 consecutive elements: 8 low bytes, 4 packed code bytes
__global__ void __launch_bounds__(256) p12_encode(const EncArgs A) {
    __shared__ uint8_t code_of[256];
    __shared__ int wsum[8];
    code_of[threadIdx.x] = A.code_of[threadIdx.x];
    __syncthreads();
    const long long e0 = ((long long)blockIdx.x * 256 + threadIdx.x) * 8;
    int esc = 0;
    uint32_t packed = 0u;
    uint8_t lows[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const long long i = e0 + k;
        const uint16_t v = i < A.n ? A.src[i] : (uint16_t)0;
        const uint32_t c = i < A.n ? code_of[v >> 8] : 0u;  // the pad nibble of an odd count is 0
        lows[k] = (uint8_t)(v & 0xff);
        packed |= c << (4 * k);
        esc += (i < A.n && c == 15u) ? 1 : 0;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k)
        if (e0 + k < A.n) A.lo[e0 + k] = lows[k];
#pragma unroll
    for (int k = 0; k < 4; ++k)
        if (e0 + 2 * k < A.n) A.hi4[(e0 >> 1) + k] = (uint8_t)((packed >> (8 * k)) & 0xff);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) esc += __shfl_xor_sync(0xffffffffu, esc, o);
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = esc;
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int w = 0; w < 8; ++w) t += wsum[w];
        A.tile_esc[blockIdx.x] = t;
    }
}

struct ScanArgs {
    int* v;  // [n + 1]: counts in, exclusive offsets out, v[n] the total
    int n;
};
// one CTA walks the tile counts 1024 at a time (a load-time pass over at most a million tiles)
__global__ void __launch_bounds__(1024) p12_scan(const ScanArgs A) {
    __shared__ int part[32];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < A.n; base += 1024) {
        const int i = base + threadIdx.x;
        const int mine = i < A.n ? A.v[i] : 0;
        int inc = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, inc, o);
            if ((threadIdx.x & 31) >= o) inc += t;
        }
        if ((threadIdx.x & 31) == 31) part[threadIdx.x >> 5] = inc;
        __syncthreads();
        if (threadIdx.x < 32) {
            int p = part[threadIdx.x];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, p, o);
                if (threadIdx.x >= o) p += t;
            }
            part[threadIdx.x] = p;  // inclusive over the warps
        }
        __syncthreads();
        const int before = carry + (threadIdx.x >= 32 ? part[(threadIdx.x >> 5) - 1] : 0);
        if (i < A.n) A.v[i] = before + inc - mine;
        __syncthreads();
        if (threadIdx.x == 1023) carry = before + inc;
        __syncthreads();
    }
    if (threadIdx.x == 0) A.v[A.n] = carry;
}

struct EscArgs {
    const uint16_t* src;
    long long n;
    uint8_t code_of[256];
    const int* tile_off;  // [tiles + 1]
    int* esc_idx;
    uint8_t* esc_val;
};
// warp w of a tile takes elements [256 w, 256 w + 256) in eight rounds of 32 consecutive elements
__global__ void __launch_bounds__(256) p12_escapes(const EscArgs A) {
    __shared__ uint8_t code_of[256];
    __shared__ int wcount[8];
    code_of[threadIdx.x] = A.code_of[threadIdx.x];
    __syncthreads();
    const int base = A.tile_off[blockIdx.x];
    if (A.tile_off[blockIdx.x + 1] == base) return;  // no escape in this tile
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long w0 = (long long)blockIdx.x * TILE + warp * 256;
    unsigned masks[8];
    uint16_t vals[8];
    int mine = 0;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        const long long i = w0 + r * 32 + lane;
        vals[r] = i < A.n ? A.src[i] : (uint16_t)0;
        const bool esc = i < A.n && code_of[vals[r] >> 8] == 15;
        masks[r] = __ballot_sync(0xffffffffu, esc);
        mine += __popc(masks[r]);
    }
    if (lane == 0) wcount[warp] = mine;
    __syncthreads();
    int at = base;
    for (int w = 0; w < warp; ++w) at += wcount[w];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        if ((masks[r] >> lane) & 1u) {
            const int pos = at + __popc(masks[r] & ((1u << lane) - 1u));
            A.esc_idx[pos] = (int)(w0 + r * 32 + lane);
            A.esc_val[pos] = (uint8_t)(vals[r] >> 8);
        }
        at += __popc(masks[r]);
    }
}

// the table from the 256 counts: fifteen rounds of "the most frequent high byte not yet taken, the smallest value among
// equals"; bytes that never occur take no slot
void choose_table(const unsigned* hist, uint8_t* table16, uint8_t* code_of) {
    bool taken[256] = {false};
    for (int i = 0; i < 256; ++i) code_of[i] = 15;
    for (int i = 0; i < 16; ++i) table16[i] = 0;
    for (int slot = 0; slot < 15; ++slot) {
        int best = -1;
        for (int b = 0; b < 256; ++b)
            if (!taken[b] && hist[b] > 0u && (best < 0 || hist[b] > hist[best])) best = b;
        if (best < 0) break;
        taken[best] = true;
        table16[slot] = (uint8_t)best;
        code_of[best] = (uint8_t)slot;
    }
}

}  // namespace

extern "C" size_t btb_b200_p12_tiles(long long n) { return n > 0 ? (size_t)((n + TILE - 1) / TILE) : 0; }

extern "C" int btb_b200_p12_hist(const void* src, long long n, void* hist, void* stream) {
    if (!src || !hist) return B2_ERR_NULL;
    if (n <= 0 || n > 2147483647LL) return B2_ERR_DOMAIN;  // escape indices are int32
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(hist, 0, 256 * sizeof(unsigned), s) != cudaSuccess) {
        (void)cudaGetLastError();
        return B2_ERR_CUDA;
    }
    HistArgs a{static_cast<const uint16_t*>(src), n, static_cast<unsigned*>(hist)};
    const long long want = (n + 256 * 16 - 1) / (256 * 16);
    const int grid = (int)(want < 1 ? 1 : want > 8LL * b2_sm_count() ? 8LL * b2_sm_count() : want);
    return b2_launch((const void*)p12_hist, dim3(grid), dim3(256), 0, s, a, 0);
}

extern "C" int btb_b200_p12_table(const unsigned* hist_host, unsigned char* table16_host, int* n_codes) {
    if (!hist_host || !table16_host || !n_codes) return B2_ERR_NULL;
    uint8_t code_of[256];
    choose_table(hist_host, table16_host, code_of);
    int n = 0;
    for (int b = 0; b < 256; ++b) n += code_of[b] != 15;
    *n_codes = n;
    return B2_OK;
}

static int code_map(const unsigned char* table16, int n_codes, uint8_t* code_of) {
    if (n_codes < 0 || n_codes > 15) return B2_ERR_DOMAIN;
    for (int i = 0; i < 256; ++i) code_of[i] = 15;
    for (int c = 0; c < n_codes; ++c) code_of[table16[c]] = (uint8_t)c;
    return B2_OK;
}

extern "C" int btb_b200_p12_encode(const void* src, long long n, const unsigned char* table16_host, int n_codes, void* lo,
                                   void* hi4, void* tile_esc, void* stream) {
    if (!src || !table16_host || !lo || !hi4 || !tile_esc) return B2_ERR_NULL;
    if (n <= 0 || n > 2147483647LL) return B2_ERR_DOMAIN;
    EncArgs a;
    a.src = static_cast<const uint16_t*>(src), a.n = n;
    if (const int rc = code_map(table16_host, n_codes, a.code_of)) return rc;
    a.lo = static_cast<uint8_t*>(lo), a.hi4 = static_cast<uint8_t*>(hi4), a.tile_esc = static_cast<int*>(tile_esc);
    const int tiles = (int)btb_b200_p12_tiles(n);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (const int rc = b2_launch((const void*)p12_encode, dim3(tiles), dim3(256), 0, s, a, 0)) return rc;
    ScanArgs sa{static_cast<int*>(tile_esc), tiles};
    return b2_launch((const void*)p12_scan, dim3(1), dim3(1024), 0, s, sa, 0);
}

extern "C" int btb_b200_p12_escapes(const void* src, long long n, const unsigned char* table16_host, int n_codes,
                                    const void* tile_off, void* esc_idx, void* esc_val, void* stream) {
    if (!src || !table16_host || !tile_off || !esc_idx || !esc_val) return B2_ERR_NULL;
    if (n <= 0 || n > 2147483647LL) return B2_ERR_DOMAIN;
    EscArgs a;
    a.src = static_cast<const uint16_t*>(src), a.n = n;
    if (const int rc = code_map(table16_host, n_codes, a.code_of)) return rc;
    a.tile_off = static_cast<const int*>(tile_off);
    a.esc_idx = static_cast<int*>(esc_idx), a.esc_val = static_cast<uint8_t*>(esc_val);
    return b2_launch((const void*)p12_escapes, dim3((unsigned)btb_b200_p12_tiles(n)), dim3(256), 0,
                     static_cast<cudaStream_t>(stream), a, 0);
}
