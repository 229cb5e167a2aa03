// The standalone pieces of the exchange between ranks (tp.cuh has the device-side protocol and what it guarantees):
// peer-mapped memory for one-process-a-GPU jobs, a kernel that sends a finished slice to every rank, the merge of the
// ranks' greedy picks, a wait and a pass-count tick of their own for the places no other kernel carries them.
#include "btb_b200_internal.h"
#include "tp.cuh"
#include "../../include/btb_b200.h"

B2_DEFINE_STATUS(tp)

namespace {

int take(const btb_b200_wait* w, B2Wait& out) {
    out = B2Wait{nullptr, nullptr, 0u};
    if (w == nullptr || w->flag == nullptr) return B2_OK;
    if (w->pass == nullptr) return B2_ERR_NULL;
    out = B2Wait{static_cast<const unsigned*>(w->flag), static_cast<const unsigned*>(w->pass), w->per_pass};
    return B2_OK;
}
int take(const btb_b200_send* s, B2Send& out) {
    memset(&out, 0, sizeof out);
    if (s == nullptr) return B2_ERR_NULL;
    if (s->n < 1 || s->n > B2_MAX_RANKS || s->stride <= 0 || s->offset < 0) return B2_ERR_DOMAIN;
    out.n = s->n, out.stride = s->stride, out.offset = s->offset;
    for (int p = 0; p < s->n; ++p) {
        if (s->out[p] == nullptr || s->flag[p] == nullptr) return B2_ERR_NULL;
        out.out[p] = s->out[p], out.flag[p] = static_cast<unsigned*>(s->flag[p]);
    }
    return B2_OK;
}

// ---- a finished local slice [M, n] into every rank's copy of the full vector [M, stride] at `offset` ---------------
struct SendArgs {
    const uint4* src;  // [M, row16] sixteen-byte units
    int M, row16;      // units a row of the slice holds
    int stride16, offset16;
    B2Wait wait;
    B2Send send;
};
__global__ void __launch_bounds__(256) xchg_send(const SendArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    if (A.wait.flag != nullptr) {
        if (threadIdx.x == 0) b2_wait_arrivals(A.wait);
        __syncthreads();
    }
    const int total = A.M * A.row16;
    for (int i = blockIdx.x * 256 + threadIdx.x; i < total; i += gridDim.x * 256) {
        const int m = i / A.row16, c = i - m * A.row16;
        const uint4 v = __ldcg(A.src + i);
        const size_t at = (size_t)m * A.stride16 + A.offset16 + c;
#pragma unroll 1
        for (int p = 0; p < A.send.n; ++p) static_cast<uint4*>(A.send.out[p])[at] = v;
    }
    __syncthreads();
    b2_signal_arrival(A.send);
}

// ---- the greedy pick over a vocabulary cut by rows -------------------------------------------------------------------
// Each rank has its slice's lowest-index argmax (btb_b200_argmax_bf16). Here it packs (value, global index) into one
// 64-bit key whose unsigned order is "larger value first, lower index first among equals" - the one-GPU rule
// (btb/engine/cuda.py:2237, native/src/sample.rs:57-67) - stores the key into every rank's table, arrives, waits for the
// other ranks' keys and takes the largest: every rank computes the same token without a collective. The picks count
// their own passes (wait.pass, advanced here); `body_pass`, when given, is the pass count of the layers' exchanges,
// advanced here too as the step's last act. phase 0: all of it; 1: pack, store and arrive only; 2: wait and merge only
// (two launches where the ranks are engines of one process taking turns on one GPU).
struct PickArgs {
    const bf16* logits;      // [T, Vl] this rank's slice
    const long long* local;  // [T] its argmax within the slice
    long long* ids;          // [T] out: the global pick
    unsigned* body_pass;     // advanced by one when not null
    int T, Vl, v_offset, rank, phase;
    B2Wait wait;
    B2Send send;             // out[p]: rank p's table u64 [ranks, 32]
};
__global__ void __launch_bounds__(32) xchg_pick(const PickArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = threadIdx.x;
    if (A.phase != 2) {
        if (t < A.T) {
        const long long li = __ldcg(A.local + t);
        const unsigned short hb = __ldcg(reinterpret_cast<const unsigned short*>(A.logits) + (size_t)t * A.Vl + li);
        const uint32_t f = (uint32_t)hb << 16;
        const uint32_t ordered = (f & 0x80000000u) ? ~f : (f | 0x80000000u);
        const unsigned long long key = ((unsigned long long)ordered << 32) | (0xFFFFFFFFu - (uint32_t)(A.v_offset + li));
        for (int p = 0; p < A.send.n; ++p) static_cast<unsigned long long*>(A.send.out[p])[A.rank * 32 + t] = key;
        }
        __syncwarp();
        b2_signal_arrival(A.send);
        if (A.phase == 1) return;
    }
    bool ok = true;
    if (t == 0) ok = b2_wait_arrivals(A.wait);
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (t < A.T && ok) {
        const unsigned long long* mine = static_cast<const unsigned long long*>(A.send.out[A.rank]);
        unsigned long long best = 0ull;
        for (int p = 0; p < A.send.n; ++p) {
            const unsigned long long k = __ldcg(mine + p * 32 + t);
            best = k > best ? k : best;
        }
        A.ids[t] = (long long)(0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFull));
    }
    __syncwarp();
    if (t == 0) {
        atomicAdd(const_cast<unsigned*>(A.wait.pass), 1u);
        if (A.body_pass != nullptr) atomicAdd(A.body_pass, 1u);
    }
}

struct WaitArgs {
    B2Wait wait;
};
__global__ void __launch_bounds__(32) xchg_wait(const WaitArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) b2_wait_arrivals(A.wait);
}

struct TickArgs {
    unsigned* pass;
};
__global__ void __launch_bounds__(32) xchg_tick(const TickArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) atomicAdd(A.pass, 1u);
}

}  // namespace

// ---- peer-mapped memory (set-up time: these allocate and are not for a decode loop) ----------------------------------
extern "C" int btb_b200_peer_alloc(size_t bytes, void** ptr) {
    if (ptr == nullptr) return B2_ERR_NULL;
    if (bytes == 0) return B2_ERR_DOMAIN;
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess || cudaMemset(p, 0, bytes) != cudaSuccess) {
        (void)cudaGetLastError();
        if (p != nullptr) cudaFree(p);
        return B2_ERR_CUDA;
    }
    *ptr = p;
    return B2_OK;
}
extern "C" int btb_b200_peer_free(void* ptr) {
    if (ptr == nullptr) return B2_ERR_NULL;
    return cudaFree(ptr) == cudaSuccess ? B2_OK : B2_ERR_CUDA;
}
extern "C" int btb_b200_peer_handle(void* ptr, unsigned char* handle64) {
    if (ptr == nullptr || handle64 == nullptr) return B2_ERR_NULL;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) {
        (void)cudaGetLastError();
        return B2_ERR_CUDA;
    }
    memcpy(handle64, &h, 64);
    return B2_OK;
}
extern "C" int btb_b200_peer_open(const unsigned char* handle64, void** ptr) {
    if (handle64 == nullptr || ptr == nullptr) return B2_ERR_NULL;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess || p == nullptr) {
        (void)cudaGetLastError();
        return B2_ERR_CUDA;
    }
    *ptr = p;
    return B2_OK;
}
extern "C" int btb_b200_peer_close(void* ptr) {
    if (ptr == nullptr) return B2_ERR_NULL;
    return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? B2_OK : B2_ERR_CUDA;
}

// ---- the exchange's own launches ---------------------------------------------------------------------------------------
extern "C" int btb_b200_xchg_send(const void* src, int M, int n, int elem_bytes, const btb_b200_wait* wait,
                                  const btb_b200_send* send, int* ctas, void* stream) {
    if (src == nullptr) return B2_ERR_NULL;
    SendArgs a;
    int rc = take(wait, a.wait);
    if (rc == B2_OK) rc = take(send, a.send);
    if (rc) return rc;
    if (M <= 0 || n <= 0 || elem_bytes <= 0 || a.send.offset + n > a.send.stride) return B2_ERR_DOMAIN;
    const long long rb = (long long)n * elem_bytes, sb = (long long)a.send.stride * elem_bytes,
                    ob = (long long)a.send.offset * elem_bytes;
    if ((rb | sb | ob) & 15 || (reinterpret_cast<uintptr_t>(src) & 15)) return B2_ERR_DOMAIN;
    for (int p = 0; p < a.send.n; ++p)
        if (reinterpret_cast<uintptr_t>(a.send.out[p]) & 15) return B2_ERR_DOMAIN;
    a.src = static_cast<const uint4*>(src);
    a.M = M, a.row16 = (int)(rb / 16), a.stride16 = (int)(sb / 16), a.offset16 = (int)(ob / 16);
    const int total = a.M * a.row16;
    const int grid = total <= 512 ? 1 : (total + 511) / 512 < 8 ? (total + 511) / 512 : 8;
    if (ctas != nullptr) *ctas = grid;
    return b2_launch((const void*)xchg_send, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), a);
}

extern "C" int btb_b200_xchg_pick(const void* logits, int T, int Vl, int v_offset, const void* local_idx, int rank,
                                  const btb_b200_wait* wait, const btb_b200_send* send, void* ids, void* body_pass,
                                  int phase, void* stream) {
    if (!logits || !local_idx || !ids) return B2_ERR_NULL;
    PickArgs a;
    int rc = take(wait, a.wait);
    if (rc == B2_OK) rc = take(send, a.send);
    if (rc) return rc;
    if (T <= 0 || T > 32 || Vl <= 0 || v_offset < 0 || rank < 0 || rank >= a.send.n || a.wait.flag == nullptr ||
        phase < 0 || phase > 2)
        return B2_ERR_DOMAIN;
    a.logits = static_cast<const bf16*>(logits), a.local = static_cast<const long long*>(local_idx);
    a.ids = static_cast<long long*>(ids), a.body_pass = static_cast<unsigned*>(body_pass);
    a.T = T, a.Vl = Vl, a.v_offset = v_offset, a.rank = rank, a.phase = phase;
    return b2_launch((const void*)xchg_pick, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), a);
}

extern "C" int btb_b200_xchg_wait(const btb_b200_wait* wait, void* stream) {
    WaitArgs a;
    const int rc = take(wait, a.wait);
    if (rc) return rc;
    if (a.wait.flag == nullptr) return B2_ERR_NULL;
    return b2_launch((const void*)xchg_wait, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), a);
}

extern "C" int btb_b200_xchg_tick(void* pass, void* stream) {
    if (pass == nullptr) return B2_ERR_NULL;
    TickArgs a{static_cast<unsigned*>(pass)};
    return b2_launch((const void*)xchg_tick, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), a);
}
