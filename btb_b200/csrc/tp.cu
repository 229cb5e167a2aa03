// The standalone pieces of the exchange between ranks (tp.cuh has the device-side protocol and what it guarantees):
// peer-mapped memory for one-process-a-GPU jobs, a kernel that sends a finished slice to every rank, the merge of the
// ranks' greedy picks, a wait and a pass-count tick of their own for the places no other kernel carries them.
#include "btb_b200_internal.h"
#include "tp.cuh"
#include "../../include/btb_b200.h"

B2_DEFINE_STATUS(tp)

namespace {

int take(const btb_b200_recv* r, B2Recv& out) {
    if (r == nullptr || r->pass == nullptr) return B2_ERR_NULL;
    out = B2Recv{static_cast<const unsigned*>(r->pass), r->per_pass, r->base};
    return B2_OK;
}
int take(const btb_b200_send* s, B2Send& out) {
    memset(&out, 0, sizeof out);
    if (s == nullptr || s->pass == nullptr) return B2_ERR_NULL;
    if (s->n < 1 || s->n > B2_MAX_RANKS || s->stride <= 0 || s->offset < 0) return B2_ERR_DOMAIN;
    out.n = s->n, out.stride = s->stride, out.offset = s->offset;
    out.pass = static_cast<const unsigned*>(s->pass), out.per_pass = s->per_pass, out.base = s->base;
    for (int p = 0; p < s->n; ++p) {
        if (s->out[p] == nullptr) return B2_ERR_NULL;
        if (reinterpret_cast<uintptr_t>(s->out[p]) & 15) return B2_ERR_DOMAIN;
        out.out[p] = static_cast<uint32_t*>(s->out[p]);
    }
    return B2_OK;
}

// ---- a finished local slice [M, n] bf16 into every rank's copy of the full vector (words [M, stride]) at `offset` ----
struct SendArgs {
    const bf16* src;
    int M, n;
    B2Send send;
};
__global__ void __launch_bounds__(256) xchg_send(const SendArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t mark = b2_hop_mark(A.send.pass, A.send.per_pass, A.send.base);
    const int n4 = A.n >> 2, total = A.M * n4;  // four elements a thread a trip: one 8-byte load, one 16-byte store a rank
    for (int i = blockIdx.x * 256 + threadIdx.x; i < total; i += gridDim.x * 256) {
        const int m = i / n4, c = i - m * n4;
        const uint2 v = __ldcg(reinterpret_cast<const uint2*>(A.src + (size_t)m * A.n) + c);
        const uint4 w = make_uint4((v.x & 0xffffu) | mark, (v.x >> 16) | mark, (v.y & 0xffffu) | mark, (v.y >> 16) | mark);
        const size_t at = (size_t)m * A.send.stride + A.send.offset + (size_t)c * 4;
#pragma unroll 1
        for (int p = 0; p < A.send.n; ++p) *reinterpret_cast<uint4*>(A.send.out[p] + at) = w;
    }
}

// ---- this rank's copy of an exchanged vector (words [M, C]) as plain bf16 [M, C], once every word has arrived --------
struct UnpackArgs {
    const uint32_t* src;
    bf16* dst;
    int total8;  // M * C / 8
    B2Recv recv;
};
__global__ void __launch_bounds__(256) xchg_unpack(const UnpackArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t mark = b2_hop_mark(A.recv.pass, A.recv.per_pass, A.recv.base);
    for (int i = blockIdx.x * 256 + threadIdx.x; i < A.total8; i += gridDim.x * 256)
        reinterpret_cast<uint4*>(A.dst)[i] = b2_take8(A.src + (size_t)i * 8, mark);
}

// ---- the greedy pick over a vocabulary cut by rows -------------------------------------------------------------------
// Each rank has its slice's lowest-index argmax (btb_b200_argmax_bf16). Here it packs (value, global index) into one
// 64-bit key whose unsigned order is "larger value first, lower index first among equals" - the one-GPU rule
// (btb/engine/cuda.py:2237, native/src/sample.rs:57-67) - and stores it into every rank's table as two 8-byte words,
// each a half of the key beside the pick's sequence number (8-byte stores are atomic: a word is whole or absent). It
// then takes every rank's key from its own table as the words arrive and keeps the largest: every rank computes the
// same token without a collective. The picks count their own passes (`pick_pass`, advanced here); `body_pass`, when
// given, is the pass count of the layers' exchanges, advanced here too as the step's last act. phase 0: all of it;
// 1: pack and store only; 2: take and merge only (two launches where the ranks are engines of one process taking
// turns on one GPU).
struct PickArgs {
    const bf16* logits;      // [T, Vl] this rank's slice
    const long long* local;  // [T] its argmax within the slice
    long long* ids;          // [T] out: the global pick
    unsigned* pick_pass;     // the picks made so far at this width
    unsigned* body_pass;     // advanced by one when not null
    int T, Vl, v_offset, rank, ranks, phase;
    unsigned long long* table[B2_MAX_RANKS];  // rank p's table: u64 [ranks, 32, 2]
};
__device__ __forceinline__ unsigned long long ld_volatile8(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__global__ void __launch_bounds__(32) xchg_pick(const PickArgs A) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = threadIdx.x;
    const unsigned long long seq = (unsigned long long)(__ldcg(A.pick_pass) + 1u);
    if (A.phase != 2 && t < A.T) {
        const long long li = __ldcg(A.local + t);
        const unsigned short hb = __ldcg(reinterpret_cast<const unsigned short*>(A.logits) + (size_t)t * A.Vl + li);
        const uint32_t f = (uint32_t)hb << 16;
        const uint32_t ordered = (f & 0x80000000u) ? ~f : (f | 0x80000000u);
        const uint32_t low = 0xFFFFFFFFu - (uint32_t)(A.v_offset + li);
        for (int p = 0; p < A.ranks; ++p) {
            unsigned long long* slot = A.table[p] + ((size_t)A.rank * 32 + t) * 2;
            slot[0] = ((unsigned long long)ordered << 32) | seq;
            slot[1] = ((unsigned long long)low << 32) | seq;
        }
    }
    if (A.phase == 1) return;
    if (t < A.T) {
        unsigned long long best = 0ull;
        bool ok = true;
        for (int p = 0; p < A.ranks && ok; ++p) {
            const unsigned long long* slot = A.table[A.rank] + ((size_t)p * 32 + t) * 2;
            unsigned long long hi = ld_volatile8(slot), lo = ld_volatile8(slot + 1);
            if (((hi ^ seq) | (lo ^ seq)) & 0xFFFFFFFFull) {
                const unsigned long long t0 = globaltimer_ns();
                for (;;) {
                    hi = ld_volatile8(slot), lo = ld_volatile8(slot + 1);
                    if ((((hi ^ seq) | (lo ^ seq)) & 0xFFFFFFFFull) == 0ull) break;
                    if (globaltimer_ns() - t0 > B2_XCHG_TIMEOUT_NS || *(volatile int*)&g_b2_status != 0) {
                        b2_fail(B2_ERR_TIMEOUT);
                        ok = false;
                        break;
                    }
                }
            }
            const unsigned long long k = (hi & 0xFFFFFFFF00000000ull) | (lo >> 32);
            best = k > best ? k : best;
        }
        if (ok) A.ids[t] = (long long)(0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFull));
    }
    __syncwarp();
    if (t == 0) {
        atomicAdd(A.pick_pass, 1u);
        if (A.body_pass != nullptr) atomicAdd(A.body_pass, 1u);
    }
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
extern "C" int btb_b200_xchg_send(const void* src, int M, int n, const btb_b200_send* send, void* stream) {
    if (src == nullptr) return B2_ERR_NULL;
    SendArgs a;
    const int rc = take(send, a.send);
    if (rc) return rc;
    if (M <= 0 || n <= 0 || (n & 3) || (a.send.offset & 3) || (a.send.stride & 3) || a.send.offset + n > a.send.stride ||
        (reinterpret_cast<uintptr_t>(src) & 7))
        return B2_ERR_DOMAIN;
    a.src = static_cast<const bf16*>(src), a.M = M, a.n = n;
    const int total = M * (n >> 2);
    const int grid = total <= 256 ? 1 : (total + 255) / 256 < 16 ? (total + 255) / 256 : 16;
    return b2_launch((const void*)xchg_send, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), a);
}

extern "C" int btb_b200_xchg_unpack(const void* words, void* dst, int M, int C, const btb_b200_recv* recv, void* stream) {
    if (words == nullptr || dst == nullptr) return B2_ERR_NULL;
    UnpackArgs a;
    const int rc = take(recv, a.recv);
    if (rc) return rc;
    if (M <= 0 || C <= 0 || (C & 7) || ((reinterpret_cast<uintptr_t>(words) | reinterpret_cast<uintptr_t>(dst)) & 15))
        return B2_ERR_DOMAIN;
    a.src = static_cast<const uint32_t*>(words), a.dst = static_cast<bf16*>(dst), a.total8 = M * (C >> 3);
    const int grid = a.total8 <= 256 ? 1 : (a.total8 + 255) / 256 < 32 ? (a.total8 + 255) / 256 : 32;
    return b2_launch((const void*)xchg_unpack, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), a);
}

extern "C" int btb_b200_xchg_pick(const void* logits, int T, int Vl, int v_offset, const void* local_idx, int rank,
                                  int ranks, void* const* tables, void* ids, void* pick_pass, void* body_pass, int phase,
                                  void* stream) {
    if (!logits || !local_idx || !ids || !tables || !pick_pass) return B2_ERR_NULL;
    if (T <= 0 || T > 32 || Vl <= 0 || v_offset < 0 || ranks < 1 || ranks > B2_MAX_RANKS || rank < 0 || rank >= ranks ||
        phase < 0 || phase > 2)
        return B2_ERR_DOMAIN;
    PickArgs a;
    memset(&a, 0, sizeof a);
    for (int p = 0; p < ranks; ++p) {
        if (tables[p] == nullptr) return B2_ERR_NULL;
        if (reinterpret_cast<uintptr_t>(tables[p]) & 15) return B2_ERR_DOMAIN;
        a.table[p] = static_cast<unsigned long long*>(tables[p]);
    }
    a.logits = static_cast<const bf16*>(logits), a.local = static_cast<const long long*>(local_idx);
    a.ids = static_cast<long long*>(ids), a.pick_pass = static_cast<unsigned*>(pick_pass);
    a.body_pass = static_cast<unsigned*>(body_pass);
    a.T = T, a.Vl = Vl, a.v_offset = v_offset, a.rank = rank, a.ranks = ranks, a.phase = phase;
    return b2_launch((const void*)xchg_pick, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), a);
}

extern "C" int btb_b200_xchg_tick(void* pass, void* stream) {
    if (pass == nullptr) return B2_ERR_NULL;
    TickArgs a{static_cast<unsigned*>(pass)};
    return b2_launch((const void*)xchg_tick, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), a);
}
