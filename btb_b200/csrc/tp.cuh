// The exchange between the ranks of one box (one process a GPU), as device-side pieces the kernels fold into their own
// prologues and epilogues.
//
// btb has no multi-GPU path; the contract here is that a sharded model computes the one-GPU bits. Every linear is cut by
// OUTPUT rows, so what ranks exchange is never a partial sum, only finished bf16 (or f32) elements of an activation
// vector each rank owns a slice of. A producer kernel therefore writes each finished element straight into EVERY rank's
// copy of the vector (plain stores to peer-mapped addresses: NVLink writes, no loads from a peer, no multicast), and
// when a CTA has written all of its elements it makes them visible system-wide and adds one to an arrival counter in
// every rank's memory. A consumer kernel waits - bounded, reporting ERR_TIMEOUT through the status word - until the
// counter says that every CTA of every rank has arrived for this pass, and then reads its LOCAL copy only.
//
// Counters only grow: a pass's target is (pass + 1) * arrivals a pass, with `pass` a device-side count of the passes
// of this width made so far (so a captured graph needs no new arguments to replay), compared wrap-safe.
#pragma once

#include "common.cuh"

#define B2_MAX_RANKS 8

// what a producer needs: every rank's copy of the vector (its own included) and every rank's arrival counter
struct B2Send {
    void* out[B2_MAX_RANKS];
    unsigned* flag[B2_MAX_RANKS];
    int n;       // ranks (0: no exchange, the kernel writes its ordinary local output)
    int stride;  // elements a row of the full vector holds
    int offset;  // where this rank's slice starts in a row
};
// what a consumer needs: its local counter, the pass count and the arrivals a pass brings
struct B2Wait {
    const unsigned* flag;  // null: nothing to wait for
    const unsigned* pass;
    unsigned per_pass;
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_sys_add(unsigned* p, unsigned v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// One thread waits until the counter has reached this pass's target; gives up after about a second (a peer that died
// between steps must not hang this GPU) and records ERR_TIMEOUT. Once any wait of this translation unit has failed the
// later ones return at once, so a broken step drains quickly. Call from ONE thread, then barrier the CTA.
#define B2_XCHG_TIMEOUT_NS 1000000000ull
__device__ __forceinline__ bool b2_wait_arrivals(const B2Wait& w) {
    if (w.flag == nullptr) return true;
    if (*(volatile int*)&g_b2_status != 0) return false;
    const unsigned target = (ld_acquire_sys(w.pass) + 1u) * w.per_pass;
    if ((int)(ld_acquire_sys(w.flag) - target) >= 0) return true;
    const unsigned long long t0 = globaltimer_ns();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if ((int)(ld_acquire_sys(w.flag) - target) >= 0) return true;
        if (globaltimer_ns() - t0 > B2_XCHG_TIMEOUT_NS) {
            b2_fail(B2_ERR_TIMEOUT);
            return false;
        }
    }
}

// After a CTA's last element is stored (every thread past a CTA barrier): one thread a rank publishes the stores and
// adds the CTA's arrival to that rank's counter.
__device__ __forceinline__ void b2_signal_arrival(const B2Send& s) {
    if ((int)threadIdx.x < s.n) {
        __threadfence_system();
        red_release_sys_add(s.flag[threadIdx.x], 1u);
    }
}
