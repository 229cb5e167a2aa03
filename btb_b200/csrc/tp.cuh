// The exchange between the ranks of one box (one process a GPU), as device-side pieces the kernels fold into their own
// prologues and epilogues.
//
// btb has no multi-GPU path; the contract here is that a sharded model computes the one-GPU bits. Every linear is cut by
// OUTPUT rows, so what ranks exchange is never a partial sum, only finished bf16 elements of an activation vector each
// rank owns a slice of. The hop is latency, not bytes (a few KB), so it is built the way low-latency collectives are:
// every element travels as ONE 4-byte word that carries its own arrival mark - the bf16 in the low half, a 16-bit
// sequence number of the hop in the high half. A producer stores each finished element's word straight into EVERY
// rank's copy of the vector (plain 4-byte stores to peer-mapped addresses: NVLink writes, atomic by size; no loads from
// a peer, no multicast, no fence, no separate flag). A consumer reads its LOCAL copy and takes a word when its mark is
// this hop's; until then it re-reads it - bounded: after about a second it records ERR_TIMEOUT in the status word and
// goes on, so a peer that died between steps cannot hang this GPU.
//
// The hop's sequence number is pass * per_pass + base: `pass` a device-side count of the passes of this width made so
// far (so a captured graph needs no new arguments to replay), `base` the hop's place in the pass. Successive writes to
// a word differ by one hop at least and by far less than 2^16, so a stale word never shows the awaited mark.
#pragma once

#include "common.cuh"

#define B2_MAX_RANKS 8

// what a producer needs: every rank's copy of the vector (its own included) as u32 words [M, stride]
struct B2Send {
    uint32_t* out[B2_MAX_RANKS];
    int n;       // ranks (0: no exchange, the kernel writes its ordinary local output)
    int stride;  // elements a row of the full vector holds
    int offset;  // where this rank's slice starts in a row
    const unsigned* pass;
    unsigned per_pass, base;
};
// what a consumer needs to know a word of this hop when it sees one (pass null: the input is plain bf16, no exchange)
struct B2Recv {
    const unsigned* pass;
    unsigned per_pass, base;
};

__device__ __forceinline__ uint32_t b2_hop_mark(const unsigned* pass, unsigned per_pass, unsigned base) {
    return ((__ldcg(pass) * per_pass + base) & 0xffffu) << 16;
}
__device__ __forceinline__ uint32_t b2_word(bf16 v, uint32_t mark) { return (uint32_t)__bfloat16_as_ushort(v) | mark; }

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint4 ld_volatile16(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

#define B2_XCHG_TIMEOUT_NS 1000000000ull
// four consecutive words of this rank's copy, once all four carry `mark`; returns the four bf16 as two packed pairs.
// Gives up after about a second (then every later wait of the translation unit returns at once: a broken step drains).
__device__ __forceinline__ uint2 b2_take4(const uint32_t* words, uint32_t mark) {
    uint4 w = ld_volatile16(words);
    auto ready = [&]() {
        return ((w.x ^ mark) & 0xffff0000u) == 0u && ((w.y ^ mark) & 0xffff0000u) == 0u && ((w.z ^ mark) & 0xffff0000u) == 0u &&
               ((w.w ^ mark) & 0xffff0000u) == 0u;
    };
    if (!ready() && *(volatile int*)&g_b2_status == 0) {
        const unsigned long long t0 = globaltimer_ns();
        for (;;) {
            bool ok = false;
            for (int i = 0; i < 32 && !ok; ++i) {
                w = ld_volatile16(words);
                ok = ready();
            }
            if (ok) break;
            if (globaltimer_ns() - t0 > B2_XCHG_TIMEOUT_NS || *(volatile int*)&g_b2_status != 0) {
                b2_fail(B2_ERR_TIMEOUT);
                break;
            }
        }
    }
    return make_uint2((w.x & 0xffffu) | (w.y << 16), (w.z & 0xffffu) | (w.w << 16));
}
// one element
__device__ __forceinline__ float b2_take1(const uint32_t* word, uint32_t mark) {
    uint32_t w = *reinterpret_cast<const volatile uint32_t*>(word);
    if (((w ^ mark) & 0xffff0000u) != 0u && *(volatile int*)&g_b2_status == 0) {
        const unsigned long long t0 = globaltimer_ns();
        for (;;) {
            w = *reinterpret_cast<const volatile uint32_t*>(word);
            if (((w ^ mark) & 0xffff0000u) == 0u) break;
            if (globaltimer_ns() - t0 > B2_XCHG_TIMEOUT_NS || *(volatile int*)&g_b2_status != 0) {
                b2_fail(B2_ERR_TIMEOUT);
                break;
            }
        }
    }
    return __uint_as_float(w << 16);
}
// eight consecutive elements (a 16-byte vector of bf16, as the kernels read activations)
__device__ __forceinline__ uint4 b2_take8(const uint32_t* words, uint32_t mark) {
    const uint2 a = b2_take4(words, mark), b = b2_take4(words + 4, mark);
    return make_uint4(a.x, a.y, b.x, b.y);
}
