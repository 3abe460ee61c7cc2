// LL ("low latency") packet channel: the in-kernel all-reduce / all-gather primitive.
//
// Every value that crosses NVLink travels as one 8-byte self-tagged packet
// [u32 tag | 32-bit payload] written with a single 64-bit store, so readiness rides in the data
// and no separate flag, counter or fence is needed (8-byte single-copy atomicity).  A producer
// publishes with ONE `multimem.st` to the NVSwitch multicast alias of the inbox (the switch
// replicates it into every rank's memory) or, when no multicast object exists, with one
// unicast store per peer.  Consumers poll only their own local replica.
//
// Same idea as the reference's LL-MC / LL-UC protocols
// (nex_n2_5_pro/kernels/common/m8_oproj_fused_protocol.cuh:24-136,
// nex_n2_5_pro/kernels/dflash/ll_wire.cuh:28-127) with three differences: one protocol serves
// every reduce site and every row count; the tag is a global call sequence number kept in
// device memory (`seq` + the site index of the launch), which makes consecutive uses alternate
// between the two halves of the inbox whatever mix of captured graphs runs; and every wait
// is bounded by wall-clock time on %globaltimer, after which the kernel records a sticky
// status and carries on to its exit instead of spinning.
#pragma once

#include "api.h"
#include "common.cuh"

namespace nexrt {

using LLChannel = ::NexrtLLChannel;   // plain C struct, see api.h

__device__ __forceinline__ void st_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void mc_st_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("multimem.st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

struct LLCall {
    unsigned int tag;    // never 0, so zero-initialised memory never matches
    unsigned int half;   // which half of the inbox this call uses
};

// `site` is the index of this launch among the channel users of one step (host constant).
__device__ __forceinline__ LLCall ll_begin(const LLChannel& ch, unsigned int site) {
    const unsigned int g = *reinterpret_cast<const volatile unsigned int*>(ch.seq) + site;
    LLCall c;
    c.tag = g | 0x80000000u;
    c.half = g & 1u;
    return c;
}

__device__ __forceinline__ size_t ll_offset(const LLChannel& ch, const LLCall& c, int src, unsigned int idx) {
    return (static_cast<size_t>(c.half) * ch.world + src) * ch.slots + idx;
}

// Publish one 32-bit payload into slot `idx` of every rank's inbox.
__device__ __forceinline__ void ll_publish(const LLChannel& ch, const LLCall& c, unsigned int idx, unsigned int payload) {
    const unsigned long long pkt = (static_cast<unsigned long long>(c.tag) << 32) | payload;
    const size_t off = ll_offset(ch, c, ch.rank, idx);
    if (ch.mc != nullptr) {
        mc_st_u64(ch.mc + off, pkt);
    } else {
        for (int p = 0; p < ch.world; ++p)
            if (p != ch.rank) st_sys_u64(ch.peer[p] + off, pkt);
    }
}

// Publish to one destination rank only (owner-directed traffic: CP partials, candidates).
__device__ __forceinline__ void ll_send(const LLChannel& ch, const LLCall& c, int dst, unsigned int idx, unsigned int payload) {
    const unsigned long long pkt = (static_cast<unsigned long long>(c.tag) << 32) | payload;
    st_sys_u64(ch.peer[dst] + ll_offset(ch, c, ch.rank, idx), pkt);
}

// Wait for slot `idx` from `src`.  Returns false (and latches status) when the budget runs out.
__device__ __forceinline__ bool ll_wait(const LLChannel& ch, const LLCall& c, int src, unsigned int idx,
                                        unsigned int* payload, int timeout_code = kStatusReduceTimeout) {
    const unsigned long long* p = ch.local + ll_offset(ch, c, src, idx);
    unsigned long long v = ld_sys_u64(p);
    if (static_cast<unsigned int>(v >> 32) != c.tag) {
        // a failure already latched by anyone makes every later wait give up at once
        const bool failed = *reinterpret_cast<volatile int*>(ch.status) != 0;
        const unsigned long long t0 = globaltimer_ns();
        unsigned int spins = 0;
        for (;;) {
            v = ld_sys_u64(p);
            if (static_cast<unsigned int>(v >> 32) == c.tag) break;
            if (failed || ((++spins & 63u) == 0 && globaltimer_ns() - t0 > ch.budget_ns)) {
                atomicCAS(ch.status, 0, timeout_code);
                *payload = 0;
                return false;
            }
        }
    }
    *payload = static_cast<unsigned int>(v);
    return true;
}

// All-reduce(sum) of one fp32 value per call: publish own, then add the world's values in rank
// order (own value from the register, never read back through the inbox).  Every rank adds the
// same bits in the same order, so the result is bitwise identical everywhere.
__device__ __forceinline__ float ll_allreduce_f32(const LLChannel& ch, const LLCall& c, unsigned int idx, float own) {
    if (ch.world == 1) return own;
    ll_publish(ch, c, idx, __float_as_uint(own));
    float vals[kMaxWorld];
    unsigned int pending = ((1u << ch.world) - 1u) & ~(1u << ch.rank);
    const bool failed = *reinterpret_cast<volatile int*>(ch.status) != 0;
    const unsigned long long t0 = globaltimer_ns();
    unsigned int spins = 0;
    while (pending) {
#pragma unroll
        for (int s = 0; s < kMaxWorld; ++s) {
            if (pending & (1u << s)) {
                const unsigned long long v = ld_sys_u64(ch.local + ll_offset(ch, c, s, idx));
                if (static_cast<unsigned int>(v >> 32) == c.tag) {
                    vals[s] = __uint_as_float(static_cast<unsigned int>(v));
                    pending &= ~(1u << s);
                }
            }
        }
        if (pending && (failed || ((++spins & 63u) == 0 && globaltimer_ns() - t0 > ch.budget_ns))) {
            atomicCAS(ch.status, 0, kStatusReduceTimeout);
#pragma unroll
            for (int s = 0; s < kMaxWorld; ++s)
                if (pending & (1u << s)) vals[s] = 0.f;
            pending = 0;
        }
    }
    float sum = 0.f;
#pragma unroll
    for (int s = 0; s < kMaxWorld; ++s)
        if (s < ch.world) sum += (s == ch.rank) ? own : vals[s];
    return sum;
}

}  // namespace nexrt
