// Device-side pieces of the NVLink peer-store exchange (see exchange.cu) that consumer kernels in other
// translation units inline into their prologues.
#pragma once

#include "common.cuh"

struct dc_xchg;

namespace dc {

constexpr int kXchgMaxWorld = 16;
constexpr int kXchgChannels = 4;

// Wire format.  Every 32-bit payload word travels as an 8-byte pair {word, epoch}: an aligned 8-byte store is
// indivisible, so a reader that sees the epoch it expects also sees the word that came with it — the data
// carries its own "arrived" flag and needs neither a fence nor a separate flag round trip.  Two pairs are
// moved per 16-byte access.  A channel of a rank's buffer holds `world` slots of slot_words pairs each;
// slot r is written by rank r (into EVERY rank's buffer) and read only by the buffer's owner.
struct XchgPeers {
    unsigned char* base[kXchgMaxWorld];
};

// What a consumer needs to read one channel of its own buffer.
struct XchgLL {
    const uint4* chan;            // this rank's copy of the channel (nullptr: the kernel reads plain memory instead)
    int64_t slot_vecs;            // 16-byte vectors (2 pairs) per rank slot
    const uint32_t* epoch;        // this rank's epoch words: epoch[channel] = exchanges started on the channel
    uint32_t* status;             // receives 401 + channel when a wait runs out
    int channel;
    int world;
    unsigned long long timeout_ns;
};

__device__ __forceinline__ uint4 ld_volatile16(const uint4* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}

// Two payload words of vector `p` once both carry epoch `want`.  Bounded: when the time limit (or, as a second
// bound, the iteration limit) runs out, the status word is set, `fail` becomes true and zeros come back, so the
// caller finishes on harmless data and the host learns of the missing peer from the status.
__device__ __forceinline__ uint2 xchg_poll(const uint4* p, uint32_t want, const XchgLL& w, unsigned long long t0, bool& fail) {
    if (!fail) {
        for (unsigned it = 0; it < (1u << 26); it++) {
            const uint4 v = ld_volatile16(p);
            if (v.y == want && v.w == want) return make_uint2(v.x, v.z);
            if ((it & 15u) == 15u) {
                if (global_timer_ns() - t0 > w.timeout_ns) break;
                __nanosleep(20);
            }
        }
        fail = true;
        atomicMax(w.status, 401u + static_cast<uint32_t>(w.channel));
    }
    return make_uint2(0u, 0u);
}

// host-side accessors used by the engine's sharded step
XchgLL xchg_ll_args(const dc_xchg* x, int channel);
int xchg_world(const dc_xchg* x);
int xchg_rank(const dc_xchg* x);
int64_t xchg_slot_bytes(const dc_xchg* x, int channel);
bool xchg_ready(const dc_xchg* x);

}  // namespace dc
