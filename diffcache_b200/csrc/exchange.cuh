// Device-side pieces of the NVLink peer-store exchange (see exchange.cu) that consumer kernels in other
// translation units inline into their prologues.
#pragma once

#include "common.cuh"

struct dc_xchg;

namespace dc {

constexpr int kXchgMaxWorld = 16;
constexpr int kXchgChannels = 4;
constexpr int kXchgFlagStride = 128;   // bytes between two flag words (one cache line each)
constexpr size_t kXchgFlagBytes = static_cast<size_t>(kXchgChannels) * kXchgMaxWorld * kXchgFlagStride;

// Buffer of a rank: [flags: kXchgChannels x kXchgMaxWorld words, 128 bytes apart | channel 0 | channel 1 | ...];
// channel c holds `world` slots of slot_bytes[c]; flag (c, r) = epoch of the last block of rank r that has
// completely arrived in slot r of channel c of THIS buffer.
struct XchgPeers {
    unsigned char* base[kXchgMaxWorld];
};

__host__ __device__ __forceinline__ uint32_t* xchg_flag(unsigned char* base, int channel, int rank) {
    return reinterpret_cast<uint32_t*>(base + (static_cast<size_t>(channel) * kXchgMaxWorld + rank) * kXchgFlagStride);
}

struct XchgWait {
    const uint32_t* flags;        // this rank's buffer (its flag region comes first); nullptr = nothing to wait for
    const uint32_t* epoch;        // this rank's epoch words: epoch[channel] = exchanges started on the channel
    uint32_t* status;             // receives 401 + channel when the wait runs out
    int channel;
    int world;
    unsigned long long timeout_ns;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}

// Block-wide: returns when every rank's block of the current epoch has arrived in this rank's buffer, or
// when the time limit (and, as a second bound, an iteration limit) runs out, in which case the status word
// is set and the caller goes on with whatever the buffer holds.  Call from all threads of the block, after
// pdl_wait(); blockDim.x >= world.
__device__ __forceinline__ void xchg_wait_all(const XchgWait& w) {
    if (w.flags != nullptr) {
        if (static_cast<int>(threadIdx.x) < w.world) {
            const uint32_t want = w.epoch[w.channel];
            const uint32_t* f = w.flags + (static_cast<size_t>(w.channel) * kXchgMaxWorld + threadIdx.x) * (kXchgFlagStride / 4);
            const unsigned long long t0 = global_timer_ns();
            bool ok = false;
            for (unsigned it = 0; it < (1u << 27); it++) {
                if (static_cast<int32_t>(ld_acquire_sys(f) - want) >= 0) { ok = true; break; }
                if (global_timer_ns() - t0 > w.timeout_ns) break;
                __nanosleep(40);
            }
            if (!ok) atomicMax(w.status, 401u + static_cast<uint32_t>(w.channel));
        }
        __syncthreads();
    }
}

// host-side accessors used by the engine's sharded step
XchgWait xchg_wait_args(const dc_xchg* x, int channel);
const unsigned char* xchg_channel_data(const dc_xchg* x, int channel);
int xchg_world(const dc_xchg* x);
int xchg_rank(const dc_xchg* x);
int64_t xchg_slot_bytes(const dc_xchg* x, int channel);
bool xchg_ready(const dc_xchg* x);

}  // namespace dc
