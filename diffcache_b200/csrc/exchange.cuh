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

// What a producer kernel needs to store its results straight into every rank's copy of a channel (fan-out fused
// into the kernel that computes the values, instead of a copy kernel afterwards).  Word w of the logical block
// (row r, word c of the row) lands at word index (r / rows_per_block) * block_stride + rank_off
// + (r % rows_per_block) * row_words + c of the channel: one contiguous block per rank (rows_per_block = all
// rows, rank_off = rank * slot words) or row groups interleaved by rank.
struct XchgOut {
    unsigned char* chan[kXchgMaxWorld];   // every rank's copy of the channel
    int world;                            // 0: no fan-out (the kernel writes its ordinary outputs only)
    int channel;
    uint32_t* epoch;                      // this rank's epoch words
    uint32_t* done;                       // CTA counter of the running exchange
    int64_t rows_per_block, block_stride, rank_off, row_words;
};

// Second half of an exchange done by the producing kernel itself (sequence-sharded step): once its own block is
// stored to every rank, the kernel waits for the other ranks' blocks in channel `ll` and writes the merged result.
struct XchgFinal {
    XchgLL ll;        // this rank's copy of the channel the kernel also fans out to
    void* out;        // final (rows, head_dim) output in the element type
    float* out_lse;   // may be NULL
};

__device__ __forceinline__ int64_t xchg_word_index(const XchgOut& o, int64_t row, int64_t col_word) {
    return (row / o.rows_per_block) * o.block_stride + o.rank_off + (row % o.rows_per_block) * o.row_words + col_word;
}
// one {word, epoch} pair to every rank
__device__ __forceinline__ void xchg_put(const XchgOut& o, uint32_t epoch, int64_t word, uint32_t value) {
    for (int r = 0; r < o.world; r++) {
        uint2* dst = reinterpret_cast<uint2*>(o.chan[r]) + word;
        asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};\n" ::"l"(dst), "r"(value), "r"(epoch) : "memory");
    }
}
// two pairs (words `word` and `word + 1`, word even) to every rank with one 16-byte store each
__device__ __forceinline__ void xchg_put2(const XchgOut& o, uint32_t epoch, int64_t word, uint32_t v0, uint32_t v1) {
    for (int r = 0; r < o.world; r++) {
        uint4* dst = reinterpret_cast<uint4*>(o.chan[r]) + word / 2;
        asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"l"(dst), "r"(v0), "r"(epoch), "r"(v1), "r"(epoch) : "memory");
    }
}
// Epoch the stores of this kernel carry.  Every participating CTA reads it before it can call xchg_finish.
__device__ __forceinline__ uint32_t xchg_next_epoch(const XchgOut& o) { return o.epoch[o.channel] + 1u; }
// Called by all threads of every participating CTA after its last put: the CTA that finishes last advances
// the channel's epoch word (read by later kernels of this rank's stream).
__device__ __forceinline__ void xchg_finish(const XchgOut& o, uint32_t epoch, unsigned n_ctas) {
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(o.done, 1u) == n_ctas - 1) {
        *o.done = 0u;
        o.epoch[o.channel] = epoch;
    }
}

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
XchgOut xchg_out_args(const dc_xchg* x, int channel);   // one block per rank; callers may change the layout fields
int xchg_world(const dc_xchg* x);
int xchg_rank(const dc_xchg* x);
int64_t xchg_slot_bytes(const dc_xchg* x, int channel);
bool xchg_ready(const dc_xchg* x);

}  // namespace dc
