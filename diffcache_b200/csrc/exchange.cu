// All-gather of small per-rank blocks over NVLink peer stores, fused with the kernels that consume them.
//
// A sequence-sharded decode step exchanges two small blocks per rank (sorted ranking keys, then partial
// attention results).  Through a collective library each exchange costs a launch plus a protocol round
// trip; here every rank owns one buffer that all its peers have mapped (CUDA IPC), a producer kernel
// stores its block straight into slot `rank` of EVERY peer's buffer with plain 16-byte st.global over
// NVLink, and the consumer kernel (prefix count, partial merge) reads only its own buffer.  No K/V row,
// and no load, ever crosses NVLink; there is no multicast and no library kernel on peer memory.
//
// Arrival is signalled by the data itself: every 32-bit word is stored as an 8-byte pair {word, epoch}
// (exchange.cuh), an aligned 8-byte store is indivisible, so the consumer polls the pairs it needs until they
// carry the epoch of the current exchange.  No fence, no flag word, no extra round trip.  Epochs only grow.
// One buffer per channel suffices for the sharded step: a rank can only start the next step's exchange on a
// channel after it consumed every peer's block of the other channel of the current step, which every peer
// sent after it finished reading this channel.  (A user with ONE exchange per step alternates channels.)
//
// Every wait is bounded (wall-clock limit, default 2 s): when it runs out the kernel records status
// 401 + channel, stops waiting and finishes on zeros, so a missing peer shows up as an error status on the
// host (dc_xchg_check), never as a hung GPU.
//
// The reference has no counterpart (single process, single GPU: src/diffcache/base.py:28).
#include <cstdint>
#include <cstdlib>
#include <cstring>

#include "exchange.cuh"

namespace dc {

namespace {

constexpr int kPushThreads = 256;

__device__ __forceinline__ void st_pairs16(uint4* p, uint32_t a, uint32_t b, uint32_t epoch) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"l"(p), "r"(a), "r"(epoch), "r"(b), "r"(epoch) : "memory");
}

// grid = (n_cta); sends n_vec 16-byte source vectors (4 words each -> two 16-byte pair vectors) into every
// peer's channel, tagged with the next epoch of the channel.  The source is (rows, vec_per_row) dense; source
// vector (row, col) lands at source-vector index row * row_stride + rank_off + col of the channel: one block
// per rank (rows = 1, rank_off = rank * slot) or rows interleaved by rank (row_stride = world * vec_per_row,
// rank_off = rank * vec_per_row).  The CTA that finishes last advances the channel's epoch word, which
// later kernels of this rank's stream read.
__global__ void __launch_bounds__(kPushThreads)
xchg_push_kernel(const uint4* __restrict__ src, int64_t n_vec, int64_t vec_per_row, int64_t row_stride, int64_t rank_off,
                 XchgPeers peers, int64_t chan_off, int channel, int world, uint32_t* epoch, uint32_t* done) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t next = epoch[channel] + 1u;   // every CTA reads it before the last one can have bumped it
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
        const uint4 w = src[i];
        const int64_t at = 2 * ((i / vec_per_row) * row_stride + rank_off + (i % vec_per_row));
        for (int r = 0; r < world; r++) {
            uint4* dst = reinterpret_cast<uint4*>(peers.base[r] + chan_off) + at;
            st_pairs16(dst, w.x, w.y, next);
            st_pairs16(dst + 1, w.z, w.w, next);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(done, 1u) == gridDim.x - 1) {
        *done = 0u;
        epoch[channel] = next;
    }
}

// Waits for the blocks of all ranks in this rank's copy of a channel and writes their payload densely to dst
// (world * slot words): for consumers that are not kernels of this library.
__global__ void __launch_bounds__(256)
xchg_collect_kernel(XchgLL w, uint32_t* __restrict__ dst, int64_t n_vec_total) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t want = w.epoch[w.channel];
    const unsigned long long t0 = global_timer_ns();
    bool fail = false;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec_total; i += stride) {
        const uint2 v = xchg_poll(w.chan + i, want, w, t0, fail);
        reinterpret_cast<uint2*>(dst)[i] = v;
    }
}

}  // namespace
}  // namespace dc

using namespace dc;

struct dc_xchg {
    int rank = 0, world = 1, device = 0, n_channels = 0;
    unsigned char* local = nullptr;            // this rank's buffer: the channels, in pair format
    size_t bytes = 0;
    unsigned char* peer[kXchgMaxWorld] = {};   // base of every rank's buffer as mapped here (peer[rank] == local)
    bool opened[kXchgMaxWorld] = {};           // mapped with cudaIpcOpenMemHandle (to be closed)
    int64_t chan_off[kXchgChannels] = {};      // byte offset of each channel's data
    int64_t slot_bytes[kXchgChannels] = {};    // PAYLOAD bytes per rank in each channel (the buffer holds twice that)
    uint32_t* words = nullptr;                 // device: epoch[kXchgChannels], done counter, status
    unsigned long long timeout_ns = 2000ull * 1000 * 1000;
};

namespace {

struct XchgDeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit XchgDeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
        if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
    }
    ~XchgDeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

#define DC_XCHG_ENTER(x)                                                  \
    if ((x) == nullptr) { set_error("null exchange"); return DC_EINVAL; } \
    XchgDeviceGuard _guard((x)->device);                                  \
    if (!_guard.ok) { set_error("cannot select device %d", (x)->device); return DC_ECUDA; }

XchgPeers peers_of(const dc_xchg* x) {
    XchgPeers p;
    for (int r = 0; r < kXchgMaxWorld; r++) p.base[r] = r < x->world ? x->peer[r] : nullptr;
    return p;
}

}  // namespace

namespace dc {

XchgLL xchg_ll_args(const dc_xchg* x, int channel) {
    XchgLL w;
    w.chan = reinterpret_cast<const uint4*>(x->local + x->chan_off[channel]);
    w.slot_vecs = x->slot_bytes[channel] / 8;
    w.epoch = x->words;
    w.status = x->words + kXchgChannels + 1;
    w.channel = channel;
    w.world = x->world;
    w.timeout_ns = x->timeout_ns;
    return w;
}

XchgOut xchg_out_args(const dc_xchg* x, int channel) {
    XchgOut o;
    for (int r = 0; r < kXchgMaxWorld; r++) o.chan[r] = r < x->world ? x->peer[r] + x->chan_off[channel] : nullptr;
    o.world = x->world;
    o.channel = channel;
    o.epoch = x->words;
    o.done = x->words + kXchgChannels;
    o.rows_per_block = INT64_MAX;
    o.block_stride = 0;
    o.rank_off = static_cast<int64_t>(x->rank) * (x->slot_bytes[channel] / 4);
    o.row_words = 0;
    return o;
}

int xchg_world(const dc_xchg* x) { return x->world; }
int xchg_rank(const dc_xchg* x) { return x->rank; }
int64_t xchg_slot_bytes(const dc_xchg* x, int channel) { return x->slot_bytes[channel]; }
bool xchg_ready(const dc_xchg* x) {
    for (int r = 0; r < x->world; r++)
        if (x->peer[r] == nullptr) return false;
    return true;
}

}  // namespace dc

extern "C" {

int dc_xchg_create(int rank, int world, int device, const int64_t* slot_bytes, int n_channels, dc_xchg** out) {
    DC_REQUIRE(out != nullptr, "dc_xchg_create: null out");
    *out = nullptr;
    DC_REQUIRE(world >= 1 && world <= kXchgMaxWorld && rank >= 0 && rank < world, "dc_xchg_create: rank %d of %d (at most %d)",
               rank, world, kXchgMaxWorld);
    DC_REQUIRE(n_channels >= 1 && n_channels <= kXchgChannels && slot_bytes != nullptr,
               "dc_xchg_create: 1..%d channels", kXchgChannels);
    XchgDeviceGuard guard(device);
    if (!guard.ok) { set_error("dc_xchg_create: cannot select device %d", device); return DC_ECUDA; }
    dc_xchg* x = new dc_xchg();
    x->rank = rank; x->world = world; x->device = device; x->n_channels = n_channels;
    size_t off = 0;
    for (int c = 0; c < n_channels; c++) {
        if (slot_bytes[c] < 0 || slot_bytes[c] % 16 != 0) {
            delete x;
            set_error("dc_xchg_create: slot size %lld of channel %d is not a non-negative multiple of 16",
                      static_cast<long long>(slot_bytes[c]), c);
            return DC_EINVAL;
        }
        x->chan_off[c] = static_cast<int64_t>(off);
        x->slot_bytes[c] = slot_bytes[c];
        off += (2 * static_cast<size_t>(slot_bytes[c]) * world + 255) / 256 * 256;   // pairs: twice the payload
    }
    x->bytes = std::max<size_t>(off, 256);
    cudaError_t err = cudaMalloc(reinterpret_cast<void**>(&x->local), x->bytes);
    if (err == cudaSuccess) err = cudaMemset(x->local, 0, x->bytes);
    if (err == cudaSuccess) err = cudaMalloc(reinterpret_cast<void**>(&x->words), 256);
    if (err == cudaSuccess) err = cudaMemset(x->words, 0, 256);
    if (err == cudaSuccess) err = cudaDeviceSynchronize();
    if (err != cudaSuccess) {
        int rc = cuda_fail(err, "dc_xchg_create");
        cudaFree(x->local); cudaFree(x->words);
        delete x;
        return rc;
    }
    x->peer[rank] = x->local;
    const char* t = std::getenv("DC_XCHG_TIMEOUT_MS");
    if (t != nullptr && *t) x->timeout_ns = static_cast<unsigned long long>(std::max(1, std::atoi(t))) * 1000ull * 1000ull;
    *out = x;
    return DC_OK;
}

int dc_xchg_destroy(dc_xchg* x) {
    if (x == nullptr) return DC_OK;
    XchgDeviceGuard guard(x->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < x->world; r++)
        if (x->opened[r] && x->peer[r]) cudaIpcCloseMemHandle(x->peer[r]);
    cudaFree(x->local);
    cudaFree(x->words);
    cudaGetLastError();
    delete x;
    return DC_OK;
}

int dc_xchg_handle_bytes(void) { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }

int dc_xchg_get_handle(dc_xchg* x, void* handle_out) {
    DC_XCHG_ENTER(x);
    DC_REQUIRE(handle_out != nullptr, "dc_xchg_get_handle: null pointer");
    cudaIpcMemHandle_t h;
    DC_CUDA_TRY(cudaIpcGetMemHandle(&h, x->local));
    std::memcpy(handle_out, &h, sizeof(h));
    return DC_OK;
}

int dc_xchg_open_peer(dc_xchg* x, int peer_rank, const void* handle) {
    DC_XCHG_ENTER(x);
    DC_REQUIRE(handle != nullptr && peer_rank >= 0 && peer_rank < x->world && peer_rank != x->rank,
               "dc_xchg_open_peer: bad peer rank %d", peer_rank);
    DC_REQUIRE(x->peer[peer_rank] == nullptr, "dc_xchg_open_peer: rank %d is already mapped", peer_rank);
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    DC_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    x->peer[peer_rank] = static_cast<unsigned char*>(p);
    x->opened[peer_rank] = true;
    return DC_OK;
}

int dc_xchg_set_peer(dc_xchg* x, int peer_rank, void* base) {
    DC_XCHG_ENTER(x);
    DC_REQUIRE(base != nullptr && peer_rank >= 0 && peer_rank < x->world && peer_rank != x->rank,
               "dc_xchg_set_peer: bad peer rank %d", peer_rank);
    x->peer[peer_rank] = static_cast<unsigned char*>(base);
    x->opened[peer_rank] = false;
    return DC_OK;
}

void* dc_xchg_local(dc_xchg* x) { return x ? x->local : nullptr; }

int dc_xchg_set_timeout_ms(dc_xchg* x, int ms) {
    DC_REQUIRE(x != nullptr && ms >= 1, "dc_xchg_set_timeout_ms: bad arguments");
    x->timeout_ns = static_cast<unsigned long long>(ms) * 1000ull * 1000ull;
    return DC_OK;
}

static int xchg_push_launch(dc_xchg* x, int channel, const void* src, int64_t n_vec, int64_t vec_per_row,
                            int64_t row_stride, int64_t rank_off, uint64_t stream) {
    const int n_cta = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(32, (n_vec + kPushThreads - 1) / kPushThreads)));
    DC_CUDA_TRY(launch_chained(xchg_push_kernel, dim3(n_cta), dim3(kPushThreads), 0, as_stream(stream), 0u,
                               static_cast<const uint4*>(src), n_vec, std::max<int64_t>(1, vec_per_row), row_stride, rank_off,
                               peers_of(x), x->chan_off[channel], channel, x->world, x->words, x->words + kXchgChannels));
    return DC_OK;
}

int dc_xchg_push(dc_xchg* x, int channel, const void* src, int64_t bytes, uint64_t stream) {
    DC_XCHG_ENTER(x);
    DC_REQUIRE(channel >= 0 && channel < x->n_channels, "dc_xchg_push: channel %d", channel);
    DC_REQUIRE(src != nullptr && bytes >= 0 && bytes % 16 == 0 && bytes <= x->slot_bytes[channel] &&
                   (reinterpret_cast<uintptr_t>(src) & 15) == 0,
               "dc_xchg_push: %lld bytes do not fit the %lld-byte slot (16-byte multiples, 16-byte aligned source)",
               static_cast<long long>(bytes), static_cast<long long>(x->slot_bytes[channel]));
    DC_REQUIRE(xchg_ready(x), "dc_xchg_push: not every peer buffer is mapped yet");
    const int64_t n_vec = bytes / 16;
    return xchg_push_launch(x, channel, src, n_vec, n_vec, 0, static_cast<int64_t>(x->rank) * (x->slot_bytes[channel] / 16), stream);
}

int dc_xchg_push_rows(dc_xchg* x, int channel, const void* src, int64_t rows, int64_t row_bytes, uint64_t stream) {
    DC_XCHG_ENTER(x);
    DC_REQUIRE(channel >= 0 && channel < x->n_channels, "dc_xchg_push_rows: channel %d", channel);
    DC_REQUIRE(src != nullptr && rows >= 1 && row_bytes >= 16 && row_bytes % 16 == 0 &&
                   rows * row_bytes <= x->slot_bytes[channel] && (reinterpret_cast<uintptr_t>(src) & 15) == 0,
               "dc_xchg_push_rows: %lld rows of %lld bytes do not fit the %lld-byte slot (16-byte multiples)",
               static_cast<long long>(rows), static_cast<long long>(row_bytes), static_cast<long long>(x->slot_bytes[channel]));
    DC_REQUIRE(xchg_ready(x), "dc_xchg_push_rows: not every peer buffer is mapped yet");
    const int64_t vpr = row_bytes / 16;
    return xchg_push_launch(x, channel, src, rows * vpr, vpr, static_cast<int64_t>(x->world) * vpr,
                            static_cast<int64_t>(x->rank) * vpr, stream);
}

int dc_xchg_collect(dc_xchg* x, int channel, void* dst, int64_t bytes, uint64_t stream) {
    DC_XCHG_ENTER(x);
    DC_REQUIRE(channel >= 0 && channel < x->n_channels, "dc_xchg_collect: channel %d", channel);
    DC_REQUIRE(dst != nullptr && bytes >= 0 && bytes % 8 == 0 && bytes <= x->slot_bytes[channel] * x->world &&
                   (reinterpret_cast<uintptr_t>(dst) & 7) == 0,
               "dc_xchg_collect: %lld bytes exceed the channel's %lld (8-byte multiples, 8-byte aligned destination)",
               static_cast<long long>(bytes), static_cast<long long>(x->slot_bytes[channel] * x->world));
    const int64_t n_vec = bytes / 8;   // one 16-byte pair vector per 8 payload bytes
    const int n_cta = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(32, (n_vec + 255) / 256)));
    DC_CUDA_TRY(launch_chained(xchg_collect_kernel, dim3(n_cta), dim3(256), 0, as_stream(stream), 0u, xchg_ll_args(x, channel),
                               static_cast<uint32_t*>(dst), n_vec));
    return DC_OK;
}

int dc_xchg_check(dc_xchg* x, uint64_t stream) {
    DC_XCHG_ENTER(x);
    uint32_t st = 0;
    cudaStream_t s = as_stream(stream);
    DC_CUDA_TRY(cudaMemcpyAsync(&st, x->words + kXchgChannels + 1, sizeof(st), cudaMemcpyDeviceToHost, s));
    DC_CUDA_TRY(cudaStreamSynchronize(s));
    if (st != 0) {
        set_error("exchange: a wait for peer data ran out (status %u: channel %u); a peer is missing or late", st, st - 401u);
        cudaMemsetAsync(x->words + kXchgChannels + 1, 0, sizeof(uint32_t), s);
        return DC_EDEVICE;
    }
    return DC_OK;
}

}  // extern "C"
