// Exact top-k select on 64-bit ranking keys (dist bits << 32 | row id), smallest first.
//
// Replaces the BinaryHeap<u64> of Index::search_bruteforce (diffcache_cpu/src/nsw.rs:600-615)
// and its into_sorted_vec (nsw.rs:621).  The heap is serial and O(n log k); here one
// thread-block cluster per problem runs an adaptive-range radix select:
//   1. the live key range [lo, hi] (initially min..max of the dist bits) is split into
//      <= 4096 equal bins, every CTA of the cluster histograms its slice of the scores in
//      shared memory and the histograms are merged into the cluster leader's shared memory
//      through distributed shared memory;
//   2. the bin holding the k-th smallest key becomes the new [lo, hi]; this repeats until
//      that bin holds few enough keys to sort in shared memory (normally after ONE pass,
//      because the range is normalised to the data);
//   3. a final pass emits every key below lo, collects the threshold bin, sorts it, takes
//      what is still needed, and a bitonic sort orders the k winners.
// Row ids are part of the key, so ties on dist go to the smaller row id exactly like the
// reference (strict '<' replacement while scanning ids upwards, nsw.rs:612).
#include <cooperative_groups.h>

#include <algorithm>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace dc {

namespace {

constexpr int kSelThreads = 1024;
constexpr int kBins = 4096;
constexpr int kBinsLog2 = 12;
constexpr int kCandCap = 2048;
constexpr int kSelUnroll = 8;   // independent loads in flight per thread
constexpr int kMaxPasses = 8;  // 64 key bits / 12 bits per pass = 6 passes at most

struct SelCtl {
    unsigned long long lo, hi;
    uint32_t need;        // how many keys are still to be taken from [lo, hi]
    uint32_t t, below, cnt;
    uint32_t out_count, cand_count, dup_count;
    uint32_t mn, mx;
    uint32_t error;
};

__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t* warp_sums, uint32_t* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t inc = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        uint32_t y = __shfl_up_sync(0xFFFFFFFFu, inc, off);
        if (lane >= off) inc += y;
    }
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        uint32_t w = warp_sums[lane];
        uint32_t winc = w;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            uint32_t y = __shfl_up_sync(0xFFFFFFFFu, winc, off);
            if (lane >= off) winc += y;
        }
        warp_sums[lane] = winc - w;  // exclusive prefix of the warp totals
        if (lane == 31) *total = winc;
    }
    __syncthreads();
    return inc - v + warp_sums[warp];
}

__device__ __forceinline__ void bitonic_sort_u64(unsigned long long* a, int n) {
    for (int size = 2; size <= n; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = threadIdx.x; i < (n >> 1); i += blockDim.x) {
                int pos = 2 * i - (i & (stride - 1));
                unsigned long long x = a[pos], y = a[pos + stride];
                bool up = (pos & size) == 0;
                if ((x > y) == up) { a[pos] = y; a[pos + stride] = x; }
            }
            __syncthreads();
        }
    }
}

// grid = (cluster_size, n_prob), cluster = (cluster_size, 1, 1).
// dynamic shared memory: out[kpad] u64 | cand[kCandCap] u64 | hist[kBins] u32
__global__ void __launch_bounds__(kSelThreads, 1)
topk_select_kernel(const uint32_t* __restrict__ bits, const uint32_t* __restrict__ ids, int64_t in_stride, int64_t n,
                   int k, const uint32_t* __restrict__ minmax, uint32_t id_offset, uint32_t* __restrict__ out_bits,
                   uint32_t* __restrict__ out_ids, int64_t out_stride, int kpad, uint32_t* __restrict__ status) {
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank = cluster.block_rank();
    const unsigned csize = cluster.num_blocks();
    const int64_t prob = blockIdx.y;
    const int tid = threadIdx.x;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    unsigned long long* s_out = reinterpret_cast<unsigned long long*>(smem_raw);
    unsigned long long* s_cand = s_out + kpad;
    uint32_t* s_hist = reinterpret_cast<uint32_t*>(s_cand + kCandCap);
    __shared__ SelCtl ctl;
    __shared__ uint32_t s_warp[32];
    __shared__ uint32_t s_total;

    // the cluster leader's copies, reached through distributed shared memory
    unsigned long long* l_out = cluster.map_shared_rank(s_out, 0);
    unsigned long long* l_cand = cluster.map_shared_rank(s_cand, 0);
    uint32_t* l_hist = cluster.map_shared_rank(s_hist, 0);
    SelCtl* l_ctl = cluster.map_shared_rank(&ctl, 0);

    const uint32_t* pb = bits + prob * in_stride;
    const uint32_t* pi = ids ? ids + prob * in_stride : nullptr;

    // slice of the problem this CTA reads
    int64_t per = (n + csize - 1) / csize;
    const int64_t begin = min(n, static_cast<int64_t>(rank) * per);
    const int64_t end = min(n, begin + per);

    const int k_eff = static_cast<int>(min(static_cast<int64_t>(k), n));

    if (tid == 0) {
        ctl.out_count = 0; ctl.cand_count = 0; ctl.dup_count = 0; ctl.error = 0;
        ctl.mn = 0xFFFFFFFFu; ctl.mx = 0u;
    }
    __syncthreads();

    unsigned long long lo = 0, hi = ~0ull;
    uint32_t need = static_cast<uint32_t>(k_eff);
    const bool take_all = (k_eff == n);

    if (!take_all) {
        // ---- key range ----
        uint32_t mn, mx;
        if (minmax != nullptr) {
            mn = minmax[2 * prob];
            mx = minmax[2 * prob + 1];
        } else {
            cluster.sync();  // leader's ctl initialised
            mn = 0xFFFFFFFFu; mx = 0u;
            for (int64_t i = begin + tid; i < end; i += kSelThreads) {
                uint32_t b = pb[i];
                mn = min(mn, b); mx = max(mx, b);
            }
            mn = __reduce_min_sync(0xFFFFFFFFu, mn);
            mx = __reduce_max_sync(0xFFFFFFFFu, mx);
            if ((tid & 31) == 0) { atomicMin(&l_ctl->mn, mn); atomicMax(&l_ctl->mx, mx); }
            cluster.sync();
            mn = l_ctl->mn; mx = l_ctl->mx;
        }
        lo = static_cast<unsigned long long>(mn) << 32;
        hi = (static_cast<unsigned long long>(mx) << 32) | 0xFFFFFFFFull;

        // ---- narrowing passes ----
        for (int pass = 0; pass < kMaxPasses; pass++) {
            const unsigned long long range = hi - lo;
            const int width = range == 0 ? 0 : 64 - __clzll(static_cast<long long>(range));
            const int shift = max(0, width - kBinsLog2);

            for (int b = tid; b < kBins; b += kSelThreads) s_hist[b] = 0;
            cluster.sync();  // every histogram is clear before anyone adds to the leader's

            for (int64_t base = begin; base < end; base += kSelThreads * kSelUnroll) {
                uint32_t bb[kSelUnroll], ii[kSelUnroll];
                bool ok[kSelUnroll];
#pragma unroll
                for (int u = 0; u < kSelUnroll; u++) {  // all loads of the batch in flight together
                    int64_t i = base + u * kSelThreads + tid;
                    ok[u] = i < end;
                    bb[u] = ok[u] ? pb[i] : 0u;
                    ii[u] = ok[u] ? (pi ? pi[i] : static_cast<uint32_t>(i)) : 0u;
                }
#pragma unroll
                for (int u = 0; u < kSelUnroll; u++) {
                    unsigned long long key = (static_cast<unsigned long long>(bb[u]) << 32) | ii[u];
                    if (ok[u] && key >= lo && key <= hi) atomicAdd(&s_hist[(key - lo) >> shift], 1u);
                }
            }
            __syncthreads();
            if (rank != 0) {
                for (int b = tid; b < kBins; b += kSelThreads) {
                    uint32_t c = s_hist[b];
                    if (c) atomicAdd(&l_hist[b], c);
                }
            }
            cluster.sync();  // merged histogram complete in the leader

            if (rank == 0) {
                // each thread owns kBins / kSelThreads = 4 consecutive bins
                uint32_t h[4], s = 0;
#pragma unroll
                for (int u = 0; u < 4; u++) { h[u] = s_hist[tid * 4 + u]; s += h[u]; }
                uint32_t ex = block_exclusive_scan(s, s_warp, &s_total);
                if (ex < need && need <= ex + s) {
                    uint32_t run = ex;
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        if (run < need && need <= run + h[u]) { ctl.t = tid * 4 + u; ctl.below = run; ctl.cnt = h[u]; }
                        run += h[u];
                    }
                }
                if (tid == 0 && s_total < need) ctl.error = 1;  // cannot happen for consistent inputs
            }
            cluster.sync();  // ctl published
            const uint32_t t = l_ctl->t, below = l_ctl->below, cnt = l_ctl->cnt;
            need -= below;
            const unsigned long long nlo = lo + (static_cast<unsigned long long>(t) << shift);
            const unsigned long long span = shift == 0 ? 0ull : ((1ull << shift) - 1ull);
            const unsigned long long nhi = (nlo + span < nlo) ? hi : min(hi, nlo + span);
            lo = nlo; hi = nhi;
            if (cnt <= kCandCap || shift == 0) break;
        }
    }

    // ---- final pass: emit keys below lo, collect the threshold bin ----
    cluster.sync();  // leader's counters are initialised / nobody still reads ctl.t
    const uint32_t base_out = static_cast<uint32_t>(k_eff) - need;  // keys strictly below lo
    const bool single_value = (lo == hi);
    const unsigned lt = (1u << (tid & 31)) - 1u;
    for (int64_t base = begin; base < end; base += kSelThreads * kSelUnroll) {
        uint32_t bb[kSelUnroll], ii[kSelUnroll];
        bool ok[kSelUnroll];
#pragma unroll
        for (int u = 0; u < kSelUnroll; u++) {
            int64_t i = base + u * kSelThreads + tid;
            ok[u] = i < end;
            bb[u] = ok[u] ? pb[i] : 0u;
            ii[u] = ok[u] ? (pi ? pi[i] : static_cast<uint32_t>(i)) : 0u;
        }
#pragma unroll
        for (int u = 0; u < kSelUnroll; u++) {
            const unsigned long long key = (static_cast<unsigned long long>(bb[u]) << 32) | ii[u];
            const bool emit = ok[u] && (take_all || key < lo);
            const bool tie = ok[u] && !take_all && key >= lo && key <= hi;
            const unsigned em = __ballot_sync(0xFFFFFFFFu, emit);
            const unsigned tm = __ballot_sync(0xFFFFFFFFu, tie);
            if (em) {  // one shared-memory atomic per warp, positions by prefix popcount
                uint32_t wbase = 0;
                if ((tid & 31) == 0) wbase = atomicAdd(&l_ctl->out_count, __popc(em));
                wbase = __shfl_sync(0xFFFFFFFFu, wbase, 0);
                if (emit) {
                    uint32_t pos = wbase + __popc(em & lt);
                    if (pos < static_cast<uint32_t>(kpad)) l_out[pos] = key;
                }
            }
            if (tm) {
                uint32_t wbase = 0;
                if ((tid & 31) == 0)
                    wbase = atomicAdd(single_value ? &l_ctl->dup_count : &l_ctl->cand_count, __popc(tm));
                wbase = __shfl_sync(0xFFFFFFFFu, wbase, 0);
                if (tie) {
                    uint32_t pos = wbase + __popc(tm & lt);
                    if (single_value) {
                        if (pos < need) l_out[base_out + pos] = key;
                    } else if (pos < kCandCap) {
                        l_cand[pos] = key;
                    }
                }
            }
        }
    }
    cluster.sync();  // all remote writes into the leader have landed
    if (rank != 0) return;

    // ---- leader: resolve the threshold bin, sort, write ----
    if (!take_all && !single_value) {
        const uint32_t cc = ctl.cand_count;
        if (cc > kCandCap || cc < need) {
            if (tid == 0) ctl.error = 2;
        } else {
            int cpad = 1;
            while (cpad < static_cast<int>(cc)) cpad <<= 1;
            for (int i = cc + tid; i < cpad; i += kSelThreads) s_cand[i] = ~0ull;
            __syncthreads();
            bitonic_sort_u64(s_cand, cpad);
            for (uint32_t i = tid; i < need; i += kSelThreads) s_out[base_out + i] = s_cand[i];
        }
    }
    __syncthreads();
    if (!take_all && ctl.out_count != base_out && tid == 0) ctl.error = 3;
    for (int i = k_eff + tid; i < kpad; i += kSelThreads) s_out[i] = ~0ull;
    __syncthreads();
    bitonic_sort_u64(s_out, kpad);
    const bool bad = ctl.error != 0;
    if (bad && tid == 0 && status) atomicMax(status, 100u + ctl.error);
    for (int i = tid; i < k; i += kSelThreads) {
        const bool live = (i < k_eff && !bad);
        unsigned long long key = live ? s_out[i] : ~0ull;
        if (out_bits) out_bits[prob * out_stride + i] = static_cast<uint32_t>(key >> 32);
        if (out_ids) out_ids[prob * out_stride + i] = static_cast<uint32_t>(key & 0xFFFFFFFFull) + (live ? id_offset : 0u);
    }
}

int pow2_floor(int x) { int p = 1; while (p * 2 <= x) p *= 2; return p; }

}  // namespace

int64_t select_scratch_bytes(int n_prob) { (void)n_prob; return 256; }

// Opt in to > 48 KB of dynamic shared memory on the current device (not a stream operation;
// done once per device, outside any graph capture).
int select_prepare() {
    static bool done[64] = {};
    int dev = 0;
    DC_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && done[dev]) return DC_OK;
    DC_CUDA_TRY(cudaFuncSetAttribute(topk_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    DC_CUDA_TRY(cudaFuncSetAttribute(topk_select_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 0));
    if (dev >= 0 && dev < 64) done[dev] = true;
    return DC_OK;
}

int topk_select(const uint32_t* bits, const uint32_t* ids, int64_t in_stride, int n_prob, int64_t n, int k,
                const uint32_t* minmax, uint32_t id_offset, uint32_t* out_bits, uint32_t* out_ids, int64_t out_stride,
                uint32_t* status, cudaStream_t stream) {
    DC_REQUIRE(bits != nullptr, "topk_select: null scores");
    DC_REQUIRE(k >= 0 && k <= DC_MAX_TOPK, "topk_select: k=%d outside [0, %d]", k, DC_MAX_TOPK);
    DC_REQUIRE(n >= 0 && n < (1ll << 32), "topk_select: n=%lld outside [0, 2^32)", static_cast<long long>(n));
    DC_REQUIRE(n_prob >= 0 && n_prob <= 65535, "topk_select: n_prob=%d", n_prob);
    if (n_prob == 0 || k == 0) return DC_OK;
    int kpad = 1;
    while (kpad < k) kpad <<= 1;
    size_t smem = static_cast<size_t>(kpad) * 8 + static_cast<size_t>(kCandCap) * 8 + kBins * 4;

    // Enough CTAs per problem to occupy the SMs, at most the portable cluster size of 8,
    // and no more than one CTA per 16K keys.
    int csize = pow2_floor(std::max(1, sm_count() / std::max(1, n_prob)));
    csize = std::min(csize, 8);
    int by_work = 1;
    while (by_work < 8 && static_cast<int64_t>(by_work) * 16384 < n) by_work <<= 1;
    csize = std::min(csize, by_work);

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(csize), static_cast<unsigned>(n_prob), 1);
    cfg.blockDim = dim3(kSelThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(csize);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    DC_CUDA_TRY(cudaLaunchKernelEx(&cfg, topk_select_kernel, bits, ids, in_stride, n, k, minmax, id_offset, out_bits,
                                   out_ids, out_stride, kpad, status));
    return DC_OK;
}

}  // namespace dc
