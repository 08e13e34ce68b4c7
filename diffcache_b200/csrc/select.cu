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
#include <cstdlib>

#include "exchange.cuh"

namespace cg = cooperative_groups;

namespace dc {

namespace {

constexpr int kSelThreads = 1024;
constexpr int kBins = 4096;
constexpr int kBinsLog2 = 12;
constexpr int kCandCap = 2048;
constexpr int kSegMax = 512;    // longest first-pass bin the in-place segment ordering accepts
constexpr int kSelUnroll = 4;   // independent loads in flight per thread
constexpr int kMaxPasses = 8;  // 64 key bits / 12 bits per pass = 6 passes at most

// Phase marks for tuning (compiled in only with -DDC_SEL_MARKS): the leader CTA of problem 0 stores the global
// timer at phase boundaries into the words behind the status word.
#ifdef DC_SEL_MARKS
#define DC_MARK(i)                                                                                          \
    do {                                                                                                    \
        if (status != nullptr && blockIdx.y == 0 && cluster.block_rank() == 0 && threadIdx.x == 0) {        \
            unsigned long long _t;                                                                          \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(_t));                                         \
            reinterpret_cast<unsigned long long*>(status)[2 + (i)] = _t;                                    \
        }                                                                                                   \
    } while (0)
#else
#define DC_MARK(i) do {} while (0)
#endif

struct SelCtl {
    unsigned long long lo, hi;
    uint32_t need;        // how many keys are still to be taken from [lo, hi]
    uint32_t t, below, cnt;
    uint32_t out_count, cand_count, dup_count;
    uint32_t raw_count;   // CTA-local: scores kept by the single-pass path
    uint32_t mn, mx;
    uint32_t max_seg;     // largest first-pass bin below the threshold bin
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

// atomicAdd(counter, 1) for every currently active lane with ONE atomic per warp: the lanes that
// reach this point together elect a leader, which reserves popc(active) slots.
__device__ __forceinline__ uint32_t warp_aggregated_inc(uint32_t* counter) {
    const unsigned active = __activemask();
    const int lane = threadIdx.x & 31;
    const int leader = __ffs(active) - 1;
    uint32_t base = 0;
    if (lane == leader) base = atomicAdd(counter, static_cast<uint32_t>(__popc(active)));
    base = __shfl_sync(active, base, leader);
    return base + __popc(active & ((1u << lane) - 1u));
}

// Calls f(bits, position) for every score of [begin, end).  16-byte loads, kSelUnroll of them in
// flight per thread, when the slice is 16-byte aligned; scalar loads otherwise and for the tail.
template <class F>
__device__ __forceinline__ void for_each_score(const uint32_t* __restrict__ pb, int64_t begin, int64_t end, F&& f) {
    const uint32_t tid = threadIdx.x;
    const uint32_t n = static_cast<uint32_t>(end - begin);
    const uint32_t first = static_cast<uint32_t>(begin);
    const uint32_t* p = pb + begin;
    uint32_t done = 0;
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
        const uint32_t nvec = n >> 2;
        const uint4* pv = reinterpret_cast<const uint4*>(p);
        for (uint32_t v0 = 0; v0 < nvec; v0 += kSelThreads * kSelUnroll) {
            uint4 w[kSelUnroll];
#pragma unroll
            for (int u = 0; u < kSelUnroll; u++) {
                const uint32_t v = v0 + u * kSelThreads + tid;
                if (v < nvec) w[u] = pv[v];
            }
#pragma unroll
            for (int u = 0; u < kSelUnroll; u++) {
                const uint32_t v = v0 + u * kSelThreads + tid;
                if (v < nvec) {
                    const uint32_t i = first + 4 * v;
                    f(w[u].x, i); f(w[u].y, i + 1); f(w[u].z, i + 2); f(w[u].w, i + 3);
                }
            }
        }
        done = nvec << 2;
    }
    for (uint32_t i = done + tid; i < n; i += kSelThreads) f(p[i], first + i);
}

// grid = (cluster_size, n_prob), cluster = (cluster_size, 1, 1).
// dynamic shared memory: out[kpad] u64 | cand[kCandCap] u64 | hist[kBins] u32 | cum[kBins] u32 | raw[raw_cap] u64
__global__ void __launch_bounds__(kSelThreads, 1)
topk_select_kernel(const uint32_t* __restrict__ bits, const uint32_t* __restrict__ ids, int64_t in_stride, int64_t n,
                   const int32_t* __restrict__ n_dev, int k, const uint32_t* minmax, uint32_t* minmax_reset,
                   uint32_t id_offset, uint32_t* __restrict__ out_bits, uint32_t* __restrict__ out_ids,
                   int64_t out_stride, int kpad, int raw_cap, uint32_t* __restrict__ status, const XchgOut xo) {
    pdl_launch_dependents();
    pdl_wait();
    if (n_dev != nullptr) n = min(n, static_cast<int64_t>(*n_dev));  // scores valid now (n is the launch's upper bound)
    // sequence-sharded search: the sorted ranking keys also go straight into every rank's exchange buffer
    const uint32_t xepoch = xo.world ? xchg_next_epoch(xo) : 0u;
    cg::cluster_group cluster = cg::this_cluster();
    DC_MARK(0);
    const unsigned rank = cluster.block_rank();
    const unsigned csize = cluster.num_blocks();
    const int64_t prob = blockIdx.y;
    const int tid = threadIdx.x;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    unsigned long long* s_out = reinterpret_cast<unsigned long long*>(smem_raw);
    unsigned long long* s_cand = s_out + kpad;
    uint32_t* s_hist = reinterpret_cast<uint32_t*>(s_cand + kCandCap);
    uint32_t* s_cum = s_hist + kBins;  // exclusive prefix of the first-pass histogram
    unsigned long long* s_raw = reinterpret_cast<unsigned long long*>(s_cum + kBins);  // (bits, position) pairs
    __shared__ SelCtl ctl;
    __shared__ uint32_t s_warp[32];
    __shared__ uint32_t s_total;

    // the cluster leader's copies, reached through distributed shared memory
    unsigned long long* l_out = cluster.map_shared_rank(s_out, 0);
    unsigned long long* l_cand = cluster.map_shared_rank(s_cand, 0);
    uint32_t* l_hist = cluster.map_shared_rank(s_hist, 0);
    uint32_t* l_cum = cluster.map_shared_rank(s_cum, 0);
    SelCtl* l_ctl = cluster.map_shared_rank(&ctl, 0);

    const uint32_t* pb = bits + prob * in_stride;
    const uint32_t* pi = ids ? ids + prob * in_stride : nullptr;

    // slice of the problem this CTA reads (a multiple of 4 scores so that slices stay 16-byte aligned)
    int64_t per = (n + csize - 1) / csize;
    per = (per + 3) & ~static_cast<int64_t>(3);
    const int64_t begin = min(n, static_cast<int64_t>(rank) * per);
    const int64_t end = min(n, begin + per);

    const int k_eff = static_cast<int>(min(static_cast<int64_t>(k), n));

    if (tid == 0) {
        ctl.out_count = 0; ctl.cand_count = 0; ctl.dup_count = 0; ctl.raw_count = 0; ctl.error = 0;
        ctl.mn = 0xFFFFFFFFu; ctl.mx = 0u; ctl.max_seg = 0;
    }
    __syncthreads();

    unsigned long long lo = 0, hi = ~0ull;
    // first-pass binning (bits only): bin = (bits - bin_lo32) >> bin_sh; used again to place winners
    uint32_t bin_lo32 = 0;
    int bin_sh = 0, passes = 0;
    bool first_bits_only = false;
    uint32_t need = static_cast<uint32_t>(k_eff);
    const bool take_all = (k_eff == n);

    auto key_of = [&](uint32_t b, uint32_t i) -> unsigned long long {
        const uint32_t id = pi ? pi[i] : i;
        return (static_cast<unsigned long long>(b) << 32) | id;
    };

    // Leader only: locate the bin that holds the `need`-th smallest key of the merged histogram
    // (ctl.t, ctl.below, ctl.cnt).  On the first pass also keep where each bin starts in sorted order
    // (s_cum), note the largest bin wholly below the threshold (ctl.max_seg) and recycle the
    // histogram as per-bin fill counters.
    auto leader_find_threshold = [&](bool first_pass) {
        uint32_t h[4], s = 0;  // each thread owns kBins / kSelThreads = 4 consecutive bins
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
        if (first_pass) {
            uint32_t run = ex;
#pragma unroll
            for (int u = 0; u < 4; u++) { s_cum[tid * 4 + u] = run; run += h[u]; }
            __syncthreads();  // ctl.t visible
            const uint32_t tt = ctl.t;
            uint32_t mseg = 0;
#pragma unroll
            for (int u = 0; u < 4; u++) {
                if (static_cast<uint32_t>(tid * 4 + u) < tt) mseg = max(mseg, h[u]);
                s_hist[tid * 4 + u] = 0;
            }
            mseg = __reduce_max_sync(0xFFFFFFFFu, mseg);
            if ((tid & 31) == 0 && mseg) atomicMax(&ctl.max_seg, mseg);
        }
    };

    bool listed = false;  // the single-pass path kept every possible winner in s_raw: no final scan needed

    if (!take_all) {
        // ---- key range ----
        uint32_t mn, mx;
        if (minmax != nullptr) {
            mn = minmax[2 * prob];
            mx = minmax[2 * prob + 1];
        } else {
            cluster.sync();  // leader's ctl initialised
            mn = 0xFFFFFFFFu; mx = 0u;
            for_each_score(pb, begin, end, [&](uint32_t b, uint32_t) { mn = min(mn, b); mx = max(mx, b); });
            mn = __reduce_min_sync(0xFFFFFFFFu, mn);
            mx = __reduce_max_sync(0xFFFFFFFFu, mx);
            if ((tid & 31) == 0) { atomicMin(&l_ctl->mn, mn); atomicMax(&l_ctl->mx, mx); }
            cluster.sync();
            mn = l_ctl->mn; mx = l_ctl->mx;
        }
        lo = static_cast<unsigned long long>(mn) << 32;
        hi = (static_cast<unsigned long long>(mx) << 32) | 0xFFFFFFFFull;

        // ---- single-pass path (one CTA per problem) ----
        // A 1/8 sample of the scores gives a bin U that almost surely lies above the k-th smallest key.
        // One full pass then histograms only bins <= U and keeps those scores in shared memory, so the
        // exact threshold bin and all winners come out of ONE read of the score array.  If the sample
        // misleads (fewer than k keys kept, or more than fit) the general two-pass path below runs.
        if (csize == 1 && raw_cap > 0) {
            const unsigned long long range0 = hi - lo;
            const int width0 = range0 == 0 ? 0 : 64 - __clzll(static_cast<long long>(range0));
            const int shift0 = max(0, width0 - kBinsLog2);
            const uint32_t lo32 = static_cast<uint32_t>(lo >> 32);
            const uint32_t span = static_cast<uint32_t>(hi >> 32) - lo32;
            const uint32_t* p0 = pb + begin;
            const uint32_t n0 = static_cast<uint32_t>(end - begin);
            if (shift0 >= 32 && n0 >= 64u * 1024u) {
                const int sh = shift0 - 32;
                for (int b = tid; b < kBins; b += kSelThreads) s_hist[b] = 0;
                __syncthreads();
                // A caller-supplied (min, max) pair may be narrower than the data: scores outside it are left
                // out of the sample (they can only mislead it; the exact pass below decides), so that no bin
                // index ever leaves the histogram.
                auto sample_one = [&](uint32_t b) {
                    const uint32_t d = b - lo32;
                    if (d <= span) atomicAdd(&s_hist[min(d >> sh, static_cast<uint32_t>(kBins - 1))], 1u);
                };
                if ((reinterpret_cast<uintptr_t>(p0) & 15) == 0) {
                    const uint4* pv = reinterpret_cast<const uint4*>(p0);
                    for (uint32_t v = tid * 8u; v < (n0 >> 2); v += kSelThreads * 8u) {
                        const uint4 w = pv[v];
                        sample_one(w.x); sample_one(w.y); sample_one(w.z); sample_one(w.w);
                    }
                } else {
                    for (uint32_t i = tid * 8u; i < n0; i += kSelThreads * 8u) sample_one(p0[i]);
                }
                __syncthreads();
                {   // U = first bin where the sample count reaches k/8 plus four standard deviations
                    const float mean = static_cast<float>(k_eff) * 0.125f;
                    const uint32_t target = static_cast<uint32_t>(mean + 4.0f * sqrtf(mean) + 8.0f);
                    uint32_t h[4], sum = 0;
#pragma unroll
                    for (int u = 0; u < 4; u++) { h[u] = s_hist[tid * 4 + u]; sum += h[u]; }
                    const uint32_t ex = block_exclusive_scan(sum, s_warp, &s_total);
                    if (tid == 0) ctl.t = kBins - 1;
                    __syncthreads();
                    if (ex < target && target <= ex + sum) {
                        uint32_t run = ex;
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            if (run < target && target <= run + h[u]) ctl.t = tid * 4 + u;
                            run += h[u];
                        }
                    }
                    __syncthreads();
                }
                const uint32_t U = ctl.t;
                for (int b = tid; b < kBins; b += kSelThreads) s_hist[b] = 0;
                __syncthreads();
                // Survivors (bin <= U, ~1.3 k of n) go to the shared list without any atomic that returns a
                // value in the loop: a warp fills private 32-slot chunks of the list (positions by ballot and
                // popcount) and only fetches a new chunk from the shared counter when the current one is full;
                // unused slots keep the 0xFF..F sentinel the list was filled with.
                for (int r = tid; r < raw_cap; r += kSelThreads) s_raw[r] = ~0ull;
                __syncthreads();
                {
                    const uint32_t lane = tid & 31;
                    const uint32_t lt = (1u << lane) - 1u;
                    uint32_t chunk_base = 0, chunk_fill = 32;  // "full": the first survivor fetches a chunk
                    auto keep_one = [&](bool valid, uint32_t b, uint32_t i) {
                        const uint32_t d = b - lo32;
                        const uint32_t bin = d >> sh;
                        const bool keep = valid && d <= span && bin <= U;
                        const unsigned mask = __ballot_sync(0xFFFFFFFFu, keep);
                        if (mask == 0) return;
                        const uint32_t cnt = __popc(mask);
                        if (chunk_fill + cnt > 32) {  // warp-uniform
                            uint32_t nb = 0;
                            if (lane == 0) nb = atomicAdd(&ctl.raw_count, 32u);
                            chunk_base = __shfl_sync(0xFFFFFFFFu, nb, 0);
                            chunk_fill = 0;
                        }
                        if (keep) {
                            atomicAdd(&s_hist[bin], 1u);
                            const uint32_t pos = chunk_base + chunk_fill + __popc(mask & lt);
                            if (pos < static_cast<uint32_t>(raw_cap)) s_raw[pos] = (static_cast<unsigned long long>(b) << 32) | i;
                        }
                        chunk_fill += cnt;
                    };
                    const uint32_t first = static_cast<uint32_t>(begin);
                    uint32_t done = 0;
                    if ((reinterpret_cast<uintptr_t>(p0) & 15) == 0) {
                        const uint32_t nvec = n0 >> 2;
                        const uint4* pv = reinterpret_cast<const uint4*>(p0);
                        for (uint32_t v0 = 0; v0 < nvec; v0 += kSelThreads * kSelUnroll) {  // bounds are warp-uniform
                            uint4 w[kSelUnroll];
#pragma unroll
                            for (int u = 0; u < kSelUnroll; u++) {
                                const uint32_t v = v0 + u * kSelThreads + tid;
                                w[u] = v < nvec ? pv[v] : make_uint4(0, 0, 0, 0);
                            }
#pragma unroll
                            for (int u = 0; u < kSelUnroll; u++) {
                                const uint32_t v = v0 + u * kSelThreads + tid;
                                const bool valid = v < nvec;
                                const uint32_t i = first + 4 * v;
                                keep_one(valid, w[u].x, i); keep_one(valid, w[u].y, i + 1);
                                keep_one(valid, w[u].z, i + 2); keep_one(valid, w[u].w, i + 3);
                            }
                        }
                        done = nvec << 2;
                    }
                    for (uint32_t i0 = done; i0 < n0; i0 += kSelThreads) {
                        const uint32_t i = i0 + tid;
                        const bool valid = i < n0;
                        keep_one(valid, valid ? p0[i] : 0u, first + i);
                    }
                }
                __syncthreads();
                bool ok = ctl.raw_count <= static_cast<uint32_t>(raw_cap);  // list extent incl. unused slots
                if (ok) {
                    leader_find_threshold(true);  // flags ctl.error = 1 when fewer than `need` keys were kept
                    __syncthreads();
                    ok = ctl.error == 0 && ctl.cnt <= kCandCap;
                    if (ok) {
                        need -= ctl.below;
                        const unsigned long long nlo = lo + (static_cast<unsigned long long>(ctl.t) << shift0);
                        const unsigned long long sp = (1ull << shift0) - 1ull;
                        hi = (nlo + sp < nlo) ? hi : min(hi, nlo + sp);
                        lo = nlo;
                        passes = 1; first_bits_only = true; bin_lo32 = lo32; bin_sh = sh;
                        listed = true;
                    }
                }
                if (!listed) {  // start over on the general path with clean state
                    __syncthreads();
                    if (tid == 0) { ctl.raw_count = 0; ctl.max_seg = 0; ctl.error = 0; }
                    __syncthreads();
                }
            }
        }

        DC_MARK(1);
        // ---- narrowing passes ----
        for (int pass = 0; pass < kMaxPasses && !listed; pass++) {
            const unsigned long long range = hi - lo;
            const int width = range == 0 ? 0 : 64 - __clzll(static_cast<long long>(range));
            const int shift = max(0, width - kBinsLog2);

            for (int b = tid; b < kBins; b += kSelThreads) s_hist[b] = 0;
            cluster.sync();  // every histogram is clear before anyone adds to the leader's

            const uint32_t lo32 = static_cast<uint32_t>(lo >> 32), hi32 = static_cast<uint32_t>(hi >> 32);
            // Bins depend on the dist bits alone while the range still spans whole ids (always true on
            // the first pass): then this is pure 32-bit work and the ids are never read.
            const bool bits_only = (static_cast<uint32_t>(lo) == 0u) && (static_cast<uint32_t>(hi) == 0xFFFFFFFFu) &&
                                   shift >= 32;
            if (pass == 0) { first_bits_only = bits_only; bin_lo32 = lo32; bin_sh = shift - 32; }
            if (bits_only) {
                const uint32_t span = hi32 - lo32;
                const int sh = shift - 32;
                for_each_score(pb, begin, end, [&](uint32_t b, uint32_t) {
                    const uint32_t d = b - lo32;
                    if (d <= span) atomicAdd(&s_hist[d >> sh], 1u);
                });
            } else {
                for_each_score(pb, begin, end, [&](uint32_t b, uint32_t i) {
                    if (b >= lo32 && b <= hi32) {
                        const unsigned long long key = key_of(b, i);
                        if (key >= lo && key <= hi) atomicAdd(&s_hist[(key - lo) >> shift], 1u);
                    }
                });
            }
            __syncthreads();
            DC_MARK(2);
            if (rank != 0) {
                for (int b = tid; b < kBins; b += kSelThreads) {
                    uint32_t c = s_hist[b];
                    if (c) atomicAdd(&l_hist[b], c);
                }
            }
            cluster.sync();  // merged histogram complete in the leader
            DC_MARK(3);

            if (rank == 0) leader_find_threshold(pass == 0);
            cluster.sync();  // ctl published
            const uint32_t t = l_ctl->t, below = l_ctl->below, cnt = l_ctl->cnt;
            need -= below;
            const unsigned long long nlo = lo + (static_cast<unsigned long long>(t) << shift);
            const unsigned long long span = shift == 0 ? 0ull : ((1ull << shift) - 1ull);
            const unsigned long long nhi = (nlo + span < nlo) ? hi : min(hi, nlo + span);
            lo = nlo; hi = nhi;
            passes = pass + 1;
            if (cnt <= kCandCap || shift == 0) break;
        }
    }

    // ---- final pass: emit keys below lo, collect the threshold bin ----
    cluster.sync();  // leader's counters are initialised / nobody still reads ctl.t
    DC_MARK(4);
    const uint32_t base_out = static_cast<uint32_t>(k_eff) - need;  // keys strictly below lo
    const bool single_value = (lo == hi);
    // One narrowing pass on the dist bits (the normal case): every winner below the threshold bin
    // goes straight to its bin's segment of the sorted output, so only short segments remain to be
    // ordered.  Otherwise winners are appended in arrival order and sorted afterwards.
    const bool bucket = !take_all && passes == 1 && first_bits_only && l_ctl->max_seg <= kSegMax;
    if (take_all) {
        for_each_score(pb, begin, end, [&](uint32_t b, uint32_t i) {
            const uint32_t pos = warp_aggregated_inc(&l_ctl->out_count);
            if (pos < static_cast<uint32_t>(kpad)) l_out[pos] = key_of(b, i);
        });
    } else {
        // Winners are ~k of n scores, so a 32-bit pre-test on the dist bits rejects almost every
        // element before its id is looked at; positions come from one shared-memory atomic each.
        const uint32_t hi32 = static_cast<uint32_t>(hi >> 32);
        auto place_key = [&](unsigned long long key) {
            const uint32_t b = static_cast<uint32_t>(key >> 32);
            if (key < lo) {
                uint32_t pos;
                if (bucket) {
                    // (clamped: a caller-supplied key range narrower than the data must not index outside the bins)
                    const uint32_t j = min((b - bin_lo32) >> bin_sh, static_cast<uint32_t>(kBins - 1));
                    pos = l_cum[j] + atomicAdd(&l_hist[j], 1u);
                } else {
                    pos = warp_aggregated_inc(&l_ctl->out_count);
                }
                if (pos < static_cast<uint32_t>(kpad)) l_out[pos] = key;
            } else if (key <= hi) {
                if (single_value) {
                    const uint32_t pos = atomicAdd(&l_ctl->dup_count, 1u);
                    if (pos < need) l_out[base_out + pos] = key;
                } else {
                    const uint32_t pos = atomicAdd(&l_ctl->cand_count, 1u);
                    if (pos < kCandCap) l_cand[pos] = key;
                }
            }
        };
        auto place = [&](uint32_t b, uint32_t i) { place_key(key_of(b, i)); };
        bool placed = false;
        if (listed) {  // every key up to the threshold bin is already in shared memory
            const uint32_t extent = ctl.raw_count;
            for (uint32_t r = tid; r < extent; r += kSelThreads) {
                const unsigned long long e = s_raw[r];
                if (e != ~0ull) place(static_cast<uint32_t>(e >> 32), static_cast<uint32_t>(e & 0xFFFFFFFFull));
            }
            placed = true;
        } else if (csize > 1 && raw_cap > 0) {
            // Cluster: placing straight from the scan makes every thread walk a serial chain of remote
            // shared-memory round trips (one per winner it happens to hold).  Instead the CTA first gathers its
            // winners and threshold-bin keys in its OWN shared memory (local atomics), then all threads flush
            // that short list together, about one entry each, so the remote round trips overlap.
            for_each_score(pb, begin, end, [&](uint32_t b, uint32_t i) {
                if (b > hi32) return;
                const unsigned long long key = key_of(b, i);
                if (key <= hi) {
                    const uint32_t pos = atomicAdd(&ctl.raw_count, 1u);
                    if (pos < static_cast<uint32_t>(raw_cap)) s_raw[pos] = key;
                }
            });
            __syncthreads();
            DC_MARK(5);
            const uint32_t cnt = ctl.raw_count;
            if (cnt <= static_cast<uint32_t>(raw_cap)) {   // (a slice with more keys than fit is placed directly below)
                for (uint32_t r = tid; r < cnt; r += kSelThreads) place_key(s_raw[r]);
                placed = true;
            }
        }
        if (!placed) {
            for_each_score(pb, begin, end, [&](uint32_t b, uint32_t i) {
                if (b > hi32) return;
                place(b, i);
            });
        }
    }
    cluster.sync();  // all remote writes into the leader have landed
    DC_MARK(6);
    if (rank != 0) return;
    // every CTA read the key range long ago: hand the pair back in the state the next scan folds into
    if (minmax_reset != nullptr && tid == 0) { minmax_reset[2 * prob] = 0xFFFFFFFFu; minmax_reset[2 * prob + 1] = 0u; }

    // ---- leader: resolve the threshold bin, sort, write ----
    if (!take_all && !single_value) {
        const uint32_t cc = ctl.cand_count;
        if (cc > kCandCap || cc < need) {
            if (tid == 0) ctl.error = 2;
        } else {
            if (cc <= 384) {
                // few keys in the threshold bin (the usual case): the place of a key among them is the number of
                // smaller keys (keys are unique, the row id is part of them) — one pass of broadcast reads
                // instead of the ~30 barrier-separated stages of a bitonic sort
                __syncthreads();
                for (uint32_t i = tid; i < cc; i += kSelThreads) {
                    const unsigned long long key = s_cand[i];
                    uint32_t rank = 0;
                    for (uint32_t j = 0; j < cc; j++) {
                        const unsigned long long other = s_cand[j];
                        rank += (other < key || (other == key && j < i)) ? 1u : 0u;   // (identical pad entries keep their order)
                    }
                    if (rank < need) s_out[base_out + rank] = key;
                }
            } else {
                int cpad = 1;
                while (cpad < static_cast<int>(cc)) cpad <<= 1;
                for (int i = cc + tid; i < cpad; i += kSelThreads) s_cand[i] = ~0ull;
                __syncthreads();
                bitonic_sort_u64(s_cand, cpad);
                for (uint32_t i = tid; i < need; i += kSelThreads) s_out[base_out + i] = s_cand[i];
            }
        }
    }
    __syncthreads();
    DC_MARK(7);
    if (bucket) {
        // The threshold-bin winners are already ordered at [base_out, k_eff).  Order the rest: the
        // rank of a key inside its (short) segment is the number of smaller keys there, and the
        // result is written straight to its final place in global memory.
        const bool bad = ctl.error != 0;
        if (bad && tid == 0 && status) atomicMax(status, 100u + ctl.error);
        for (int p = tid; p < k; p += kSelThreads) {
            unsigned long long key = ~0ull;
            int target = p;
            if (!bad && p < k_eff) {
                key = s_out[p];
                if (static_cast<uint32_t>(p) < base_out) {
                    const uint32_t j = min((static_cast<uint32_t>(key >> 32) - bin_lo32) >> bin_sh,
                                           static_cast<uint32_t>(kBins - 1));
                    const uint32_t seg = s_cum[j];
                    const uint32_t cnt = min(s_hist[j], static_cast<uint32_t>(k_eff) - min(seg, static_cast<uint32_t>(k_eff)));
                    uint32_t rank = 0;
                    for (uint32_t i = 0; i < cnt; i++) rank += (s_out[seg + i] < key) ? 1u : 0u;
                    target = static_cast<int>(min(seg + rank, static_cast<uint32_t>(k_eff - 1)));
                }
            }
            const bool live = (!bad && p < k_eff);
            if (out_bits) out_bits[prob * out_stride + target] = static_cast<uint32_t>(key >> 32);
            if (out_ids)
                out_ids[prob * out_stride + target] = static_cast<uint32_t>(key & 0xFFFFFFFFull) + (live ? id_offset : 0u);
            if (xo.world) xchg_put(xo, xepoch, xo.rank_off + prob * out_stride + target, static_cast<uint32_t>(key >> 32));
        }
        if (xo.world) xchg_finish(xo, xepoch, gridDim.y);
        __syncthreads();
        DC_MARK(8);
        return;
    }
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
        if (xo.world) xchg_put(xo, xepoch, xo.rank_off + prob * out_stride + i, static_cast<uint32_t>(key >> 32));
    }
    if (xo.world) xchg_finish(xo, xepoch, gridDim.y);
}

int pow2_floor(int x) { int p = 1; while (p * 2 <= x) p *= 2; return p; }

// ---- merge of per-rank sorted candidate lists without moving ids ----
// Sequence-sharded search: every rank holds, per problem, its own k best ranking keys in ascending order, and
// has received the lists of all ranks ((world, n_prob, k), 0xFFFFFFFF pads).  Because each list is sorted, the
// global k best that rank r owns are a PREFIX of its list; this kernel returns the length of that prefix for
// `my_rank`.  The global rank of my i-th key b is i + sum over lower ranks of #(keys <= b) + sum over higher
// ranks of #(keys < b): rows of a lower rank have smaller global ids, so on equal dist bits they come first —
// the reference's tie rule (nsw.rs:74-91,612) restated for contiguous row shards.  Lists live in shared
// memory (world * k * 4 bytes); one CTA per problem.
constexpr int kMergeThreads = 1024;

__global__ void __launch_bounds__(kMergeThreads)
merge_sorted_count_kernel(const uint32_t* __restrict__ bits_all, int64_t rank_stride, int world, int n_prob, int k,
                          int my_rank, int32_t* __restrict__ out_count, const XchgLL ll) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) uint32_t s_lists[];
    __shared__ int s_sum[kMergeThreads / 32];
    const int p = blockIdx.x, tid = threadIdx.x;
    if (ll.chan != nullptr) {
        // lists delivered by peer stores as {key, epoch} pairs into this rank's exchange buffer: every pair is
        // polled until it carries the current epoch (k is even, so a problem's list starts on a pair vector)
        const uint32_t want = ll.epoch[ll.channel];
        const unsigned long long t0 = global_timer_ns();
        bool fail = false;
        // the loads of up to eight ranks' vectors are issued before the first is examined, so a thread pays
        // one round trip per batch; only vectors that have not arrived yet are polled one by one
        const int64_t base = (static_cast<int64_t>(p) * k) / 2;
        for (int v = tid; v < k / 2; v += kMergeThreads) {
            for (int r0 = 0; r0 < world; r0 += 8) {
                uint4 w[8];
#pragma unroll
                for (int j = 0; j < 8; j++)
                    if (r0 + j < world) w[j] = ld_volatile16(ll.chan + (r0 + j) * ll.slot_vecs + base + v);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    if (r0 + j >= world) continue;
                    uint2 d = make_uint2(w[j].x, w[j].z);
                    if (w[j].y != want || w[j].w != want)
                        d = xchg_poll(ll.chan + (r0 + j) * ll.slot_vecs + base + v, want, ll, t0, fail);
                    uint32_t* dst = s_lists + static_cast<size_t>(r0 + j) * k;
                    dst[2 * v] = d.x;
                    dst[2 * v + 1] = d.y;
                }
            }
        }
    } else
    for (int r = 0; r < world; r++) {
        const uint32_t* src = bits_all + r * rank_stride + static_cast<int64_t>(p) * k;   // rank r's (n_prob, k) lists
        uint32_t* dst = s_lists + static_cast<size_t>(r) * k;
        if ((k & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
            for (int i = tid; i < k / 4; i += kMergeThreads)
                reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
        } else {
            for (int i = tid; i < k; i += kMergeThreads) dst[i] = src[i];
        }
    }
    __syncthreads();
    const uint32_t* mine = s_lists + static_cast<size_t>(my_rank) * k;
    int winners = 0;
    for (int i = tid; i < k; i += kMergeThreads) {
        const uint32_t b = mine[i];
        if (b == 0xFFFFFFFFu) continue;  // pad: this rank holds fewer than k rows
        uint32_t rank = static_cast<uint32_t>(i);
        // stops at the first list that pushes the key out of the best k (most keys beyond the first k / world)
        for (int r = 0; r < world && rank < static_cast<uint32_t>(k); r++) {
            if (r == my_rank) continue;
            const uint32_t* list = s_lists + static_cast<size_t>(r) * k;
            // lower ranks: keys <= b; higher ranks: keys < b, i.e. keys <= b - 1 (none when b == 0)
            const uint32_t bound = r < my_rank ? b : b - 1u;
            int lo = 0, hi = (r > my_rank && b == 0u) ? 0 : k;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (list[mid] <= bound) lo = mid + 1; else hi = mid;
            }
            rank += static_cast<uint32_t>(lo);
        }
        if (rank < static_cast<uint32_t>(k)) winners++;
    }
    winners = __reduce_add_sync(0xFFFFFFFFu, winners);
    if ((tid & 31) == 0) s_sum[tid >> 5] = winners;
    __syncthreads();
    if (tid == 0) {
        int total = 0;
        for (int w = 0; w < kMergeThreads / 32; w++) total += s_sum[w];
        out_count[p] = total;
    }
}

}  // namespace

// rank_stride: elements between two ranks' (n_prob, k) lists; 0 = dense (n_prob * k).
// ll (may be NULL): the lists arrive in pair format in an exchange channel instead of bits_all.
int merge_sorted_count(const uint32_t* bits_all, int world, int n_prob, int k, int my_rank, int32_t* out_count,
                       cudaStream_t stream, const XchgLL* ll, int64_t rank_stride) {
    if (rank_stride == 0) rank_stride = static_cast<int64_t>(n_prob) * k;
    DC_REQUIRE((bits_all || ll) && out_count, "merge_sorted_count: null pointer");
    DC_REQUIRE(ll == nullptr || k % 2 == 0, "merge_sorted_count: k=%d must be even for lists delivered by the peer exchange", k);
    DC_REQUIRE(world >= 1 && my_rank >= 0 && my_rank < world, "merge_sorted_count: rank %d of %d", my_rank, world);
    DC_REQUIRE(k >= 1 && k <= DC_MAX_TOPK, "merge_sorted_count: k=%d outside [1, %d]", k, DC_MAX_TOPK);
    DC_REQUIRE(n_prob >= 0 && n_prob <= 65535, "merge_sorted_count: n_prob=%d", n_prob);
    const size_t smem = static_cast<size_t>(world) * k * sizeof(uint32_t);
    DC_REQUIRE(smem <= 200 * 1024, "merge_sorted_count: world*k=%lld keys do not fit the 200 KB of shared memory",
               static_cast<long long>(world) * k);
    if (n_prob == 0) return DC_OK;
    static PerDeviceOnce once;
    int rc0 = once.run([](int) {
        DC_CUDA_TRY(cudaFuncSetAttribute(merge_sorted_count_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        return DC_OK;
    });
    if (rc0 != DC_OK) return rc0;
    XchgLL w = {};
    if (ll != nullptr) w = *ll;
    DC_CUDA_TRY(launch_chained(merge_sorted_count_kernel, dim3(n_prob), dim3(kMergeThreads), smem, stream, 0u, bits_all,
                               rank_stride, world, n_prob, k, my_rank, out_count, w));
    return DC_OK;
}

int64_t select_scratch_bytes(int n_prob) { (void)n_prob; return 256; }

// Opt in to > 48 KB of dynamic shared memory on the current device (not a stream operation;
// done once per device, outside any graph capture).
int select_prepare() {
    static PerDeviceOnce once;
    return once.run([](int) {
        DC_CUDA_TRY(cudaFuncSetAttribute(topk_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        DC_CUDA_TRY(cudaFuncSetAttribute(topk_select_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 0));
        return DC_OK;
    });
}

// minmax_reset (may be NULL, may alias minmax): per-problem (min, max) pairs that the kernel sets back
// to (0xFFFFFFFF, 0) once it has read them, ready for the next scan's atomic min / max.
// n: scores per problem the launch is sized for; n_dev (may be NULL): device word with the number that is
// valid when the kernel runs (<= n).
// xout (may be NULL): the sorted ranking keys are also stored, in pair format, into every rank's copy of an
// exchange channel (problem p's list at word rank_off + p * out_stride).
int topk_select(const uint32_t* bits, const uint32_t* ids, int64_t in_stride, int n_prob, int64_t n, int k,
                const uint32_t* minmax, uint32_t id_offset, uint32_t* out_bits, uint32_t* out_ids, int64_t out_stride,
                uint32_t* status, cudaStream_t stream, uint32_t* minmax_reset, const int32_t* n_dev, const XchgOut* xout) {
    DC_REQUIRE(bits != nullptr, "topk_select: null scores");
    DC_REQUIRE(k >= 0 && k <= DC_MAX_TOPK, "topk_select: k=%d outside [0, %d]", k, DC_MAX_TOPK);
    DC_REQUIRE(n >= 0 && n < (1ll << 32), "topk_select: n=%lld outside [0, 2^32)", static_cast<long long>(n));
    DC_REQUIRE(n_prob >= 0 && n_prob <= 65535, "topk_select: n_prob=%d", n_prob);
    if (n_prob == 0 || k == 0) return DC_OK;
    int kpad = 1;
    while (kpad < k) kpad <<= 1;
    size_t smem = static_cast<size_t>(kpad) * 8 + static_cast<size_t>(kCandCap) * 8 + 2 * kBins * 4;
    // scores kept by the single-pass path: room for every winner, a full threshold bin and the sampling slack
    int raw_cap = 2 * kpad + kCandCap;
    if (smem + static_cast<size_t>(raw_cap) * 8 > 200 * 1024) raw_cap = 0;
    smem += static_cast<size_t>(raw_cap) * 8;

    // Enough CTAs per problem to occupy the SMs, at most the portable cluster size of 8, and no more than one
    // CTA per 8K keys (measured on 8 problems x 32 448 keys, k = 1024: 14.8 us with one CTA per 16K keys, 13.0
    // with one per 8K, 13.7 with one per 4K; a cluster of 16 CTAs was slower wherever it applied).
    static const int max_cluster = [] {   // DC_SELECT_MAX_CLUSTER: 1, 2, 4 or 8 (default) CTAs per problem at most
        const char* v = std::getenv("DC_SELECT_MAX_CLUSTER");
        const int c = (v != nullptr && *v) ? std::atoi(v) : 8;
        return c >= 8 ? 8 : c >= 4 ? 4 : c >= 2 ? 2 : 1;
    }();
    int csize = pow2_floor(std::max(1, sm_count() / std::max(1, n_prob)));
    csize = std::min(csize, max_cluster);
    int by_work = 1;
    while (by_work < 8 && static_cast<int64_t>(by_work) * 8192 < n) by_work <<= 1;
    csize = std::min(csize, by_work);

    XchgOut xo = {};
    if (xout != nullptr) xo = *xout;
    DC_CUDA_TRY(launch_chained(topk_select_kernel, dim3(static_cast<unsigned>(csize), static_cast<unsigned>(n_prob), 1),
                               dim3(kSelThreads, 1, 1), smem, stream, static_cast<unsigned>(csize), bits, ids, in_stride, n,
                               n_dev, k, minmax, minmax_reset, id_offset, out_bits, out_ids, out_stride, kpad, raw_cap,
                               status, xo));
    return DC_OK;
}

}  // namespace dc
