// Score scan: dist bits of the retrieval query against every stored key.
//
// Replaces the loop body of Index::search_bruteforce (diffcache_cpu/src/nsw.rs:601-607)
// with Index::distance QKDist (nsw.rs:129-139): one 256-byte row read + 128 MACs per key,
// done here as a pure HBM stream.  The store is read exactly once, the dot products are
// accumulated in fp32 on the CUDA cores (this is a GEMV: one query vector per key stream, so
// there is no dense contraction to hand to the tensor cores), and the only thing written back
// is one 4-byte ranking key per row (1.6 % of the bytes read).
//
// Four kernels compute the same thing (selected by the environment variable DC_SCAN_VARIANT; the fourth,
// "tcgen05" — TMA-fed tensor-core tiles with the accumulator in tensor memory — lives in scan_tc.cu):
//   "wide"   (default) 32-byte global loads, each warp-wide load covers 1 KB of consecutive rows;
//   "narrow" 16-byte global loads (512 B per warp-wide load);
//   "tma"    rows brought in by the TMA engine, one 32 KB cp.async.bulk per stage of a shared-memory
//            ring completing on mbarriers, one producer warp and eight consumer warps per persistent
//            CTA; bit-identical to "narrow".  Measured slower than the register loads (0.626 ms against
//            0.599 ms for 4.28 GB of keys), which is why it is not the default.
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace dc {

int score_scan_tc(const void* keys, int64_t prob_stride, int n_prob, int64_t n, const int32_t* n_dev, int head_dim, int dtype,
                  const void* q, int q_mode, int group, int kv_heads, int64_t q_stride_b, uint32_t* scores,
                  int64_t score_stride, uint32_t* minmax, uint32_t* status, cudaStream_t stream);

namespace {

constexpr int kScanThreads = 256;
constexpr int kScanWarps = kScanThreads / 32;
constexpr int kLoadsPerTile = 8;  // 16-byte loads in flight per lane

// grid = (chunks, n_prob); each CTA streams `rows_per_cta` consecutive rows of one problem.
template <int DT, int LPR>
__global__ void __launch_bounds__(kScanThreads)
score_scan_kernel(const uint16_t* __restrict__ keys, int64_t prob_stride, int64_t n, const int32_t* __restrict__ n_dev,
                  const uint16_t* __restrict__ q, int q_mode, int group, int kv_heads, int64_t q_stride_b,
                  uint32_t* __restrict__ scores, int64_t score_stride, uint32_t* __restrict__ minmax, int rows_per_cta) {
    pdl_launch_dependents();
    pdl_wait();
    // rows valid now (the grid was sized for an upper bound); the load is issued together with the query loads
    // below so that their latencies overlap, and only then decides whether this CTA has rows at all
    const int64_t n_now = n_dev != nullptr ? static_cast<int64_t>(*n_dev) : n;
    constexpr int D = LPR * 8;
    constexpr int R = 32 / LPR;               // rows covered by one warp-wide load
    constexpr int TR = kLoadsPerTile * R;     // rows per warp tile
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int col = lane % LPR;               // 16-byte chunk of the row this lane owns
    const int sub = lane / LPR;               // which of the R rows of a load
    const int64_t prob = blockIdx.y;

    float qv[8];
    load_query8<DT>(query_base(q, prob, D, q_mode, group, kv_heads, q_stride_b), D, q_mode, group, col * 8, qv);
    n = n_now;
    if (static_cast<int64_t>(blockIdx.x) * rows_per_cta >= n) return;

    const uint16_t* kp = keys + prob * prob_stride + col * 8;
    uint32_t* sp = scores + prob * score_stride;

    const int64_t row0 = static_cast<int64_t>(blockIdx.x) * rows_per_cta;
    const int64_t row_end = min(n, row0 + rows_per_cta);
    const int my_i = treduce_base<kLoadsPerTile, LPR>(lane);  // load index whose row this lane finishes
    const bool writer = (col & ((1 << treduce_plain_bits<kLoadsPerTile, LPR>()) - 1)) == 0;

    uint32_t lo = 0xFFFFFFFFu, hi = 0u;

    for (int64_t tile = row0 + warp * TR; tile < row_end; tile += kScanWarps * TR) {
        uint4 w[kLoadsPerTile];
        if (tile + TR <= row_end) {
#pragma unroll
            for (int i = 0; i < kLoadsPerTile; i++) w[i] = ld_stream16(kp + (tile + i * R + sub) * D);
        } else {
#pragma unroll
            for (int i = 0; i < kLoadsPerTile; i++) {
                int64_t r = min(tile + i * R + sub, row_end - 1);
                w[i] = ld_stream16(kp + r * D);
            }
        }
        float part[kLoadsPerTile];
#pragma unroll
        for (int i = 0; i < kLoadsPerTile; i++) {
            float f[8];
            unpack8<DT>(w[i], f);
            float a = f[0] * qv[0];
#pragma unroll
            for (int j = 1; j < 8; j++) a = fmaf(f[j], qv[j], a);
            part[i] = a;
        }
        treduce<kLoadsPerTile, LPR>(part, lane);
        const int64_t r = tile + my_i * R + sub;
        if (writer && r < row_end) {
            uint32_t b = dist_bits(part[0]);
            sp[r] = b;
            lo = min(lo, b);
            hi = max(hi, b);
        }
    }

    if (minmax != nullptr) {
        __shared__ uint32_t s_lo, s_hi;
        if (threadIdx.x == 0) { s_lo = 0xFFFFFFFFu; s_hi = 0u; }
        __syncthreads();
        lo = __reduce_min_sync(0xFFFFFFFFu, lo);
        hi = __reduce_max_sync(0xFFFFFFFFu, hi);
        if (lane == 0) { atomicMin(&s_lo, lo); atomicMax(&s_hi, hi); }
        __syncthreads();
        if (threadIdx.x == 0 && s_lo <= s_hi) {
            atomicMin(&minmax[2 * prob], s_lo);
            atomicMax(&minmax[2 * prob + 1], s_hi);
        }
    }
}


// Same scan with 32-byte loads: LW = D/16 lanes share a row (16 elements per lane), one warp-wide
// load covers 32/LW consecutive rows = 1 KB.  Half the load instructions per byte.
template <int DT, int LW>
__global__ void __launch_bounds__(kScanThreads)
score_scan_wide_kernel(const uint16_t* __restrict__ keys, int64_t prob_stride, int64_t n,
                       const int32_t* __restrict__ n_dev, const uint16_t* __restrict__ q, int q_mode, int group,
                       int kv_heads, int64_t q_stride_b, uint32_t* __restrict__ scores, int64_t score_stride,
                       uint32_t* __restrict__ minmax, int rows_per_cta) {
    pdl_launch_dependents();
    pdl_wait();
    // rows valid now (the grid was sized for an upper bound); the load is issued together with the query loads
    // below so that their latencies overlap, and only then decides whether this CTA has rows at all
    const int64_t n_now = n_dev != nullptr ? static_cast<int64_t>(*n_dev) : n;
    constexpr int D = LW * 16;
    constexpr int R = 32 / LW;
    constexpr int TR = kLoadsPerTile * R;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int col = lane % LW;
    const int sub = lane / LW;
    const int64_t prob = blockIdx.y;

    float qv[16];
    {
        float a[8], b[8];
        const uint16_t* qb = query_base(q, prob, D, q_mode, group, kv_heads, q_stride_b);
        load_query8<DT>(qb, D, q_mode, group, col * 16, a);
        load_query8<DT>(qb, D, q_mode, group, col * 16 + 8, b);
#pragma unroll
        for (int j = 0; j < 8; j++) { qv[j] = a[j]; qv[8 + j] = b[j]; }
    }
    n = n_now;
    if (static_cast<int64_t>(blockIdx.x) * rows_per_cta >= n) return;
    const uint16_t* kp = keys + prob * prob_stride + col * 16;
    uint32_t* sp = scores + prob * score_stride;
    const int64_t row0 = static_cast<int64_t>(blockIdx.x) * rows_per_cta;
    const int64_t row_end = min(n, row0 + rows_per_cta);
    const int my_i = treduce_base<kLoadsPerTile, LW>(lane);
    const bool writer = (col & ((1 << treduce_plain_bits<kLoadsPerTile, LW>()) - 1)) == 0;
    uint32_t lo = 0xFFFFFFFFu, hi = 0u;

    for (int64_t tile = row0 + warp * TR; tile < row_end; tile += kScanWarps * TR) {
        Wide32 w[kLoadsPerTile];
        if (tile + TR <= row_end) {
#pragma unroll
            for (int i = 0; i < kLoadsPerTile; i++) w[i] = ld_stream32(kp + (tile + i * R + sub) * D);
        } else {
#pragma unroll
            for (int i = 0; i < kLoadsPerTile; i++) w[i] = ld_stream32(kp + min(tile + i * R + sub, row_end - 1) * D);
        }
        float part[kLoadsPerTile];
#pragma unroll
        for (int i = 0; i < kLoadsPerTile; i++) {
            float f[8], g[8];
            unpack8<DT>(w[i].lo, f);
            unpack8<DT>(w[i].hi, g);
            float a = f[0] * qv[0];
#pragma unroll
            for (int j = 1; j < 8; j++) a = fmaf(f[j], qv[j], a);
#pragma unroll
            for (int j = 0; j < 8; j++) a = fmaf(g[j], qv[8 + j], a);
            part[i] = a;
        }
        treduce<kLoadsPerTile, LW>(part, lane);
        constexpr int CNT = treduce_count<kLoadsPerTile, LW>();
#pragma unroll
        for (int c = 0; c < CNT; c++) {
            const int64_t r = tile + (my_i + c) * R + sub;
            if (writer && r < row_end) {
                uint32_t b = dist_bits(part[c]);
                sp[r] = b;
                lo = min(lo, b);
                hi = max(hi, b);
            }
        }
    }
    if (minmax != nullptr) {
        __shared__ uint32_t s_lo, s_hi;
        if (threadIdx.x == 0) { s_lo = 0xFFFFFFFFu; s_hi = 0u; }
        __syncthreads();
        lo = __reduce_min_sync(0xFFFFFFFFu, lo);
        hi = __reduce_max_sync(0xFFFFFFFFu, hi);
        if (lane == 0) { atomicMin(&s_lo, lo); atomicMax(&s_hi, hi); }
        __syncthreads();
        if (threadIdx.x == 0 && s_lo <= s_hi) {
            atomicMin(&minmax[2 * prob], s_lo);
            atomicMax(&minmax[2 * prob + 1], s_hi);
        }
    }
}

// ---- the same scan fed by the TMA engine ----
constexpr int kTmaConsWarps = 8;
constexpr int kTmaThreads = (kTmaConsWarps + 1) * 32;
constexpr int kTmaStages = 4;
constexpr int kTmaStageBytes = 32 * 1024;

__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.shared::cta.b64 st, [%0];\n}\n" ::"r"(smem_u32(bar)) : "memory");
}

// Persistent CTAs; work unit u = one stage (32 KB of consecutive rows of one problem), unit u goes to
// CTA u % gridDim.x so that the CTAs of the grid read one contiguous window of the store at a time.
// Warp kTmaConsWarps is the producer: one lane waits for a free stage and issues ONE bulk copy for it.
// The consumer warps each own 1/8 of the stage's rows (exactly one warp tile), pull them into registers,
// release the stage, and then do the arithmetic of score_scan_kernel.  Every mbarrier wait is bounded;
// a wait that runs out stores 201 (producer) or 202 (consumer) in *status and the thread leaves.
template <int DT, int LPR>
__global__ void __launch_bounds__(kTmaThreads, 1)
score_scan_tma_kernel(const uint16_t* __restrict__ keys, int64_t prob_stride, int64_t n,
                      const int32_t* __restrict__ n_dev, int n_prob, const uint16_t* __restrict__ q, int q_mode,
                      int group, int kv_heads, int64_t q_stride_b, uint32_t* __restrict__ scores, int64_t score_stride,
                      uint32_t* __restrict__ minmax, uint32_t* __restrict__ status, int q_table) {
    pdl_launch_dependents();
    pdl_wait();
    if (n_dev != nullptr) n = *n_dev;
    constexpr int D = LPR * 8;
    constexpr int R = 32 / LPR;
    constexpr int TR = kLoadsPerTile * R;
    constexpr int STAGE_ROWS = kTmaStageBytes / (D * 2);
    static_assert(STAGE_ROWS == kTmaConsWarps * TR, "a stage is one warp tile per consumer warp");
    extern __shared__ __align__(128) unsigned char tma_ring[];
    __shared__ unsigned long long full[kTmaStages], empty[kTmaStages];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t units_per_prob = (n + STAGE_ROWS - 1) / STAGE_ROWS;
    const int64_t total = units_per_prob * n_prob;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kTmaStages; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], kTmaConsWarps); }
        mbar_init_fence();
    }
    // A CTA meets every problem (a few stages of each), so the retrieval queries of all problems are formed
    // once into shared memory behind the ring (q_table != 0: they fit) instead of at every change of problem.
    uint16_t* s_q = reinterpret_cast<uint16_t*>(tma_ring + static_cast<size_t>(kTmaStages) * kTmaStageBytes);
    if (q_table) {
        for (int i = threadIdx.x; i < n_prob * LPR; i += kTmaThreads) {
            float f[8];
            load_query8<DT>(query_base(q, i / LPR, D, q_mode, group, kv_heads, q_stride_b), D, q_mode, group,
                            (i % LPR) * 8, f);
            uint4 w;
            w.x = float_to_elem<DT>(f[0]) | (static_cast<uint32_t>(float_to_elem<DT>(f[1])) << 16);
            w.y = float_to_elem<DT>(f[2]) | (static_cast<uint32_t>(float_to_elem<DT>(f[3])) << 16);
            w.z = float_to_elem<DT>(f[4]) | (static_cast<uint32_t>(float_to_elem<DT>(f[5])) << 16);
            w.w = float_to_elem<DT>(f[6]) | (static_cast<uint32_t>(float_to_elem<DT>(f[7])) << 16);
            *reinterpret_cast<uint4*>(s_q + static_cast<size_t>(i) * 8) = w;
        }
    }
    // ... and its (min, max) pairs are gathered in shared memory and folded into global memory once, at the
    // end: all CTAs change problem at about the same time, and 8 warps x all CTAs firing atomics at the same
    // two words at once was measured to cost more than 100 us per scan.
    uint32_t* s_mm = reinterpret_cast<uint32_t*>(s_q + static_cast<size_t>(n_prob) * LPR * 8);
    if (q_table)
        for (int i = threadIdx.x; i < n_prob; i += kTmaThreads) { s_mm[2 * i] = 0xFFFFFFFFu; s_mm[2 * i + 1] = 0u; }
    __syncthreads();
    if (warp == kTmaConsWarps) {
        if (lane == 0) {
            int64_t it = 0;
            for (int64_t u = blockIdx.x; u < total; u += gridDim.x, it++) {
                const int s = static_cast<int>(it % kTmaStages);
                if (it >= kTmaStages && !mbar_wait_bounded(&empty[s], static_cast<unsigned>((it / kTmaStages - 1) & 1))) {
                    if (status) atomicMax(status, 201u);
                    break;
                }
                const int64_t p = u / units_per_prob, r0 = (u % units_per_prob) * STAGE_ROWS;
                const unsigned bytes = static_cast<unsigned>(min(static_cast<int64_t>(STAGE_ROWS), n - r0)) * D * 2;
                mbar_arrive_expect_tx(&full[s], bytes);
                bulk_copy_g2s(tma_ring + static_cast<size_t>(s) * kTmaStageBytes, keys + p * prob_stride + r0 * D, bytes,
                              &full[s]);
            }
        }
        return;
    }
    const int col = lane % LPR, sub = lane / LPR;
    const int my_i = treduce_base<kLoadsPerTile, LPR>(lane);
    const bool writer = (col & ((1 << treduce_plain_bits<kLoadsPerTile, LPR>()) - 1)) == 0;
    uint32_t lo = 0xFFFFFFFFu, hi = 0u;
    int64_t cur_p = -1;
    auto flush_minmax = [&]() {  // warp-uniform
        lo = __reduce_min_sync(0xFFFFFFFFu, lo);
        hi = __reduce_max_sync(0xFFFFFFFFu, hi);
        if (minmax != nullptr && lane == 0 && lo <= hi) {
            uint32_t* mm = q_table ? s_mm : minmax;
            atomicMin(&mm[2 * cur_p], lo);
            atomicMax(&mm[2 * cur_p + 1], hi);
        }
        lo = 0xFFFFFFFFu; hi = 0u;
    };
    float qv[8];
    int64_t it = 0;
    for (int64_t u = blockIdx.x; u < total; u += gridDim.x, it++) {
        const int s = static_cast<int>(it % kTmaStages);
        const int64_t p = u / units_per_prob, r0 = (u % units_per_prob) * STAGE_ROWS;
        if (p != cur_p) {
            if (cur_p >= 0) flush_minmax();
            cur_p = p;
            if (q_table) unpack8<DT>(*reinterpret_cast<const uint4*>(s_q + (p * LPR + col) * 8), qv);
            else load_query8<DT>(query_base(q, p, D, q_mode, group, kv_heads, q_stride_b), D, q_mode, group, col * 8, qv);
        }
        // warp-uniform outcome: either every lane saw the stage arrive or the whole warp gives up
        if (!__all_sync(0xFFFFFFFFu, mbar_wait_bounded(&full[s], static_cast<unsigned>((it / kTmaStages) & 1)))) {
            if (status && lane == 0) atomicMax(status, 202u);
            break;
        }
        const int rows = static_cast<int>(min(static_cast<int64_t>(STAGE_ROWS), n - r0));
        const unsigned char* st = tma_ring + static_cast<size_t>(s) * kTmaStageBytes;
        uint4 w[kLoadsPerTile];
#pragma unroll
        for (int i = 0; i < kLoadsPerTile; i++) {
            const int r = warp * TR + i * R + sub;
            w[i] = *reinterpret_cast<const uint4*>(st + (static_cast<size_t>(r) * D + col * 8) * 2);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);  // the rows are in registers: the producer may refill the stage
        float part[kLoadsPerTile];
#pragma unroll
        for (int i = 0; i < kLoadsPerTile; i++) {
            float f[8];
            unpack8<DT>(w[i], f);
            float a = f[0] * qv[0];
#pragma unroll
            for (int j = 1; j < 8; j++) a = fmaf(f[j], qv[j], a);
            part[i] = a;
        }
        treduce<kLoadsPerTile, LPR>(part, lane);
        const int r = warp * TR + my_i * R + sub;
        if (writer && r < rows) {   // rows past the end of the problem hold stale bytes of an earlier stage
            const uint32_t b = dist_bits(part[0]);
            scores[p * score_stride + r0 + r] = b;
            lo = min(lo, b);
            hi = max(hi, b);
        }
    }
    if (cur_p >= 0) flush_minmax();
    if (q_table && minmax != nullptr) {
        // the consumer warps only (the producer warp has left): named barrier 1, kTmaConsWarps * 32 threads
        asm volatile("bar.sync 1, %0;\n" ::"n"(kTmaConsWarps * 32) : "memory");
        for (int i = threadIdx.x; i < n_prob; i += kTmaConsWarps * 32) {
            if (s_mm[2 * i] <= s_mm[2 * i + 1]) {
                atomicMin(&minmax[2 * i], s_mm[2 * i]);
                atomicMax(&minmax[2 * i + 1], s_mm[2 * i + 1]);
            }
        }
    }
}

int env_int(const char* name, int dflt) {
    const char* s = std::getenv(name);
    if (s == nullptr || *s == 0) return dflt;
    return std::atoi(s);
}

// Rows per CTA of the register kernels.  1024 (256 KB of keys) for launches of many waves; a launch of only a few
// waves (a shard of a long sequence, one kv head of a layer) takes the chunk size that fills whole waves of the
// two CTAs an SM holds, so that no partial wave trails: 8 problems x 131 072 rows run as exactly two waves of
// 1792-row CTAs (43.1 us) instead of 3.46 waves of 1024-row ones (44.3 us).
int auto_rows_per_cta(int64_t n, int n_prob, int unit) {
    const int64_t slots = 2ll * sm_count();
    auto cost = [&](int64_t rows) {   // waves x (rows + what the set-up of a CTA costs, in rows)
        const int64_t ctas = ((n + rows - 1) / rows) * n_prob;
        return ((ctas + slots - 1) / slots) * (rows + 128);
    };
    if (((n + 1023) / 1024) * n_prob >= 8 * slots) return 1024;
    int best = 1024;
    int64_t best_cost = cost(1024);
    for (int rows = unit; rows <= 2048; rows += unit) {
        if (rows < 512) continue;
        const int64_t c = cost(rows);
        if (c < best_cost) { best = rows; best_cost = c; }
    }
    return best;
}

template <int DT, int LPR>
int launch_scan(const void* keys, int64_t prob_stride, int n_prob, int64_t n, const int32_t* n_dev, const void* q,
                int q_mode, int group, int kv_heads, int64_t q_stride_b, uint32_t* scores, int64_t score_stride,
                uint32_t* minmax, uint32_t* status, cudaStream_t stream) {
    constexpr int TR = kLoadsPerTile * (32 / LPR);
    static const int rows_env = env_int("DC_SCAN_ROWS_PER_CTA", 0);   // 0: chosen per launch
    // twice the 16-byte kernel's granule, so that the 32-byte kernel (twice the rows per load) divides it too
    const int rows_cfg = rows_env > 0 ? rows_env : auto_rows_per_cta(n, n_prob, 2 * kScanWarps * TR);
    int rows_per_cta = ((rows_cfg + kScanWarps * TR - 1) / (kScanWarps * TR)) * (kScanWarps * TR);
    int64_t chunks = (n + rows_per_cta - 1) / rows_per_cta;
    dim3 grid(static_cast<unsigned>(chunks), static_cast<unsigned>(n_prob));
    const char* variant = std::getenv("DC_SCAN_VARIANT");  // read per call: "wide" (default), "narrow", "tma", "tcgen05"
    if (variant != nullptr && std::strcmp(variant, "tcgen05") == 0) {
        const int rc = score_scan_tc(keys, prob_stride, n_prob, n, n_dev, LPR * 8, DT, q, q_mode, group, kv_heads, q_stride_b,
                                     scores, score_stride, minmax, status, stream);
        if (rc != DC_ESTATE) return rc;   // DC_ESTATE: not applicable to this shape, use the default kernel
    }
    const bool want_tma = variant != nullptr && std::strcmp(variant, "tma") == 0;
    const bool want_narrow = variant != nullptr && std::strcmp(variant, "narrow") == 0;
    if (want_tma) {
        constexpr int kRing = kTmaStages * kTmaStageBytes;
        constexpr int kQTableMax = 64 * 1024;   // ring + table stay below the 227 KB a CTA may use
        static PerDeviceOnce once;
        int rc0 = once.run([](int) {
            DC_CUDA_TRY(cudaFuncSetAttribute(score_scan_tma_kernel<DT, LPR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kRing + kQTableMax));
            return DC_OK;
        });
        if (rc0 != DC_OK) return rc0;
        const size_t table_bytes = static_cast<size_t>(n_prob) * (LPR * 16 + 8);   // queries + (min, max) pairs
        const int q_table = table_bytes <= static_cast<size_t>(kQTableMax) ? 1 : 0;
        DC_CUDA_TRY(launch_chained(score_scan_tma_kernel<DT, LPR>, dim3(sm_count()), dim3(kTmaThreads),
                                   kRing + (q_table ? table_bytes : 0), stream, 0u, static_cast<const uint16_t*>(keys),
                                   prob_stride, n, n_dev, n_prob, static_cast<const uint16_t*>(q), q_mode, group, kv_heads,
                                   q_stride_b, scores, score_stride, minmax, status, q_table));
        return DC_OK;
    }
    if (!want_narrow && LPR >= 8 && prob_stride % 16 == 0 && (reinterpret_cast<uintptr_t>(keys) & 31) == 0) {
        // rows_per_cta is a multiple of 8 warps x 8 loads x (32 / (LPR/2)) rows as well (LPR >= 8)
        DC_CUDA_TRY(launch_chained(score_scan_wide_kernel<DT, LPR / 2>, grid, dim3(kScanThreads), 0, stream, 0u,
                                   static_cast<const uint16_t*>(keys), prob_stride, n, n_dev,
                                   static_cast<const uint16_t*>(q), q_mode, group, kv_heads, q_stride_b, scores,
                                   score_stride, minmax, rows_per_cta));
        return DC_OK;
    }
    DC_CUDA_TRY(launch_chained(score_scan_kernel<DT, LPR>, grid, dim3(kScanThreads), 0, stream, 0u,
                               static_cast<const uint16_t*>(keys), prob_stride, n, n_dev, static_cast<const uint16_t*>(q),
                               q_mode, group, kv_heads, q_stride_b, scores, score_stride, minmax, rows_per_cta));
    return DC_OK;
}

}  // namespace

// n: rows per problem the launch is sized for; n_dev (may be NULL): device word holding the number of rows
// that are valid when the kernel runs (<= n), for launches replayed from a graph while the store grows.
int score_scan(const void* keys, int64_t prob_stride, int n_prob, int64_t n, int head_dim, int dtype, const void* q,
               int q_mode, int group, uint32_t* scores, int64_t score_stride, uint32_t* minmax, cudaStream_t stream,
               uint32_t* status, int kv_heads, int64_t q_stride_b, const int32_t* n_dev) {
    DC_REQUIRE(keys && q && scores, "score_scan: null pointer");
    DC_REQUIRE(dtype == DC_BF16 || dtype == DC_FP16, "score_scan: dtype %d not supported", dtype);
    DC_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256, "score_scan: head_dim %d not in {64,128,256}",
               head_dim);
    DC_REQUIRE(n_prob >= 0 && n_prob <= 65535 && n >= 0, "score_scan: bad sizes n_prob=%d n=%lld", n_prob,
               static_cast<long long>(n));
    DC_REQUIRE(q_mode == 0 || (q_mode == 1 && group >= 1), "score_scan: bad q_mode/group");
    DC_REQUIRE(q_stride_b == 0 || (q_mode == 1 && kv_heads >= 1 && n_prob % kv_heads == 0 && q_stride_b % 8 == 0),
               "score_scan: a batch stride needs q_mode 1, kv_heads dividing n_prob and a multiple of 8 elements");
    if (kv_heads < 1) kv_heads = 1;
    DC_REQUIRE(prob_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(keys) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(q) & 15) == 0,
               "score_scan: keys/q must be 16-byte aligned and prob_stride a multiple of 8 elements");
    if (n_prob == 0 || n == 0) return DC_OK;
#define DC_SCAN_CASE(DT, LPR) \
    return launch_scan<DT, LPR>(keys, prob_stride, n_prob, n, n_dev, q, q_mode, group, kv_heads, q_stride_b, scores, \
                                score_stride, minmax, status, stream)
    if (dtype == DC_BF16) {
        if (head_dim == 64) DC_SCAN_CASE(DC_BF16, 8);
        if (head_dim == 128) DC_SCAN_CASE(DC_BF16, 16);
        DC_SCAN_CASE(DC_BF16, 32);
    } else {
        if (head_dim == 64) DC_SCAN_CASE(DC_FP16, 8);
        if (head_dim == 128) DC_SCAN_CASE(DC_FP16, 16);
        DC_SCAN_CASE(DC_FP16, 32);
    }
#undef DC_SCAN_CASE
}

}  // namespace dc
