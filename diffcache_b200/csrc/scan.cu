// Score scan: dist bits of the retrieval query against every stored key.
//
// Replaces the loop body of Index::search_bruteforce (diffcache_cpu/src/nsw.rs:601-607)
// with Index::distance QKDist (nsw.rs:129-139): one 256-byte row read + 128 MACs per key,
// done here as a pure HBM stream.  The store is read exactly once with 16-byte loads that
// are contiguous across the warp (each load instruction covers 512 contiguous bytes), the
// dot products are accumulated in fp32 on the CUDA cores (this is a GEMV: one query vector
// per key stream, so there is no dense contraction to hand to the tensor cores), and the
// only thing written back is one 4-byte ranking key per row (1.6 % of the bytes read).
#include <cstdlib>

#include "common.cuh"

namespace dc {

namespace {

constexpr int kScanThreads = 256;
constexpr int kScanWarps = kScanThreads / 32;
constexpr int kLoadsPerTile = 8;  // 16-byte loads in flight per lane

// grid = (chunks, n_prob); each CTA streams `rows_per_cta` consecutive rows of one problem.
template <int DT, int LPR>
__global__ void __launch_bounds__(kScanThreads)
score_scan_kernel(const uint16_t* __restrict__ keys, int64_t prob_stride, int64_t n, const uint16_t* __restrict__ q,
                  int q_mode, int group, uint32_t* __restrict__ scores, int64_t score_stride,
                  uint32_t* __restrict__ minmax, int rows_per_cta) {
    constexpr int D = LPR * 8;
    constexpr int R = 32 / LPR;               // rows covered by one warp-wide load
    constexpr int TR = kLoadsPerTile * R;     // rows per warp tile
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int col = lane % LPR;               // 16-byte chunk of the row this lane owns
    const int sub = lane / LPR;               // which of the R rows of a load
    const int64_t prob = blockIdx.y;

    float qv[8];
    load_query8<DT>(q, prob, D, q_mode, group, col * 8, qv);

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
score_scan_wide_kernel(const uint16_t* __restrict__ keys, int64_t prob_stride, int64_t n, const uint16_t* __restrict__ q,
                       int q_mode, int group, uint32_t* __restrict__ scores, int64_t score_stride,
                       uint32_t* __restrict__ minmax, int rows_per_cta) {
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
        load_query8<DT>(q, prob, D, q_mode, group, col * 16, a);
        load_query8<DT>(q, prob, D, q_mode, group, col * 16 + 8, b);
#pragma unroll
        for (int j = 0; j < 8; j++) { qv[j] = a[j]; qv[8 + j] = b[j]; }
    }
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

int env_int(const char* name, int dflt) {
    const char* s = std::getenv(name);
    if (s == nullptr || *s == 0) return dflt;
    return std::atoi(s);
}

template <int DT, int LPR>
int launch_scan(const void* keys, int64_t prob_stride, int n_prob, int64_t n, const void* q, int q_mode, int group,
                uint32_t* scores, int64_t score_stride, uint32_t* minmax, cudaStream_t stream) {
    constexpr int TR = kLoadsPerTile * (32 / LPR);
    static int rows_cfg = env_int("DC_SCAN_ROWS_PER_CTA", 1024);
    int rows_per_cta = ((rows_cfg + kScanWarps * TR - 1) / (kScanWarps * TR)) * (kScanWarps * TR);
    int64_t chunks = (n + rows_per_cta - 1) / rows_per_cta;
    dim3 grid(static_cast<unsigned>(chunks), static_cast<unsigned>(n_prob));
    static int wide = env_int("DC_SCAN_WIDE", 1);
    if (wide && LPR >= 8 && prob_stride % 16 == 0 && (reinterpret_cast<uintptr_t>(keys) & 31) == 0) {
        // rows_per_cta is a multiple of 8 warps x 8 loads x (32 / (LPR/2)) rows as well (LPR >= 8)
        score_scan_wide_kernel<DT, LPR / 2><<<grid, kScanThreads, 0, stream>>>(
            static_cast<const uint16_t*>(keys), prob_stride, n, static_cast<const uint16_t*>(q), q_mode, group, scores,
            score_stride, minmax, rows_per_cta);
        DC_CUDA_TRY(cudaGetLastError());
        return DC_OK;
    }
    score_scan_kernel<DT, LPR><<<grid, kScanThreads, 0, stream>>>(
        static_cast<const uint16_t*>(keys), prob_stride, n, static_cast<const uint16_t*>(q), q_mode, group, scores,
        score_stride, minmax, rows_per_cta);
    DC_CUDA_TRY(cudaGetLastError());
    return DC_OK;
}

}  // namespace

int score_scan(const void* keys, int64_t prob_stride, int n_prob, int64_t n, int head_dim, int dtype, const void* q,
               int q_mode, int group, uint32_t* scores, int64_t score_stride, uint32_t* minmax, cudaStream_t stream) {
    DC_REQUIRE(keys && q && scores, "score_scan: null pointer");
    DC_REQUIRE(dtype == DC_BF16 || dtype == DC_FP16, "score_scan: dtype %d not supported", dtype);
    DC_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256, "score_scan: head_dim %d not in {64,128,256}",
               head_dim);
    DC_REQUIRE(n_prob >= 0 && n_prob <= 65535 && n >= 0, "score_scan: bad sizes n_prob=%d n=%lld", n_prob,
               static_cast<long long>(n));
    DC_REQUIRE(q_mode == 0 || (q_mode == 1 && group >= 1), "score_scan: bad q_mode/group");
    DC_REQUIRE(prob_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(keys) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(q) & 15) == 0,
               "score_scan: keys/q must be 16-byte aligned and prob_stride a multiple of 8 elements");
    if (n_prob == 0 || n == 0) return DC_OK;
#define DC_SCAN_CASE(DT, LPR) \
    return launch_scan<DT, LPR>(keys, prob_stride, n_prob, n, q, q_mode, group, scores, score_stride, minmax, stream)
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
