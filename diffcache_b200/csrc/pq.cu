// Product-quantisation baseline: asymmetric-distance (ADC) lookup-table scorer and exact
// rerank.  The reference ships no PQ code (evaluation/impl/pqcache is an empty directory);
// the definition implemented here is the one stated in include/diffcache_b200.h.
#include "common.cuh"

namespace dc {

namespace {

// lut[p][m][c] = <q_p[m*ds .. (m+1)*ds), centroid[p][m][c][:]>; one thread per table entry,
// dims accumulated in order with fp32 FMAs.
template <int DT>
__global__ void pq_build_lut_kernel(const uint16_t* __restrict__ q, int q_mode, int group,
                                    const float* __restrict__ centroids, int dim, int n_sub,
                                    float* __restrict__ lut) {
    const int64_t prob = blockIdx.y;
    const int m = blockIdx.x;
    const int c = threadIdx.x;  // 256 threads
    const int ds = dim / n_sub;
    extern __shared__ float s_q[];  // ds floats
    if (c < ds) {
        const int d = m * ds + c;
        float v;
        if (q_mode == 0) {
            v = elem_to_float<DT>(q[prob * dim + d]);
        } else {
            float s = 0.0f;
            for (int g = 0; g < group; g++) s += elem_to_float<DT>(q[(prob * group + g) * dim + d]);
            v = elem_to_float<DT>(float_to_elem<DT>(s * (1.0f / static_cast<float>(group))));
        }
        s_q[c] = v;
    }
    __syncthreads();
    const float* cen = centroids + ((prob * n_sub + m) * 256 + c) * ds;
    float s = 0.0f;
    for (int d = 0; d < ds; d++) s = fmaf(s_q[d], cen[d], s);
    lut[(prob * n_sub + m) * 256 + c] = s;
}

constexpr int kAdcThreads = 256;

// ADC scan: 16 one-byte codes per row (one 16-byte load per row per thread), 16 table
// lookups from shared memory, summed in subspace order.  grid = (chunks, n_prob).
template <int M>
__global__ void __launch_bounds__(kAdcThreads)
pq_adc_scan_kernel(const uint8_t* __restrict__ codes, int64_t prob_stride, int64_t n, const float* __restrict__ lut,
                   uint32_t* __restrict__ scores, int64_t score_stride, uint32_t* __restrict__ minmax,
                   int rows_per_cta) {
    __shared__ float s_lut[M * 256];
    const int64_t prob = blockIdx.y;
    for (int i = threadIdx.x; i < M * 256; i += kAdcThreads) s_lut[i] = lut[prob * M * 256 + i];
    __syncthreads();
    const uint8_t* cp = codes + prob * prob_stride;
    uint32_t* sp = scores + prob * score_stride;
    const int64_t row0 = static_cast<int64_t>(blockIdx.x) * rows_per_cta;
    const int64_t row_end = min(n, row0 + rows_per_cta);
    uint32_t lo = 0xFFFFFFFFu, hi = 0u;
    int64_t r_first = row0 + threadIdx.x;
    if (M == 16) {
        // Four rows per thread and iteration: four 16-byte loads in flight, and the 64 table lookups of the four
        // rows interleave, so the shared-memory latency of one row's chain is hidden by the others.  Each row is
        // still summed in subspace order.
        constexpr int U = 4;
        for (; r_first + (U - 1) * kAdcThreads < row_end; r_first += U * kAdcThreads) {
            uint4 w[U];
#pragma unroll
            for (int u = 0; u < U; u++) w[u] = ld_stream16(cp + (r_first + u * kAdcThreads) * M);
            float acc[U];
#pragma unroll
            for (int u = 0; u < U; u++) acc[u] = 0.0f;
#pragma unroll
            for (int j = 0; j < 16; j++) {
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const uint32_t word = j < 4 ? w[u].x : j < 8 ? w[u].y : j < 12 ? w[u].z : w[u].w;
                    acc[u] += s_lut[j * 256 + ((word >> (8 * (j % 4))) & 0xFFu)];
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const uint32_t b = dist_bits(acc[u]);
                sp[r_first + u * kAdcThreads] = b;
                lo = min(lo, b);
                hi = max(hi, b);
            }
        }
    }
    for (int64_t r = r_first; r < row_end; r += kAdcThreads) {
        float s = 0.0f;
        if (M % 16 == 0) {
#pragma unroll
            for (int blk = 0; blk < M / 16; blk++) {
                uint4 w = ld_stream16(cp + r * M + blk * 16);
                const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    uint32_t code = (ww[j / 4] >> (8 * (j % 4))) & 0xFFu;
                    s += s_lut[(blk * 16 + j) * 256 + code];
                }
            }
        } else {
#pragma unroll
            for (int m = 0; m < M; m++) s += s_lut[m * 256 + cp[r * M + m]];
        }
        uint32_t b = dist_bits(s);
        sp[r] = b;
        lo = min(lo, b);
        hi = max(hi, b);
    }
    if (minmax != nullptr) {
        __shared__ uint32_t s_lo, s_hi;
        if (threadIdx.x == 0) { s_lo = 0xFFFFFFFFu; s_hi = 0u; }
        __syncthreads();
        lo = __reduce_min_sync(0xFFFFFFFFu, lo);
        hi = __reduce_max_sync(0xFFFFFFFFu, hi);
        if ((threadIdx.x & 31) == 0) { atomicMin(&s_lo, lo); atomicMax(&s_hi, hi); }
        __syncthreads();
        if (threadIdx.x == 0 && s_lo <= s_hi) {
            atomicMin(&minmax[2 * prob], s_lo);
            atomicMax(&minmax[2 * prob + 1], s_hi);
        }
    }
}

// Exact re-scoring of candidate rows: LPR lanes per row, fp32 accumulation, same lane/tree
// order as the full scan so that a row scores identically on both paths.
template <int DT, int LPR>
__global__ void rerank_kernel(const uint16_t* __restrict__ keys, int64_t prob_stride, const uint16_t* __restrict__ q,
                              int q_mode, int group, const uint32_t* __restrict__ ids, int64_t ids_stride, int n_ids,
                              uint32_t* __restrict__ out_bits) {
    constexpr int D = LPR * 8;
    constexpr int R = 32 / LPR;
    constexpr int NL = 8;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col = lane % LPR, sub = lane / LPR;
    const int64_t prob = blockIdx.y;
    float qv[8];
    load_query8<DT>(query_base(q, prob, D, q_mode, group, 1, 0), D, q_mode, group, col * 8, qv);
    const int warps = blockDim.x / 32;
    const int tile0 = (blockIdx.x * warps + warp) * (NL * R);
    if (tile0 >= n_ids) return;
    const uint16_t* kp = keys + prob * prob_stride + col * 8;
    uint4 w[NL];
    uint32_t id[NL];
#pragma unroll
    for (int i = 0; i < NL; i++) {
        int j = min(tile0 + i * R + sub, n_ids - 1);
        id[i] = ids[prob * ids_stride + j];
        w[i] = id[i] != 0xFFFFFFFFu ? ld_stream16(kp + static_cast<int64_t>(id[i]) * D) : make_uint4(0, 0, 0, 0);
    }
    float part[NL];
#pragma unroll
    for (int i = 0; i < NL; i++) {
        float f[8];
        unpack8<DT>(w[i], f);
        float a = f[0] * qv[0];
#pragma unroll
        for (int j = 1; j < 8; j++) a = fmaf(f[j], qv[j], a);
        part[i] = a;
    }
    treduce<NL, LPR>(part, lane);
    const int my_i = treduce_base<NL, LPR>(lane);
    const bool writer = (col & ((1 << treduce_plain_bits<NL, LPR>()) - 1)) == 0;
    const int j = tile0 + my_i * R + sub;
    if (writer && j < n_ids) {
        const uint32_t rid = ids[prob * ids_stride + j];
        out_bits[prob * ids_stride + j] = rid != 0xFFFFFFFFu ? dist_bits(part[0]) : 0xFFFFFFFFu;
    }
}

}  // namespace

int pq_build_lut(const void* q, int q_mode, int group, int dtype, const float* centroids, int n_prob, int head_dim,
                 int n_sub, float* lut, cudaStream_t stream) {
    DC_REQUIRE(q && centroids && lut, "pq_build_lut: null pointer");
    DC_REQUIRE(dtype == DC_BF16 || dtype == DC_FP16, "pq_build_lut: dtype %d not supported", dtype);
    DC_REQUIRE(n_sub >= 1 && head_dim % n_sub == 0 && head_dim / n_sub <= 256, "pq_build_lut: bad n_sub=%d for head_dim=%d",
               n_sub, head_dim);
    DC_REQUIRE(n_prob >= 0 && n_prob <= 65535, "pq_build_lut: n_prob=%d", n_prob);
    if (n_prob == 0) return DC_OK;
    dim3 grid(n_sub, n_prob);
    size_t smem = (head_dim / n_sub) * sizeof(float);
    if (dtype == DC_BF16)
        pq_build_lut_kernel<DC_BF16><<<grid, 256, smem, stream>>>(static_cast<const uint16_t*>(q), q_mode, group,
                                                                 centroids, head_dim, n_sub, lut);
    else
        pq_build_lut_kernel<DC_FP16><<<grid, 256, smem, stream>>>(static_cast<const uint16_t*>(q), q_mode, group,
                                                                 centroids, head_dim, n_sub, lut);
    DC_CUDA_TRY(cudaGetLastError());
    return DC_OK;
}

int pq_adc_scan(const uint8_t* codes, int64_t prob_stride, int n_prob, int64_t n, int n_sub, const float* lut,
                uint32_t* scores, int64_t score_stride, uint32_t* minmax, cudaStream_t stream) {
    DC_REQUIRE(codes && lut && scores, "pq_adc_scan: null pointer");
    DC_REQUIRE(n_sub == 8 || n_sub == 16 || n_sub == 32, "pq_adc_scan: n_sub=%d not in {8,16,32}", n_sub);
    DC_REQUIRE(n_prob >= 0 && n_prob <= 65535 && n >= 0, "pq_adc_scan: bad sizes");
    DC_REQUIRE((reinterpret_cast<uintptr_t>(codes) & 15) == 0 && prob_stride % 16 == 0,
               "pq_adc_scan: codes must be 16-byte aligned");
    if (n_prob == 0 || n == 0) return DC_OK;
    const int rows_per_cta = 4096;
    dim3 grid(static_cast<unsigned>((n + rows_per_cta - 1) / rows_per_cta), n_prob);
    if (n_sub == 8)
        pq_adc_scan_kernel<8><<<grid, kAdcThreads, 0, stream>>>(codes, prob_stride, n, lut, scores, score_stride, minmax, rows_per_cta);
    else if (n_sub == 16)
        pq_adc_scan_kernel<16><<<grid, kAdcThreads, 0, stream>>>(codes, prob_stride, n, lut, scores, score_stride, minmax, rows_per_cta);
    else
        pq_adc_scan_kernel<32><<<grid, kAdcThreads, 0, stream>>>(codes, prob_stride, n, lut, scores, score_stride, minmax, rows_per_cta);
    DC_CUDA_TRY(cudaGetLastError());
    return DC_OK;
}

int rerank_scores(const void* keys, int64_t prob_stride, int n_prob, int head_dim, int dtype, const void* q, int q_mode,
                  int group, const uint32_t* ids, int64_t ids_stride, int n_ids, uint32_t* out_bits,
                  cudaStream_t stream) {
    DC_REQUIRE(keys && q && ids && out_bits, "rerank_scores: null pointer");
    DC_REQUIRE(dtype == DC_BF16 || dtype == DC_FP16, "rerank_scores: dtype %d not supported", dtype);
    DC_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256, "rerank_scores: head_dim %d not in {64,128,256}",
               head_dim);
    DC_REQUIRE(n_prob >= 0 && n_prob <= 65535 && n_ids >= 0, "rerank_scores: bad sizes");
    if (n_prob == 0 || n_ids == 0) return DC_OK;
    const int lpr = head_dim / 8;
    const int rows_per_warp = 8 * (32 / lpr);
    const int warps = 4;
    dim3 grid((n_ids + rows_per_warp * warps - 1) / (rows_per_warp * warps), n_prob);
    const uint16_t* k16 = static_cast<const uint16_t*>(keys);
    const uint16_t* q16 = static_cast<const uint16_t*>(q);
#define DC_RR(DT, LPR) rerank_kernel<DT, LPR><<<grid, warps * 32, 0, stream>>>(k16, prob_stride, q16, q_mode, group, ids, ids_stride, n_ids, out_bits)
    if (dtype == DC_BF16) {
        if (lpr == 8) DC_RR(DC_BF16, 8); else if (lpr == 16) DC_RR(DC_BF16, 16); else DC_RR(DC_BF16, 32);
    } else {
        if (lpr == 8) DC_RR(DC_FP16, 8); else if (lpr == 16) DC_RR(DC_FP16, 16); else DC_RR(DC_FP16, 32);
    }
#undef DC_RR
    DC_CUDA_TRY(cudaGetLastError());
    return DC_OK;
}

}  // namespace dc
