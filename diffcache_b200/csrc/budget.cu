// Adaptive retrieval budget ("k-check").
//
// The reference stops its graph search early at the checkpoints of `k_check_seq` when a power-law
// fit of the best logits says the top-h keys already hold `attn_mass_threshold` of the attention
// mass: fit_alpha_from_logits / estimate_top_h_mass / k_check_early_stoppable
// (diffcache_cpu/src/nsw.rs:198-300), applied at diffcache_cpu/src/nsw.rs:339-376.  With an exact
// scan the best-first ranking keys of every problem are already on the device, so the same test is
// a small epilogue of the select: one CTA per problem walks the checkpoints with running sums and
// writes the first h that passes (k if none does); the attention kernel then skips the rows
// beyond that budget.
#include "common.cuh"

namespace dc {

namespace {

constexpr int kBudgetThreads = 256;
constexpr int kMaxCheckpoints = 16;
constexpr int kMinRank = 5;  // the reference fits ranks >= 5 (nsw.rs:292)

struct BudgetSeq {
    int n;
    int h[kMaxCheckpoints];
};

__device__ __forceinline__ double block_sum(double v, double* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    __syncthreads();  // scratch free again
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    double s = 0.0;
    for (int w = 0; w < kBudgetThreads / 32; w++) s += scratch[w];
    return s;
}

// bits: (n_prob, stride) best-first ranking keys; budget[p] = first passing checkpoint or k.
__global__ void __launch_bounds__(kBudgetThreads)
adaptive_budget_kernel(const uint32_t* __restrict__ bits, int64_t stride, int k, const int32_t* __restrict__ n_dev,
                       float sqrt_dim, BudgetSeq seq, float threshold, int32_t* __restrict__ budget) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ double scratch[kBudgetThreads / 32];
    const int64_t prob = blockIdx.x;
    if (n_dev != nullptr) k = min(k, *n_dev);  // keys beyond the rows the store holds are pads
    if (k <= 0) {
        if (threadIdx.x == 0) budget[prob] = 0;
        return;
    }
    const uint32_t* b = bits + prob * stride;
    const int tid = threadIdx.x;
    const float z0 = (65536.0f - __uint_as_float(b[0])) / sqrt_dim;  // best logit = maximum of every head
    double sx = 0, sy = 0, sxx = 0, sxy = 0, head = 0;
    int prev = 0, result = k;
    for (int e = 0; e < seq.n; e++) {
        const int h = seq.h[e];
        if (h >= k) break;
        if (h <= prev) continue;
        double px = 0, py = 0, pxx = 0, pxy = 0, ph = 0;
        for (int i = prev + tid; i < h; i += kBudgetThreads) {
            const float z = (65536.0f - __uint_as_float(b[i])) / sqrt_dim;
            ph += static_cast<double>(expf(z - z0));
            if (i >= kMinRank - 1) {
                const double x = log(static_cast<double>(i + 1));
                px += x; py += z; pxx += x * x; pxy += x * static_cast<double>(z);
            }
        }
        sx += block_sum(px, scratch);
        sy += block_sum(py, scratch);
        sxx += block_sum(pxx, scratch);
        sxy += block_sum(pxy, scratch);
        head += block_sum(ph, scratch);
        prev = h;
        if (kMinRank >= h) continue;                       // fit undefined (nsw.rs:203-205)
        const double n = static_cast<double>(h - kMinRank + 1);
        const double denom = n * sxx - sx * sx;
        if (n < 2.0 || fabs(denom) < 1e-12) continue;
        const float alpha = static_cast<float>(-(n * sxy - sx * sy) / denom);
        if (alpha <= 1.0f) continue;                        // infinite tail mass in the model (nsw.rs:253-256)
        const float zh = (65536.0f - __uint_as_float(b[h - 1])) / sqrt_dim;
        const float headf = static_cast<float>(head);
        const float tail = expf(zh - z0) * static_cast<float>(h) / (alpha - 1.0f);
        const float den = headf + tail;
        if (den > 0.0f && headf / den >= threshold) { result = h; break; }
    }
    if (tid == 0) budget[prob] = result;
}

}  // namespace

int adaptive_budget(const uint32_t* bits, int64_t stride, int n_prob, int k, int head_dim, const int* seq, int n_seq,
                    float threshold, int32_t* budget, cudaStream_t stream, const int32_t* n_dev) {
    DC_REQUIRE(bits && budget, "adaptive_budget: null pointer");
    DC_REQUIRE(n_prob >= 0 && k >= 1 && head_dim >= 1, "adaptive_budget: bad sizes");
    DC_REQUIRE(n_seq >= 0 && n_seq <= kMaxCheckpoints && (n_seq == 0 || seq != nullptr),
               "adaptive_budget: at most %d checkpoints", kMaxCheckpoints);
    if (n_prob == 0) return DC_OK;
    BudgetSeq s;
    s.n = n_seq;
    for (int i = 0; i < kMaxCheckpoints; i++) s.h[i] = i < n_seq ? seq[i] : 0;
    DC_CUDA_TRY(launch_chained(adaptive_budget_kernel, dim3(n_prob), dim3(kBudgetThreads), 0, stream, 0u, bits, stride, k,
                               n_dev, sqrtf(static_cast<float>(head_dim)), s, threshold, budget));
    return DC_OK;
}

}  // namespace dc
