// Sparse gather-attention with split-K and log-sum-exp merge.
//
// Replaces, for one decode step, the gather loop of Index::search_bruteforce
// (diffcache_cpu/src/nsw.rs:623-629), the host->device copy of the gathered rows
// (src/diffcache/kvcache/diffcache.py:196-209) and flash_attn_with_kvcache over
// [retrieved | prefix | suffix | new token] (src/diffcache/base.py:134-142).
// The selected rows are read in place from the HBM store: every row is one contiguous
// 2*head_dim-byte segment fetched with 16-byte loads by the lanes that share it, all
// query heads of the kv head are served from the same read, and the row list of a problem
// is split over several CTAs whose (max, sum, accumulator) partials are merged by
// log-sum-exp in a second small kernel.
#include <cmath>
#include <cstdlib>

#include "common.cuh"

namespace dc {

namespace {

constexpr int kAttThreads = 256;
constexpr int kAttWarps = kAttThreads / 32;
constexpr int kAttLoads = 4;   // rows per lane per tile
constexpr int kAttStages = 3;  // shared-memory ring depth (tiles)
constexpr float kLog2e = 1.4426950408889634f;

struct AttendArgs {
    const uint16_t* k_store;
    const uint16_t* v_store;
    int64_t prob_stride;   // elements between problems in the store
    int64_t n_rows;        // valid rows per problem in the store
    int kv_heads;
    int group;             // query heads per kv head
    const uint16_t* q;     // (n_prob*group, D)
    const uint32_t* sel;   // (n_prob, sel_stride) row ids, or nullptr
    int64_t sel_stride;
    int n_sel;
    int64_t sel_base;      // id - sel_base = local row; ids outside [0, n_rows) are skipped
    const uint16_t* k_new; // (n_prob, D) or nullptr
    const uint16_t* v_new;
    uint16_t* res_k;       // resident rows
    uint16_t* res_v;
    int64_t res_stride_b, res_stride_h;
    int res_len;
    float scale_log2;      // softmax scale * log2(e)
    int n_split;
    float* part_acc;       // (n_prob, group, n_split, D)
    float* part_ml;        // (n_prob, group, n_split, 2)
};

// 16-byte asynchronous global->shared copy (LDGSTS); src_bytes = 0 writes zeros instead.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, int src_bytes) {
    const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// grid = (n_split, n_prob, head_chunks); GC query heads of one kv head per CTA.
//
// The rows of a split are processed in tiles of TILE rows.  Tiles are staged through a ring of
// kAttStages shared-memory buffers filled with asynchronous 16-byte copies issued kAttStages-1
// tiles ahead, so the bytes in flight per SM are set by shared memory (two CTAs x two tiles x
// TILE x 4*D bytes), not by registers; the row ids of the tile after that are fetched one
// iteration earlier still, so a copy never waits for its address.
template <int DT, int LPR, int GC>
__global__ void __launch_bounds__(kAttThreads)
sparse_attend_kernel(const AttendArgs a) {
    constexpr int D = LPR * 8;
    constexpr int R = 32 / LPR;                 // rows per warp-wide access
    constexpr int WR = kAttLoads * R;           // rows per warp per tile
    constexpr int TILE = kAttWarps * WR;        // rows per CTA tile
    constexpr int NV = kAttLoads * GC;          // partial dot products per lane per tile
    constexpr int NRG = kAttWarps * R;          // row groups whose accumulators are merged at the end
    constexpr int CNT = treduce_count<NV, LPR>();
    constexpr int PLAIN = treduce_plain_bits<NV, LPR>();
    constexpr int NS = kAttStages;
    constexpr int STAGE_ELEMS = 2 * TILE * D;   // K tile then V tile

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int col = lane % LPR, sub = lane / LPR;
    const int64_t prob = blockIdx.y;
    const int split = blockIdx.x;
    const int g0 = blockIdx.z * GC;             // first query head of this chunk
    const int b = static_cast<int>(prob / a.kv_heads), h = static_cast<int>(prob % a.kv_heads);

    extern __shared__ __align__(16) unsigned char att_smem[];
    uint16_t* s_stage = reinterpret_cast<uint16_t*>(att_smem);                    // [NS][2][TILE][D]
    float (*s_red)[GC][D + 4] = reinterpret_cast<float (*)[GC][D + 4]>(att_smem); // reuses the ring at the end
    __shared__ unsigned char s_valid[NS][TILE];
    __shared__ float s_p[GC][TILE];
    __shared__ float s_alpha[GC], s_m[GC], s_l[GC];

    const int has_new = a.k_new != nullptr ? 1 : 0;
    const int total = a.n_sel + a.res_len + has_new;
    const int per = (total + a.n_split - 1) / a.n_split;
    const int j0 = min(total, split * per);
    const int j1 = min(total, j0 + per);
    const int n_tiles = (j1 - j0 + TILE - 1) / TILE;

    // query heads of this chunk, pre-multiplied by scale*log2(e); heads beyond `group` are zero
    float qv[GC][8];
#pragma unroll
    for (int g = 0; g < GC; g++) {
        if (g0 + g < a.group) {
            uint4 w = *reinterpret_cast<const uint4*>(a.q + (prob * a.group + g0 + g) * D + col * 8);
            float f[8];
            unpack8<DT>(w, f);
#pragma unroll
            for (int j = 0; j < 8; j++) qv[g][j] = f[j] * a.scale_log2;
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++) qv[g][j] = 0.0f;
        }
    }

    const uint16_t* kst = a.k_store + prob * a.prob_stride;
    const uint16_t* vst = a.v_store + prob * a.prob_stride;
    uint16_t* rk = a.res_k ? a.res_k + b * a.res_stride_b + h * a.res_stride_h : nullptr;
    uint16_t* rv = a.res_v ? a.res_v + b * a.res_stride_b + h * a.res_stride_h : nullptr;
    const uint32_t* selp = a.sel ? a.sel + prob * a.sel_stride : nullptr;

    // flash-attn's in-place append of the new token (base.py:134-142): one CTA per problem
    if (has_new && split == 0 && blockIdx.z == 0 && rk != nullptr && tid < LPR) {
        reinterpret_cast<uint4*>(rk + static_cast<int64_t>(a.res_len) * D)[tid] =
            reinterpret_cast<const uint4*>(a.k_new + prob * D)[tid];
        reinterpret_cast<uint4*>(rv + static_cast<int64_t>(a.res_len) * D)[tid] =
            reinterpret_cast<const uint4*>(a.v_new + prob * D)[tid];
    }

    if (tid < GC) { s_m[tid] = -INFINITY; s_l[tid] = 0.0f; }

    float acc[GC][8];
#pragma unroll
    for (int g = 0; g < GC; g++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[g][j] = 0.0f;

    const int base_idx = treduce_base<NV, LPR>(lane);
    const bool writer = (col & ((1 << PLAIN) - 1)) == 0;

    // Row ids of this lane's kAttLoads rows of tile `t` (0xFFFFFFFF where the slot is not a store row).
    auto fetch_ids = [&](int t, uint32_t (&ids)[kAttLoads]) {
#pragma unroll
        for (int i = 0; i < kAttLoads; i++) {
            const int j = j0 + t * TILE + warp * WR + i * R + sub;
            ids[i] = (t < n_tiles && j < j1 && j < a.n_sel) ? selp[j] : 0xFFFFFFFFu;
        }
    };
    // Issue the copies of tile `t` into its ring slot (one commit group per call, possibly empty).
    auto issue_tile = [&](int t, const uint32_t (&ids)[kAttLoads]) {
        if (t < n_tiles) {
            uint16_t* ks = s_stage + (t % NS) * STAGE_ELEMS;
            uint16_t* vs = ks + TILE * D;
#pragma unroll
            for (int i = 0; i < kAttLoads; i++) {
                const int r = warp * WR + i * R + sub;
                const int j = j0 + t * TILE + r;
                const uint16_t* kp = nullptr;
                const uint16_t* vp = nullptr;
                if (j < j1) {
                    if (j < a.n_sel) {
                        const int64_t row = static_cast<int64_t>(ids[i]) - a.sel_base;
                        if (row >= 0 && row < a.n_rows) { kp = kst + row * D; vp = vst + row * D; }
                    } else if (j < a.n_sel + a.res_len) {
                        const int64_t row = j - a.n_sel;
                        kp = rk + row * D; vp = rv + row * D;
                    } else {
                        kp = a.k_new + prob * D; vp = a.v_new + prob * D;
                    }
                }
                const bool ok = kp != nullptr;
                // a skipped slot is zero-filled (src size 0) from any valid address
                cp_async16(ks + r * D + col * 8, ok ? kp + col * 8 : a.q, ok ? 16 : 0);
                cp_async16(vs + r * D + col * 8, ok ? vp + col * 8 : a.q, ok ? 16 : 0);
                if (col == 0) s_valid[t % NS][r] = ok ? 1 : 0;
            }
        }
        cp_async_commit();
    };

    uint32_t ids[kAttLoads];
#pragma unroll
    for (int t = 0; t < NS - 1; t++) {  // prologue: tiles 0 .. NS-2
        fetch_ids(t, ids);
        issue_tile(t, ids);
    }
    fetch_ids(NS - 1, ids);

    for (int t = 0; t < n_tiles; t++) {
        __syncthreads();  // tile t-1 fully consumed: its ring slot and s_p may be overwritten
        issue_tile(t + NS - 1, ids);
        fetch_ids(t + NS, ids);
        cp_async_wait<NS - 1>();
        __syncthreads();  // every thread's copies of tile t have landed

        const uint16_t* ks = s_stage + (t % NS) * STAGE_ELEMS;
        const uint16_t* vs = ks + TILE * D;
        const unsigned char* valid = s_valid[t % NS];

        // ---- Q.K partial dot products from shared memory ----
        float part[NV];
#pragma unroll
        for (int i = 0; i < kAttLoads; i++) {
            const int r = warp * WR + i * R + sub;
            const uint4 w = *reinterpret_cast<const uint4*>(ks + r * D + col * 8);
            float f[8];
            unpack8<DT>(w, f);
#pragma unroll
            for (int g = 0; g < GC; g++) {
                float sdot = f[0] * qv[g][0];
#pragma unroll
                for (int j = 1; j < 8; j++) sdot = fmaf(f[j], qv[g][j], sdot);
                part[i * GC + g] = sdot;
            }
        }
        treduce<NV, LPR>(part, lane);
        if (writer) {
#pragma unroll
            for (int c = 0; c < CNT; c++) {
                const int idx = base_idx + c;       // = i * GC + g
                const int i = idx / GC, g = idx % GC;
                const int r = warp * WR + i * R + sub;
                s_p[g][r] = valid[r] ? part[c] : -INFINITY;
            }
        }
        __syncthreads();

        // ---- online softmax: warp g owns query head g ----
        if (warp < GC) {
            const int g = warp;
            float mx = -INFINITY;
            for (int r = lane; r < TILE; r += 32) mx = fmaxf(mx, s_p[g][r]);
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
            const float m_old = s_m[g];
            const float m_new = fmaxf(m_old, mx);
            float sum = 0.0f;
            for (int r = lane; r < TILE; r += 32) {
                float sc = s_p[g][r];
                float p = (sc == -INFINITY) ? 0.0f : exp2f(sc - m_new);
                s_p[g][r] = p;
                sum += p;
            }
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
            if (lane == 0) {
                float alpha = (m_old == -INFINITY) ? 0.0f : exp2f(m_old - m_new);
                s_alpha[g] = alpha;
                s_m[g] = m_new;
                s_l[g] = s_l[g] * alpha + sum;
            }
        }
        __syncthreads();

        // ---- P.V ----
#pragma unroll
        for (int g = 0; g < GC; g++) {
            float alpha = s_alpha[g];
#pragma unroll
            for (int j = 0; j < 8; j++) acc[g][j] *= alpha;
        }
#pragma unroll
        for (int i = 0; i < kAttLoads; i++) {
            const int r = warp * WR + i * R + sub;
            const uint4 w = *reinterpret_cast<const uint4*>(vs + r * D + col * 8);
            float f[8];
            unpack8<DT>(w, f);
#pragma unroll
            for (int g = 0; g < GC; g++) {
                float p = s_p[g][r];
#pragma unroll
                for (int j = 0; j < 8; j++) acc[g][j] = fmaf(p, f[j], acc[g][j]);
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();  // the ring is idle: reuse it for the cross-row-group reduction

    // ---- merge the row groups' accumulators and write this split's partial ----
    const int rg = warp * R + sub;
#pragma unroll
    for (int g = 0; g < GC; g++) {
        *reinterpret_cast<float4*>(&s_red[rg][g][col * 8]) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
        *reinterpret_cast<float4*>(&s_red[rg][g][col * 8 + 4]) = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
    }
    __syncthreads();
    for (int e = tid; e < GC * D; e += kAttThreads) {
        int g = e / D, d = e % D;
        if (g0 + g >= a.group) continue;
        float s = 0.0f;
#pragma unroll
        for (int r = 0; r < NRG; r++) s += s_red[r][g][d];
        a.part_acc[((prob * a.group + g0 + g) * a.n_split + split) * D + d] = s;
    }
    if (tid < GC && g0 + tid < a.group) {
        float* ml = a.part_ml + ((prob * a.group + g0 + tid) * a.n_split + split) * 2;
        ml[0] = s_m[tid];
        ml[1] = s_l[tid];
    }
}

// Merge partials: part s of row r is acc[s*acc_ps + r*acc_rs .. +dim), (m, l) at ml[s*ml_ps + r*ml_rs].
// Split-K layout (rows, n_part, D): acc_ps = D, acc_rs = n_part*D.  All-gather layout
// (n_part, rows, D): acc_ps = part stride, acc_rs = D.  Writes either the normalised output in the
// element type (+ optional natural-log LSE) or the merged un-normalised (acc, m, l).
template <int DT>
__global__ void lse_combine_kernel(const float* __restrict__ part_acc, int64_t acc_ps, int64_t acc_rs,
                                   const float* __restrict__ part_ml, int64_t ml_ps, int64_t ml_rs, int n_part,
                                   int dim, uint16_t* __restrict__ out, float* __restrict__ out_lse,
                                   float* __restrict__ out_acc, float* __restrict__ out_ml) {
    const int64_t row = blockIdx.x;
    auto ml_at = [&](int s) { return part_ml + s * ml_ps + row * ml_rs; };
    auto acc_at = [&](int s) { return part_acc + s * acc_ps + row * acc_rs; };
    float m = -INFINITY;
    for (int s = 0; s < n_part; s++) m = fmaxf(m, ml_at(s)[0]);
    float l = 0.0f;
    for (int s = 0; s < n_part; s++) {
        const float* ml = ml_at(s);
        if (ml[0] != -INFINITY) l += ml[1] * exp2f(ml[0] - m);
    }
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        float o = 0.0f;
        for (int s = 0; s < n_part; s++) {
            const float ms = ml_at(s)[0];
            if (ms != -INFINITY) o += acc_at(s)[d] * exp2f(ms - m);
        }
        if (out) out[row * dim + d] = float_to_elem<DT>(l > 0.0f ? o / l : 0.0f);
        if (out_acc) out_acc[row * dim + d] = o;
    }
    if (threadIdx.x == 0) {
        if (out_lse) out_lse[row] = l > 0.0f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
        if (out_ml) { out_ml[row * 2] = m; out_ml[row * 2 + 1] = l; }
    }
}

constexpr size_t kAttSmemBytes = static_cast<size_t>(kAttStages) * 2 * (kAttWarps * kAttLoads * 4) * 64 * sizeof(uint16_t);
// = stages x (K,V) x TILE x D x 2 bytes; TILE x D = 32 lanes-rows x 8 loads x 4 warps x 8 elements for every D

template <int DT, int LPR, int GC>
int launch_attend_gc(const AttendArgs& a, dim3 grid, cudaStream_t stream) {
    // > 48 KB of dynamic shared memory needs an opt-in per kernel and device (not a stream operation)
    static bool ready[64] = {};
    int dev = 0;
    DC_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !ready[dev]) {
        DC_CUDA_TRY(cudaFuncSetAttribute(sparse_attend_kernel<DT, LPR, GC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kAttSmemBytes)));
        if (dev >= 0 && dev < 64) ready[dev] = true;
    }
    sparse_attend_kernel<DT, LPR, GC><<<grid, kAttThreads, kAttSmemBytes, stream>>>(a);
    DC_CUDA_TRY(cudaGetLastError());
    return DC_OK;
}

template <int DT, int LPR>
int launch_attend(const AttendArgs& a, int n_prob, cudaStream_t stream) {
    int gc = a.group >= 3 ? 4 : a.group;
    int chunks = (a.group + gc - 1) / gc;
    dim3 grid(static_cast<unsigned>(a.n_split), static_cast<unsigned>(n_prob), static_cast<unsigned>(chunks));
    if (gc == 1) return launch_attend_gc<DT, LPR, 1>(a, grid, stream);
    if (gc == 2) return launch_attend_gc<DT, LPR, 2>(a, grid, stream);
    return launch_attend_gc<DT, LPR, 4>(a, grid, stream);
}

}  // namespace

int attend_splits(int n_prob, int total_rows) {
    // One wave: two CTAs fit on an SM (shared-memory ring), so split each problem's row list until
    // the grid has about 2 x SMs CTAs, never more; at least 32 rows per split.
    static const int per_sm = [] {
        const char* s = std::getenv("DC_ATTEND_CTAS_PER_SM");
        int v = (s && *s) ? std::atoi(s) : 2;
        return std::min(std::max(v, 1), 4);  // the scratch buffer is sized for at most 4 per SM
    }();
    int target = std::max(1, (per_sm * sm_count()) / std::max(1, n_prob));
    int by_rows = std::max(1, (total_rows + 31) / 32);
    return std::max(1, std::min(std::min(target, by_rows), 256));
}

int64_t attend_scratch_bytes(int n_prob, int group, int head_dim) {
    // attend_splits() never makes more than 4*SMs + n_prob CTAs per head chunk (and at most 256 per problem)
    int64_t ctas = std::min<int64_t>(static_cast<int64_t>(n_prob) * 256, 4ll * sm_count() + n_prob);
    return ctas * group * (head_dim + 2) * static_cast<int64_t>(sizeof(float));
}

int lse_combine(const float* acc, int64_t acc_ps, int64_t acc_rs, const float* ml, int64_t ml_ps, int64_t ml_rs,
                int n_part, int64_t rows, int head_dim, int dtype, void* out, float* out_lse, float* out_acc,
                float* out_ml, cudaStream_t stream) {
    DC_REQUIRE(acc && ml && n_part >= 1 && rows >= 0, "lse_combine: bad arguments");
    DC_REQUIRE(dtype == DC_BF16 || dtype == DC_FP16, "lse_combine: dtype %d not supported", dtype);
    if (rows == 0) return DC_OK;
    int threads = std::min(256, ((head_dim + 31) / 32) * 32);
    if (dtype == DC_BF16)
        lse_combine_kernel<DC_BF16><<<static_cast<unsigned>(rows), threads, 0, stream>>>(
            acc, acc_ps, acc_rs, ml, ml_ps, ml_rs, n_part, head_dim, static_cast<uint16_t*>(out), out_lse, out_acc,
            out_ml);
    else
        lse_combine_kernel<DC_FP16><<<static_cast<unsigned>(rows), threads, 0, stream>>>(
            acc, acc_ps, acc_rs, ml, ml_ps, ml_rs, n_part, head_dim, static_cast<uint16_t*>(out), out_lse, out_acc,
            out_ml);
    DC_CUDA_TRY(cudaGetLastError());
    return DC_OK;
}

int sparse_attend(const void* k_store, const void* v_store, int64_t prob_stride, int64_t n_rows, int n_prob,
                  int kv_heads, int group, int head_dim, int dtype, const void* q, const uint32_t* sel,
                  int64_t sel_stride, int n_sel, int64_t sel_base, const void* k_new, const void* v_new, void* res_k,
                  void* res_v, int64_t res_stride_b, int64_t res_stride_h, int res_len, float scale, void* out,
                  float* out_lse, float* out_acc, float* out_ml, void* scratch, cudaStream_t stream) {
    DC_REQUIRE(q != nullptr && scratch != nullptr, "sparse_attend: null q/scratch");
    DC_REQUIRE(dtype == DC_BF16 || dtype == DC_FP16, "sparse_attend: dtype %d not supported", dtype);
    DC_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256, "sparse_attend: head_dim %d not in {64,128,256}",
               head_dim);
    DC_REQUIRE(n_prob >= 0 && n_prob <= 65535 && kv_heads >= 1 && n_prob % kv_heads == 0,
               "sparse_attend: n_prob=%d must be a multiple of kv_heads=%d", n_prob, kv_heads);
    DC_REQUIRE(group >= 1 && group <= 64, "sparse_attend: group=%d", group);
    DC_REQUIRE(n_sel >= 0 && res_len >= 0, "sparse_attend: negative length");
    DC_REQUIRE(n_sel == 0 || (sel && k_store && v_store), "sparse_attend: selection given without store/ids");
    DC_REQUIRE((k_new == nullptr) == (v_new == nullptr), "sparse_attend: k_new and v_new must both be set or both be NULL");
    DC_REQUIRE(res_len == 0 || (res_k && res_v), "sparse_attend: res_len > 0 needs resident buffers");
    DC_REQUIRE((out != nullptr) != (out_acc != nullptr && out_ml != nullptr),
               "sparse_attend: give either out or (out_acc, out_ml)");
    DC_REQUIRE(prob_stride % 8 == 0 && res_stride_b % 8 == 0 && res_stride_h % 8 == 0,
               "sparse_attend: strides must be multiples of 8 elements");
    DC_REQUIRE(((reinterpret_cast<uintptr_t>(k_store) | reinterpret_cast<uintptr_t>(v_store) |
                 reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_new) |
                 reinterpret_cast<uintptr_t>(v_new) | reinterpret_cast<uintptr_t>(res_k) |
                 reinterpret_cast<uintptr_t>(res_v)) & 15) == 0,
               "sparse_attend: every row pointer must be 16-byte aligned");
    if (n_prob == 0) return DC_OK;

    const int total = n_sel + res_len + (k_new ? 1 : 0);
    AttendArgs a;
    a.k_store = static_cast<const uint16_t*>(k_store);
    a.v_store = static_cast<const uint16_t*>(v_store);
    a.prob_stride = prob_stride;
    a.n_rows = n_rows;
    a.kv_heads = kv_heads;
    a.group = group;
    a.q = static_cast<const uint16_t*>(q);
    a.sel = sel;
    a.sel_stride = sel_stride;
    a.n_sel = n_sel;
    a.sel_base = sel_base;
    a.k_new = static_cast<const uint16_t*>(k_new);
    a.v_new = static_cast<const uint16_t*>(v_new);
    a.res_k = static_cast<uint16_t*>(res_k);
    a.res_v = static_cast<uint16_t*>(res_v);
    a.res_stride_b = res_stride_b;
    a.res_stride_h = res_stride_h;
    a.res_len = res_len;
    a.scale_log2 = (scale > 0.0f ? scale : 1.0f / std::sqrt(static_cast<float>(head_dim))) * kLog2e;
    a.n_split = attend_splits(n_prob, total);
    a.part_acc = static_cast<float*>(scratch);
    a.part_ml = a.part_acc + static_cast<int64_t>(n_prob) * a.n_split * group * head_dim;

    int rc;
#define DC_ATT_CASE(DT, LPR) rc = launch_attend<DT, LPR>(a, n_prob, stream)
    if (dtype == DC_BF16) {
        if (head_dim == 64) DC_ATT_CASE(DC_BF16, 8);
        else if (head_dim == 128) DC_ATT_CASE(DC_BF16, 16);
        else DC_ATT_CASE(DC_BF16, 32);
    } else {
        if (head_dim == 64) DC_ATT_CASE(DC_FP16, 8);
        else if (head_dim == 128) DC_ATT_CASE(DC_FP16, 16);
        else DC_ATT_CASE(DC_FP16, 32);
    }
#undef DC_ATT_CASE
    if (rc != DC_OK) return rc;
    return lse_combine(a.part_acc, head_dim, static_cast<int64_t>(a.n_split) * head_dim, a.part_ml, 2,
                       static_cast<int64_t>(a.n_split) * 2, a.n_split, static_cast<int64_t>(n_prob) * group, head_dim,
                       dtype, out, out_lse, out_acc, out_ml, stream);
}

}  // namespace dc

// ---------------------------------------------------------------------------------------------
// Sparse attention for callers that cannot allocate device memory.
//
// Some hosts of this library hand the whole of HBM to their own pool at start-up (inference
// servers do) or forbid cudaMalloc once they are serving, because it synchronises the device.
// Such a caller cannot provide the split-K scratch buffer dc_sparse_attend asks for, so this
// variant keeps the scratch in a fixed array that is part of the library image: every GPU that
// loads the library holds DC_NOALLOC_SCRATCH_BYTES (4 MiB) of it until the process exits.
//
// The array's name is only a host-side handle; the device address is looked up once per device
// with cudaGetSymbolAddress (with that device current) by the FIRST call on that device, so the
// first call on a device should be made before any stream capture.  Later calls only launch
// kernels.  Nothing here calls cudaMalloc, cudaFree or any allocating routine.
//
// All calls on a device share the one array.  It keeps whatever the previous call left there;
// that is harmless because the attention kernel writes every partial slot (accumulator, max,
// sum — empty splits included) before the merge kernel of the same call reads it, so nothing has
// to start at zero.  Two calls whose kernels overlap on the GPU (different streams, or graphs
// replayed concurrently) race on the array and must be serialised by the caller.
namespace dc {
namespace {

constexpr size_t kNoAllocScratchBytes = DC_NOALLOC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// Device address of g_noalloc_scratch on the current device (nullptr + error code on failure).
int noalloc_scratch_ptr(void** out) {
    static void* ptrs[64] = {};
    static bool ready[64] = {};
    *out = nullptr;
    int dev = 0;
    DC_CUDA_TRY(cudaGetDevice(&dev));
    DC_REQUIRE(dev >= 0 && dev < 64, "dc_sparse_attend_noalloc: device ordinal %d not supported", dev);
    if (!ready[dev]) {
        void* p = nullptr;
        DC_CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        DC_REQUIRE(p != nullptr, "dc_sparse_attend_noalloc: no device address for the static scratch array");
        ptrs[dev] = p;
        ready[dev] = true;
    }
    *out = ptrs[dev];
    return DC_OK;
}

}  // namespace
}  // namespace dc

extern "C" int dc_sparse_attend_noalloc(const void* k_store, const void* v_store, int64_t prob_stride, int64_t n_rows,
                                        int n_prob, int kv_heads, int group, int head_dim, int dtype, const void* q,
                                        const uint32_t* sel, int64_t sel_stride, int n_sel, int64_t sel_base,
                                        const void* k_new, const void* v_new, void* res_k, void* res_v,
                                        int64_t res_stride_b, int64_t res_stride_h, int res_len, float scale,
                                        void* out, float* out_lse, float* out_acc, float* out_ml, uint64_t stream) {
    using namespace dc;
    DC_REQUIRE(n_prob >= 0 && n_prob <= 65535 && group >= 1 && group <= 64 && n_sel >= 0 && res_len >= 0,
               "dc_sparse_attend_noalloc: bad sizes");
    DC_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256,
               "dc_sparse_attend_noalloc: head_dim %d not in {64,128,256}", head_dim);
    const int total = n_sel + res_len + (k_new ? 1 : 0);
    const int64_t need = static_cast<int64_t>(n_prob) * attend_splits(n_prob, total) * group * (head_dim + 2) *
                         static_cast<int64_t>(sizeof(float));
    if (need > static_cast<int64_t>(kNoAllocScratchBytes)) {
        set_error("dc_sparse_attend_noalloc: this problem needs %lld bytes of split-K scratch but the static array "
                  "holds %lld (DC_NOALLOC_SCRATCH_BYTES); use dc_sparse_attend with a caller-provided buffer",
                  static_cast<long long>(need), static_cast<long long>(kNoAllocScratchBytes));
        return DC_EINVAL;
    }
    void* scratch = nullptr;
    int rc = noalloc_scratch_ptr(&scratch);
    if (rc != DC_OK) return rc;
    return sparse_attend(k_store, v_store, prob_stride, n_rows, n_prob, kv_heads, group, head_dim, dtype, q, sel,
                         sel_stride, n_sel, sel_base, k_new, v_new, res_k, res_v, res_stride_b, res_stride_h, res_len,
                         scale, out, out_lse, out_acc, out_ml, scratch, as_stream(stream));
}
