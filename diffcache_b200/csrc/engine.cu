// Engine object and the extern "C" boundary (declared in include/diffcache_b200.h).
//
// dc_engine is the HBM-resident counterpart of DataLayer<bf16> + Index<T>
// (diffcache_cpu/src/lib.rs:189-197, diffcache_cpu/src/nsw.rs:47-56): it owns the key and
// value stores K,V[bsz*kv_heads][max_ctx_len][head_dim] and every scratch buffer a decode
// step needs, all allocated once in dc_create so that the per-step calls only enqueue
// kernels (they can be captured in a CUDA graph).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"

namespace dc {

// ---- kernels defined in the other translation units ----
int score_scan(const void* keys, int64_t prob_stride, int n_prob, int64_t n, int head_dim, int dtype, const void* q,
               int q_mode, int group, uint32_t* scores, int64_t score_stride, uint32_t* minmax, cudaStream_t stream,
               uint32_t* status = nullptr, int kv_heads = 1, int64_t q_stride_b = 0);
int topk_select(const uint32_t* bits, const uint32_t* ids, int64_t in_stride, int n_prob, int64_t n, int k,
                const uint32_t* minmax, uint32_t id_offset, uint32_t* out_bits, uint32_t* out_ids, int64_t out_stride,
                uint32_t* status, cudaStream_t stream, uint32_t* minmax_reset = nullptr);
int select_prepare();
int64_t select_scratch_bytes(int n_prob);
int merge_sorted_count(const uint32_t* bits_all, int world, int n_prob, int k, int my_rank, int32_t* out_count,
                       cudaStream_t stream);
int sparse_attend(const void* k_store, const void* v_store, int64_t prob_stride, int64_t n_rows, int n_prob,
                  int kv_heads, int group, int head_dim, int dtype, const void* q, const uint32_t* sel,
                  int64_t sel_stride, int n_sel, int64_t sel_base, const void* k_new, const void* v_new, void* res_k,
                  void* res_v, int64_t res_stride_b, int64_t res_stride_h, int res_len, float scale, void* out,
                  float* out_lse, float* out_acc, float* out_ml, void* scratch, cudaStream_t stream,
                  const int32_t* sel_count = nullptr, int64_t q_stride_b = 0, int64_t new_stride_b = 0);
int adaptive_budget(const uint32_t* bits, int64_t stride, int n_prob, int k, int head_dim, const int* seq, int n_seq,
                    float threshold, int32_t* budget, cudaStream_t stream);
int64_t attend_scratch_bytes(int n_prob, int group, int head_dim);
int lse_combine(const float* acc, int64_t acc_ps, int64_t acc_rs, const float* ml, int64_t ml_ps, int64_t ml_rs,
                int n_part, int64_t rows, int head_dim, int dtype, void* out, float* out_lse, float* out_acc,
                float* out_ml, cudaStream_t stream);
int pq_build_lut(const void* q, int q_mode, int group, int dtype, const float* centroids, int n_prob, int head_dim,
                 int n_sub, float* lut, cudaStream_t stream);
int pq_adc_scan(const uint8_t* codes, int64_t prob_stride, int n_prob, int64_t n, int n_sub, const float* lut,
                uint32_t* scores, int64_t score_stride, uint32_t* minmax, cudaStream_t stream);
int rerank_scores(const void* keys, int64_t prob_stride, int n_prob, int head_dim, int dtype, const void* q, int q_mode,
                  int group, const uint32_t* ids, int64_t ids_stride, int n_ids, uint32_t* out_bits,
                  cudaStream_t stream);

// ---- error state ----
static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t err, const char* what) {
    set_error("CUDA error %d (%s) in %s", static_cast<int>(err), cudaGetErrorString(err), what);
    return err == cudaErrorMemoryAllocation ? DC_ENOMEM : DC_ECUDA;
}

int sm_count() {
    static std::atomic<int> cached[64];  // zero-initialised; a racing first call stores the same value twice
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev >= 0 && dev < 64) {
        const int c = cached[dev].load(std::memory_order_relaxed);
        if (c > 0) return c;
    }
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    if (dev >= 0 && dev < 64) cached[dev].store(n, std::memory_order_relaxed);
    return n;
}

namespace {

__global__ void init_minmax_kernel(uint32_t* minmax, int n_prob) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_prob) { minmax[2 * i] = 0xFFFFFFFFu; minmax[2 * i + 1] = 0u; }
}

// out[p][i][:] = store[p][ids[p][i]][:] with 16-byte lanes; ids beyond n_valid rows copy zeros
__global__ void gather_rows_kernel(const uint16_t* __restrict__ store, int64_t prob_stride, int dim,
                                   const uint32_t* __restrict__ ids, int64_t ids_stride, int n_ids,
                                   uint16_t* __restrict__ out) {
    const int lanes = dim / 8;
    const int64_t prob = blockIdx.y;
    const int rows_per_block = blockDim.x / lanes;
    const int i = blockIdx.x * rows_per_block + threadIdx.x / lanes;
    const int c = threadIdx.x % lanes;
    if (i >= n_ids || threadIdx.x >= rows_per_block * lanes) return;
    const uint32_t id = ids[prob * ids_stride + i];
    uint4 w = make_uint4(0, 0, 0, 0);
    if (id != 0xFFFFFFFFu) w = *reinterpret_cast<const uint4*>(store + prob * prob_stride + static_cast<int64_t>(id) * dim + c * 8);
    *reinterpret_cast<uint4*>(out + (prob * n_ids + i) * dim + c * 8) = w;
}

// strided (batch, head, row) -> store copy for device-resident sources
__global__ void ingest_rows_kernel(const uint16_t* __restrict__ src, int64_t stride_b, int64_t stride_h,
                                   int64_t stride_s, int kv_heads, int dim, int64_t seq_len,
                                   uint16_t* __restrict__ store, int64_t prob_stride, int64_t row0) {
    const int lanes = dim / 8;
    const int64_t prob = blockIdx.y;
    const int rows_per_block = blockDim.x / lanes;
    const int64_t s = static_cast<int64_t>(blockIdx.x) * rows_per_block + threadIdx.x / lanes;
    const int c = threadIdx.x % lanes;
    if (s >= seq_len || threadIdx.x >= rows_per_block * lanes) return;
    const int64_t b = prob / kv_heads, h = prob % kv_heads;
    const uint16_t* sp = src + b * stride_b + h * stride_h + s * stride_s + c * 8;
    *reinterpret_cast<uint4*>(store + prob * prob_stride + (row0 + s) * dim + c * 8) = *reinterpret_cast<const uint4*>(sp);
}

template <int DT>
__global__ void keys_to_f32_kernel(const uint16_t* __restrict__ store, int64_t prob_stride, int64_t ctx, int dim,
                                   float* __restrict__ out) {
    const int64_t prob = blockIdx.y;
    const int64_t per = ctx * dim;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < per;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        out[prob * per + i] = elem_to_float<DT>(store[prob * prob_stride + i]);
}

bool is_device_ptr(const void* p) {
    if (p == nullptr) return true;
    cudaPointerAttributes at;
    cudaError_t e = cudaPointerGetAttributes(&at, p);
    if (e != cudaSuccess) { cudaGetLastError(); return false; }
    return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}

}  // namespace
}  // namespace dc

using namespace dc;

struct dc_engine {
    int bsz = 0, q_heads = 0, kv_heads = 0, head_dim = 0, dtype = 0, device = 0;
    int n_prob = 0, group = 0;
    int64_t max_ctx = 0, ctx_len = 0, row_offset = 0;
    int64_t prob_stride = 0;   // elements
    int64_t score_stride = 0;  // elements
    uint16_t* k = nullptr;
    uint16_t* v = nullptr;
    uint32_t* scores = nullptr;
    uint32_t* minmax = nullptr;
    uint32_t* sel_idx = nullptr;   // (n_prob, DC_MAX_TOPK) worst case, used with stride = k
    uint32_t* sel_bits = nullptr;
    uint32_t* status = nullptr;
    void* att_scratch = nullptr;
    uint16_t* q_dev = nullptr;     // staging for host-side queries (n_prob*group, D)
    uint16_t* stage_k = nullptr;   // lazily allocated staging for host-side dc_query outputs
    uint16_t* stage_v = nullptr;
    int64_t stage_rows = 0;
    std::vector<cudaEvent_t> phase_events;  // 4 per timed step: before scan, after scan, after select, after attend
    int phase_cap = 0, phase_count = 0;
    int32_t* budget = nullptr;     // per-problem adaptive budget (k-check), n_prob entries
    int budget_seq[16] = {};
    int budget_n = 0;              // 0 = adaptive budget off
    float budget_threshold = 0.9f;
};

namespace {

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
        if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

#define DC_ENGINE_ENTER(e)                                         \
    if ((e) == nullptr) { set_error("null engine"); return DC_EINVAL; } \
    DeviceGuard _guard((e)->device);                               \
    if (!_guard.ok) { set_error("cannot select device %d", (e)->device); return DC_ECUDA; }

int init_minmax(dc_engine* e, cudaStream_t s) {
    init_minmax_kernel<<<(e->n_prob + 127) / 128, 128, 0, s>>>(e->minmax, e->n_prob);
    DC_CUDA_TRY(cudaGetLastError());
    return DC_OK;
}

int gather_rows(const void* store, int64_t prob_stride, int n_prob, int dim, const uint32_t* ids, int64_t ids_stride,
                int n_ids, void* out, cudaStream_t s) {
    if (n_prob == 0 || n_ids == 0) return DC_OK;
    const int lanes = dim / 8;
    const int rows_per_block = 256 / lanes;
    dim3 grid((n_ids + rows_per_block - 1) / rows_per_block, n_prob);
    gather_rows_kernel<<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(store), prob_stride, dim, ids, ids_stride,
                                            n_ids, static_cast<uint16_t*>(out));
    DC_CUDA_TRY(cudaGetLastError());
    return DC_OK;
}

// scan + select on the engine's own buffers; leaves (bits, ids) of the k best rows per problem in
// out_bits/out_ids (row stride k).  q: device pointer, q_mode as in dc_score_scan.
int scan_and_select(dc_engine* e, const void* q, int q_mode, int k, uint32_t id_offset, uint32_t* out_bits,
                    uint32_t* out_ids, cudaStream_t s, cudaEvent_t* ev = nullptr, int64_t q_stride_b = 0) {
    // e->minmax is in its initial state here: set once in dc_create, and put back by every select
    if (ev) DC_CUDA_TRY(cudaEventRecord(ev[0], s));
    int rc = score_scan(e->k, e->prob_stride, e->n_prob, e->ctx_len, e->head_dim, e->dtype, q, q_mode, e->group, e->scores,
                    e->score_stride, e->minmax, s, e->status, e->kv_heads, q_stride_b);
    if (rc) return rc;
    if (ev) DC_CUDA_TRY(cudaEventRecord(ev[1], s));
    rc = topk_select(e->scores, nullptr, e->score_stride, e->n_prob, e->ctx_len, k, e->minmax, id_offset, out_bits,
                     out_ids, k, e->status, s, e->minmax);
    if (rc) return rc;
    if (ev) DC_CUDA_TRY(cudaEventRecord(ev[2], s));
    return DC_OK;
}

int copy_rows_in(dc_engine* e, const void* src, uint16_t* store, int64_t seq_len, int64_t row0, int64_t stride_b,
                 int64_t stride_h, int64_t stride_s, cudaStream_t s) {
    const int D = e->head_dim;
    const size_t es = sizeof(uint16_t);
    if (seq_len == 0) return DC_OK;
    if (is_device_ptr(src)) {
        const int lanes = D / 8;
        const int rows_per_block = 256 / lanes;
        dim3 grid(static_cast<unsigned>((seq_len + rows_per_block - 1) / rows_per_block), e->n_prob);
        ingest_rows_kernel<<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(src), stride_b, stride_h, stride_s,
                                                e->kv_heads, D, seq_len, store, e->prob_stride, row0);
        DC_CUDA_TRY(cudaGetLastError());
        return DC_OK;
    }
    // host source: one pitched copy per problem (rows of D elements, source pitch = stride_s)
    if (stride_s == D && stride_h == seq_len * D && stride_b == e->kv_heads * stride_h) {
        DC_CUDA_TRY(cudaMemcpy2DAsync(store + row0 * D, e->prob_stride * es, src, seq_len * D * es, seq_len * D * es,
                                      e->n_prob, cudaMemcpyHostToDevice, s));
        return DC_OK;
    }
    for (int p = 0; p < e->n_prob; p++) {
        const int64_t b = p / e->kv_heads, h = p % e->kv_heads;
        const uint16_t* sp = static_cast<const uint16_t*>(src) + b * stride_b + h * stride_h;
        DC_CUDA_TRY(cudaMemcpy2DAsync(store + p * e->prob_stride + row0 * D, D * es, sp, stride_s * es, D * es, seq_len,
                                      cudaMemcpyHostToDevice, s));
    }
    return DC_OK;
}

int check_status_word(dc_engine* e, cudaStream_t s) {
    uint32_t st = 0;
    DC_CUDA_TRY(cudaMemcpyAsync(&st, e->status, sizeof(st), cudaMemcpyDeviceToHost, s));
    DC_CUDA_TRY(cudaStreamSynchronize(s));
    if (st != 0) {
        set_error("a kernel reported internal status %u", st);
        cudaMemsetAsync(e->status, 0, sizeof(uint32_t), s);
        return DC_EDEVICE;
    }
    return DC_OK;
}

}  // namespace

extern "C" {

const char* dc_last_error(void) { return g_err; }

int dc_version(void) { return 100; }

int dc_create(int bsz, int q_heads, int kv_heads, int head_dim, int64_t max_ctx_len, int dtype, int device,
              dc_engine** out) {
    DC_REQUIRE(out != nullptr, "dc_create: null out");
    *out = nullptr;
    DC_REQUIRE(bsz >= 1 && kv_heads >= 1 && q_heads >= 1, "dc_create: bsz/q_heads/kv_heads must be positive");
    DC_REQUIRE(q_heads % kv_heads == 0, "q_head_num must be multiple of kv_head_num");
    DC_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256, "dc_create: head_dim %d not in {64,128,256}",
               head_dim);
    DC_REQUIRE(dtype == DC_BF16 || dtype == DC_FP16, "dc_create: dtype %d not supported", dtype);
    DC_REQUIRE(max_ctx_len >= 1 && max_ctx_len < (1ll << 31), "dc_create: max_ctx_len=%lld outside [1, 2^31)",
               static_cast<long long>(max_ctx_len));
    DC_REQUIRE(static_cast<int64_t>(bsz) * kv_heads <= 65535, "dc_create: bsz*kv_heads must be <= 65535");
    DeviceGuard guard(device);
    if (!guard.ok) { set_error("dc_create: cannot select device %d", device); return DC_ECUDA; }

    dc_engine* e = new dc_engine();
    e->bsz = bsz; e->q_heads = q_heads; e->kv_heads = kv_heads; e->head_dim = head_dim; e->dtype = dtype;
    e->device = device; e->n_prob = bsz * kv_heads; e->group = q_heads / kv_heads;
    e->max_ctx = max_ctx_len;
    e->prob_stride = max_ctx_len * head_dim;
    e->score_stride = (max_ctx_len + 3) / 4 * 4;
    const size_t store_bytes = static_cast<size_t>(e->n_prob) * e->prob_stride * sizeof(uint16_t);
    cudaError_t err = cudaSuccess;
    auto alloc = [&](void** p, size_t bytes) {
        if (err == cudaSuccess) err = cudaMalloc(p, std::max<size_t>(bytes, 256));
    };
    alloc(reinterpret_cast<void**>(&e->k), store_bytes);
    alloc(reinterpret_cast<void**>(&e->v), store_bytes);
    alloc(reinterpret_cast<void**>(&e->scores), static_cast<size_t>(e->n_prob) * e->score_stride * sizeof(uint32_t));
    alloc(reinterpret_cast<void**>(&e->minmax), static_cast<size_t>(e->n_prob) * 2 * sizeof(uint32_t));
    const size_t sel_cap = static_cast<size_t>(std::min<int64_t>(DC_MAX_TOPK, max_ctx_len));
    alloc(reinterpret_cast<void**>(&e->sel_idx), static_cast<size_t>(e->n_prob) * sel_cap * sizeof(uint32_t));
    alloc(reinterpret_cast<void**>(&e->sel_bits), static_cast<size_t>(e->n_prob) * sel_cap * sizeof(uint32_t));
    alloc(reinterpret_cast<void**>(&e->status), 256);
    alloc(reinterpret_cast<void**>(&e->budget), static_cast<size_t>(e->n_prob) * sizeof(int32_t));
    alloc(&e->att_scratch, static_cast<size_t>(attend_scratch_bytes(e->n_prob, e->group, head_dim)));
    alloc(reinterpret_cast<void**>(&e->q_dev), static_cast<size_t>(bsz) * q_heads * head_dim * sizeof(uint16_t));
    if (err == cudaSuccess) err = cudaMemset(e->status, 0, 256);
    if (err == cudaSuccess) err = cudaMemset(e->k, 0, store_bytes);   // the reference zero-fills its store
    if (err == cudaSuccess) err = cudaMemset(e->v, 0, store_bytes);   // (HugeArray, diffcache_cpu/src/lib.rs:91-105)
    if (err != cudaSuccess) {
        int rc = cuda_fail(err, "dc_create allocation");
        dc_destroy(e);
        return rc;
    }
    int rc = select_prepare();
    if (rc == DC_OK) rc = init_minmax(e, nullptr);
    if (rc == DC_OK && cudaDeviceSynchronize() != cudaSuccess) rc = cuda_fail(cudaGetLastError(), "dc_create");
    if (rc) { dc_destroy(e); return rc; }
    *out = e;
    return DC_OK;
}

int dc_destroy(dc_engine* e) {
    if (e == nullptr) return DC_OK;
    DeviceGuard guard(e->device);
    cudaDeviceSynchronize();
    cudaFree(e->k); cudaFree(e->v); cudaFree(e->scores); cudaFree(e->minmax); cudaFree(e->sel_idx);
    cudaFree(e->sel_bits); cudaFree(e->status); cudaFree(e->budget); cudaFree(e->att_scratch); cudaFree(e->q_dev);
    cudaFree(e->stage_k); cudaFree(e->stage_v);
    for (cudaEvent_t ev : e->phase_events) cudaEventDestroy(ev);
    cudaGetLastError();
    delete e;
    return DC_OK;
}

int dc_set_row_offset(dc_engine* e, int64_t row_offset) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(row_offset >= 0 && row_offset + e->max_ctx < (1ll << 32), "dc_set_row_offset: offset out of range");
    e->row_offset = row_offset;
    return DC_OK;
}

int dc_prefill(dc_engine* e, const void* keys, const void* vals, int64_t seq_len, int64_t stride_b, int64_t stride_h,
               int64_t stride_s, uint64_t stream) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(keys && vals, "dc_prefill: null keys/vals");
    DC_REQUIRE(seq_len >= 0 && seq_len <= e->max_ctx, "dc_prefill: seq_len=%lld exceeds max_ctx_len=%lld",
               static_cast<long long>(seq_len), static_cast<long long>(e->max_ctx));
    DC_REQUIRE(stride_b % 8 == 0 && stride_h % 8 == 0 && stride_s % 8 == 0 &&
                   ((reinterpret_cast<uintptr_t>(keys) | reinterpret_cast<uintptr_t>(vals)) & 15) == 0,
               "dc_prefill: pointers must be 16-byte aligned and strides multiples of 8 elements");
    cudaStream_t s = as_stream(stream);
    int rc = copy_rows_in(e, keys, e->k, seq_len, 0, stride_b, stride_h, stride_s, s);
    if (rc) return rc;
    rc = copy_rows_in(e, vals, e->v, seq_len, 0, stride_b, stride_h, stride_s, s);
    if (rc) return rc;
    e->ctx_len = seq_len;
    if (!is_device_ptr(keys) || !is_device_ptr(vals)) DC_CUDA_TRY(cudaStreamSynchronize(s));
    return DC_OK;
}

int dc_insert(dc_engine* e, const void* keys, const void* vals, uint64_t stream) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(keys && vals, "dc_insert: null keys/vals");
    if (e->ctx_len >= e->max_ctx) { set_error("dc_insert: store is full (max_ctx_len=%lld)", static_cast<long long>(e->max_ctx)); return DC_ESTATE; }
    cudaStream_t s = as_stream(stream);
    const size_t rb = e->head_dim * sizeof(uint16_t);
    DC_CUDA_TRY(cudaMemcpy2DAsync(e->k + e->ctx_len * e->head_dim, e->prob_stride * sizeof(uint16_t), keys, rb, rb,
                                  e->n_prob, cudaMemcpyDefault, s));
    DC_CUDA_TRY(cudaMemcpy2DAsync(e->v + e->ctx_len * e->head_dim, e->prob_stride * sizeof(uint16_t), vals, rb, rb,
                                  e->n_prob, cudaMemcpyDefault, s));
    e->ctx_len += 1;
    if (!is_device_ptr(keys) || !is_device_ptr(vals)) DC_CUDA_TRY(cudaStreamSynchronize(s));
    return DC_OK;
}

int dc_ctx_len(dc_engine* e, int64_t* out) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(out != nullptr, "dc_ctx_len: null out");
    *out = e->ctx_len;
    return DC_OK;
}

int dc_check_status(dc_engine* e, uint64_t stream) {
    DC_ENGINE_ENTER(e);
    return check_status_word(e, as_stream(stream));
}

int dc_query(dc_engine* e, const void* q_mean, int ef, void* out_keys, void* out_vals, int32_t* out_idx,
             uint32_t* out_bits, uint64_t stream) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(q_mean != nullptr, "dc_query: null query");
    DC_REQUIRE(ef >= 0, "dc_query: negative ef");
    const int k = static_cast<int>(std::min<int64_t>(ef, e->ctx_len));  // lib.rs:374
    DC_REQUIRE(k <= DC_MAX_TOPK, "dc_query: ef=%d exceeds DC_MAX_TOPK=%d", k, DC_MAX_TOPK);
    if (k == 0) return DC_OK;
    cudaStream_t s = as_stream(stream);
    const int D = e->head_dim;
    const size_t es = sizeof(uint16_t);
    bool host_io = false;

    const void* q_dev = q_mean;
    if (!is_device_ptr(q_mean)) {
        host_io = true;
        DC_CUDA_TRY(cudaMemcpyAsync(e->q_dev, q_mean, static_cast<size_t>(e->n_prob) * D * es, cudaMemcpyHostToDevice, s));
        q_dev = e->q_dev;
    }
    int rc = scan_and_select(e, q_dev, 0, k, 0u, e->sel_bits, e->sel_idx, s);
    if (rc) return rc;

    const size_t rows = static_cast<size_t>(e->n_prob) * k;
    const bool k_host = out_keys && !is_device_ptr(out_keys);
    const bool v_host = out_vals && !is_device_ptr(out_vals);
    if ((k_host || v_host) && e->stage_rows < static_cast<int64_t>(rows)) {
        DC_CUDA_TRY(cudaStreamSynchronize(s));
        cudaFree(e->stage_k); cudaFree(e->stage_v);
        e->stage_k = e->stage_v = nullptr; e->stage_rows = 0;
        DC_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&e->stage_k), rows * D * es));
        DC_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&e->stage_v), rows * D * es));
        e->stage_rows = static_cast<int64_t>(rows);
    }
    if (out_keys) {
        void* dst = k_host ? static_cast<void*>(e->stage_k) : out_keys;
        rc = gather_rows(e->k, e->prob_stride, e->n_prob, D, e->sel_idx, k, k, dst, s);
        if (rc) return rc;
        if (k_host) { host_io = true; DC_CUDA_TRY(cudaMemcpyAsync(out_keys, dst, rows * D * es, cudaMemcpyDeviceToHost, s)); }
    }
    if (out_vals) {
        void* dst = v_host ? static_cast<void*>(e->stage_v) : out_vals;
        rc = gather_rows(e->v, e->prob_stride, e->n_prob, D, e->sel_idx, k, k, dst, s);
        if (rc) return rc;
        if (v_host) { host_io = true; DC_CUDA_TRY(cudaMemcpyAsync(out_vals, dst, rows * D * es, cudaMemcpyDeviceToHost, s)); }
    }
    if (out_idx) {
        if (!is_device_ptr(out_idx)) host_io = true;
        DC_CUDA_TRY(cudaMemcpyAsync(out_idx, e->sel_idx, rows * sizeof(uint32_t), cudaMemcpyDefault, s));
    }
    if (out_bits) {
        if (!is_device_ptr(out_bits)) host_io = true;
        DC_CUDA_TRY(cudaMemcpyAsync(out_bits, e->sel_bits, rows * sizeof(uint32_t), cudaMemcpyDefault, s));
    }
    if (host_io) return check_status_word(e, s);
    return DC_OK;
}

int dc_get_keys(dc_engine* e, float* out) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(out != nullptr, "dc_get_keys: null out");
    if (e->ctx_len == 0) return DC_OK;
    const size_t n = static_cast<size_t>(e->n_prob) * e->ctx_len * e->head_dim;
    float* dst = out;
    float* tmp = nullptr;
    if (!is_device_ptr(out)) {
        DC_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&tmp), n * sizeof(float)));
        dst = tmp;
    }
    dim3 grid(256, e->n_prob);
    if (e->dtype == DC_BF16) keys_to_f32_kernel<DC_BF16><<<grid, 256>>>(e->k, e->prob_stride, e->ctx_len, e->head_dim, dst);
    else keys_to_f32_kernel<DC_FP16><<<grid, 256>>>(e->k, e->prob_stride, e->ctx_len, e->head_dim, dst);
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess && tmp) err = cudaMemcpy(out, tmp, n * sizeof(float), cudaMemcpyDeviceToHost);
    if (err == cudaSuccess) err = cudaDeviceSynchronize();
    if (tmp) cudaFree(tmp);
    if (err != cudaSuccess) return cuda_fail(err, "dc_get_keys");
    return DC_OK;
}

int dc_export_rows(dc_engine* e, void* keys_out, void* vals_out) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(keys_out && vals_out, "dc_export_rows: null pointer");
    if (e->ctx_len == 0) return DC_OK;
    const size_t row_bytes = static_cast<size_t>(e->ctx_len) * e->head_dim * sizeof(uint16_t);
    DC_CUDA_TRY(cudaMemcpy2D(keys_out, row_bytes, e->k, e->prob_stride * sizeof(uint16_t), row_bytes, e->n_prob,
                             cudaMemcpyDefault));
    DC_CUDA_TRY(cudaMemcpy2D(vals_out, row_bytes, e->v, e->prob_stride * sizeof(uint16_t), row_bytes, e->n_prob,
                             cudaMemcpyDefault));
    return DC_OK;
}

int dc_update_r_sq(dc_engine* e, const float* r_sq, int n) {
    DC_ENGINE_ENTER(e);
    (void)r_sq;
    DC_REQUIRE(n == e->kv_heads, "r_sq length must match kv_head_num");
    return DC_OK;
}

int dc_decode_attend(dc_engine* e, const void* q, const void* k_new, const void* v_new, void* res_k, void* res_v,
                     int64_t res_stride_b, int64_t res_stride_h, int res_len, int topk, float scale, void* out,
                     int32_t* out_idx, float* out_lse, uint64_t stream) {
    return dc_decode_attend_strided(e, q, 0, k_new, v_new, 0, res_k, res_v, res_stride_b, res_stride_h, res_len, topk,
                                    scale, out, out_idx, out_lse, stream);
}

int dc_decode_attend_strided(dc_engine* e, const void* q, int64_t q_stride_b, const void* k_new, const void* v_new,
                             int64_t new_stride_b, void* res_k, void* res_v, int64_t res_stride_b,
                             int64_t res_stride_h, int res_len, int topk, float scale, void* out, int32_t* out_idx,
                             float* out_lse, uint64_t stream) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(q && out, "dc_decode_attend: null q/out");
    DC_REQUIRE(q_stride_b >= 0 && new_stride_b >= 0 && q_stride_b % 8 == 0 && new_stride_b % 8 == 0,
               "dc_decode_attend: batch strides must be non-negative multiples of 8 elements");
    DC_REQUIRE(q_stride_b == 0 || q_stride_b >= static_cast<int64_t>(e->q_heads) * e->head_dim,
               "dc_decode_attend: q batch stride smaller than one batch of query heads");
    DC_REQUIRE(new_stride_b == 0 || new_stride_b >= static_cast<int64_t>(e->kv_heads) * e->head_dim,
               "dc_decode_attend: k_new/v_new batch stride smaller than one batch of kv heads");
    DC_REQUIRE(topk >= 0, "dc_decode_attend: negative topk");
    const int k = static_cast<int>(std::min<int64_t>(topk, e->ctx_len));
    DC_REQUIRE(k <= DC_MAX_TOPK, "dc_decode_attend: topk=%d exceeds DC_MAX_TOPK=%d", k, DC_MAX_TOPK);
    DC_REQUIRE(k + res_len + (k_new ? 1 : 0) >= 1, "dc_decode_attend: nothing to attend over");
    cudaStream_t s = as_stream(stream);
    int rc;
    cudaEvent_t* ev = nullptr;
    if (k > 0 && e->phase_count < e->phase_cap) ev = &e->phase_events[4 * e->phase_count];
    if (k > 0) {
        rc = scan_and_select(e, q, 1, k, 0u, e->sel_bits, e->sel_idx, s, ev, q_stride_b);
        if (rc) return rc;
    }
    const int32_t* sel_count = nullptr;
    if (k > 0 && e->budget_n > 0) {  // k-check epilogue of the select: rows beyond the budget are not attended
        rc = adaptive_budget(e->sel_bits, k, e->n_prob, k, e->head_dim, e->budget_seq, e->budget_n, e->budget_threshold,
                             e->budget, s);
        if (rc) return rc;
        sel_count = e->budget;
    }
    rc = sparse_attend(e->k, e->v, e->prob_stride, e->ctx_len, e->n_prob, e->kv_heads, e->group, e->head_dim, e->dtype,
                       q, e->sel_idx, k, k, 0, k_new, v_new, res_k, res_v, res_stride_b, res_stride_h, res_len, scale,
                       out, out_lse, nullptr, nullptr, e->att_scratch, s, sel_count, q_stride_b, new_stride_b);
    if (rc) return rc;
    if (ev) {
        DC_CUDA_TRY(cudaEventRecord(ev[3], s));
        e->phase_count += 1;
    }
    if (out_idx && k > 0)
        DC_CUDA_TRY(cudaMemcpyAsync(out_idx, e->sel_idx, static_cast<size_t>(e->n_prob) * k * sizeof(uint32_t),
                                    cudaMemcpyDeviceToDevice, s));
    return DC_OK;
}

int dc_set_adaptive_budget(dc_engine* e, const int32_t* k_check_seq, int n_seq, float attn_mass_threshold) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(n_seq >= 0 && n_seq <= 16, "dc_set_adaptive_budget: at most 16 checkpoints (got %d)", n_seq);
    DC_REQUIRE(n_seq == 0 || k_check_seq != nullptr, "dc_set_adaptive_budget: null k_check_seq");
    for (int i = 0; i < n_seq; i++) {
        DC_REQUIRE(k_check_seq[i] >= 1 && (i == 0 || k_check_seq[i] > k_check_seq[i - 1]),
                   "dc_set_adaptive_budget: k_check_seq must be positive and increasing");
        e->budget_seq[i] = k_check_seq[i];
    }
    e->budget_n = n_seq;
    e->budget_threshold = attn_mass_threshold;
    return DC_OK;
}

int dc_get_budget(dc_engine* e, int32_t* out, uint64_t stream) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(out != nullptr, "dc_get_budget: null out");
    DC_CUDA_TRY(cudaMemcpyAsync(out, e->budget, static_cast<size_t>(e->n_prob) * sizeof(int32_t), cudaMemcpyDefault,
                                as_stream(stream)));
    if (!is_device_ptr(out)) DC_CUDA_TRY(cudaStreamSynchronize(as_stream(stream)));
    return DC_OK;
}

int dc_adaptive_budget(const uint32_t* sel_bits, int64_t stride, int n_prob, int k, int head_dim,
                       const int32_t* k_check_seq, int n_seq, float attn_mass_threshold, int32_t* out_budget,
                       uint64_t stream) {
    return adaptive_budget(sel_bits, stride, n_prob, k, head_dim, k_check_seq, n_seq, attn_mass_threshold, out_budget,
                           as_stream(stream));
}

int dc_set_phase_timing(dc_engine* e, int max_steps) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(max_steps >= 0 && max_steps <= 100000, "dc_set_phase_timing: max_steps=%d", max_steps);
    while (static_cast<int>(e->phase_events.size()) < 4 * max_steps) {
        cudaEvent_t ev;
        DC_CUDA_TRY(cudaEventCreate(&ev));
        e->phase_events.push_back(ev);
    }
    e->phase_cap = max_steps;
    e->phase_count = 0;
    return DC_OK;
}

int dc_get_phase_times(dc_engine* e, float* scan_ms, float* select_ms, float* attend_ms, int* steps) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(scan_ms && select_ms && attend_ms && steps, "dc_get_phase_times: null pointer");
    *scan_ms = *select_ms = *attend_ms = 0.0f;
    *steps = e->phase_count;
    for (int i = 0; i < e->phase_count; i++) {
        cudaEvent_t* ev = &e->phase_events[4 * i];
        DC_CUDA_TRY(cudaEventSynchronize(ev[3]));
        float a = 0, b = 0, c = 0;
        DC_CUDA_TRY(cudaEventElapsedTime(&a, ev[0], ev[1]));
        DC_CUDA_TRY(cudaEventElapsedTime(&b, ev[1], ev[2]));
        DC_CUDA_TRY(cudaEventElapsedTime(&c, ev[2], ev[3]));
        *scan_ms += a; *select_ms += b; *attend_ms += c;
    }
    return DC_OK;
}

int dc_local_topk(dc_engine* e, const void* q, int topk, uint32_t* out_bits, uint32_t* out_gidx, uint64_t stream) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(q && out_bits && out_gidx, "dc_local_topk: null pointer");
    DC_REQUIRE(topk >= 1 && topk <= DC_MAX_TOPK, "dc_local_topk: topk=%d outside [1, %d]", topk, DC_MAX_TOPK);
    cudaStream_t s = as_stream(stream);
    if (e->ctx_len == 0) {
        DC_CUDA_TRY(cudaMemsetAsync(out_bits, 0xFF, static_cast<size_t>(e->n_prob) * topk * sizeof(uint32_t), s));
        DC_CUDA_TRY(cudaMemsetAsync(out_gidx, 0xFF, static_cast<size_t>(e->n_prob) * topk * sizeof(uint32_t), s));
        return DC_OK;
    }
    return scan_and_select(e, q, 1, topk, static_cast<uint32_t>(e->row_offset), out_bits, out_gidx, s);
}

int dc_attend_owned(dc_engine* e, const void* q, const uint32_t* sel_gidx, int n_sel, const void* k_new,
                    const void* v_new, void* res_k, void* res_v, int64_t res_stride_b, int64_t res_stride_h,
                    int res_len, float scale, float* out_acc, float* out_ml, const int32_t* sel_count,
                    uint64_t stream) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(q && out_acc && out_ml, "dc_attend_owned: null pointer");
    return sparse_attend(e->k, e->v, e->prob_stride, e->ctx_len, e->n_prob, e->kv_heads, e->group, e->head_dim,
                         e->dtype, q, sel_gidx, n_sel, n_sel, e->row_offset, k_new, v_new, res_k, res_v, res_stride_b,
                         res_stride_h, res_len, scale, nullptr, nullptr, out_acc, out_ml, e->att_scratch,
                         as_stream(stream), sel_count);
}

// ---- stateless kernels ----

int dc_score_scan(const void* keys, int64_t prob_stride, int n_prob, int64_t n, int head_dim, int dtype, const void* q,
                  int q_mode, int group, uint32_t* scores, int64_t score_stride, uint32_t* minmax, uint64_t stream) {
    return score_scan(keys, prob_stride, n_prob, n, head_dim, dtype, q, q_mode, group, scores, score_stride, minmax,
                      as_stream(stream));
}

int64_t dc_select_scratch_bytes(int n_prob) { return select_scratch_bytes(n_prob); }

int dc_merge_sorted_count(const uint32_t* bits_all, int world, int n_prob, int k, int my_rank, int32_t* out_count,
                          uint64_t stream) {
    return merge_sorted_count(bits_all, world, n_prob, k, my_rank, out_count, as_stream(stream));
}

int dc_topk_select(const uint32_t* bits, const uint32_t* ids, int64_t in_stride, int n_prob, int64_t n, int k,
                   const uint32_t* minmax, uint32_t* out_bits, uint32_t* out_ids, int64_t out_stride, void* scratch,
                   uint64_t stream) {
    DC_REQUIRE(scratch != nullptr, "dc_topk_select: null scratch");
    int rc = select_prepare();
    if (rc) return rc;
    return topk_select(bits, ids, in_stride, n_prob, n, k, minmax, 0u, out_bits, out_ids, out_stride,
                       static_cast<uint32_t*>(scratch), as_stream(stream));
}

int64_t dc_attend_scratch_bytes(int n_prob, int group, int head_dim) {
    return attend_scratch_bytes(n_prob, group, head_dim);
}

int dc_sparse_attend(const void* k_store, const void* v_store, int64_t prob_stride, int64_t n_rows, int n_prob,
                     int kv_heads, int group, int head_dim, int dtype, const void* q, const uint32_t* sel,
                     int64_t sel_stride, int n_sel, int64_t sel_base, const void* k_new, const void* v_new, void* res_k,
                     void* res_v, int64_t res_stride_b, int64_t res_stride_h, int res_len, float scale, void* out,
                     float* out_lse, float* out_acc, float* out_ml, void* scratch, uint64_t stream) {
    return sparse_attend(k_store, v_store, prob_stride, n_rows, n_prob, kv_heads, group, head_dim, dtype, q, sel,
                         sel_stride, n_sel, sel_base, k_new, v_new, res_k, res_v, res_stride_b, res_stride_h, res_len,
                         scale, out, out_lse, out_acc, out_ml, scratch, as_stream(stream));
}

int dc_lse_combine(const float* acc, int64_t acc_part_stride, const float* ml, int64_t ml_part_stride, int n_part,
                   int64_t rows, int head_dim, int dtype, void* out, float* out_lse, uint64_t stream) {
    DC_REQUIRE(out != nullptr, "dc_lse_combine: null out");
    DC_REQUIRE(acc_part_stride >= rows * head_dim && ml_part_stride >= rows * 2, "dc_lse_combine: part strides too small");
    return lse_combine(acc, acc_part_stride, head_dim, ml, ml_part_stride, 2, n_part, rows, head_dim, dtype, out,
                       out_lse, nullptr, nullptr, as_stream(stream));
}

int dc_gather_rows(const void* store, int64_t prob_stride, int n_prob, int head_dim, const uint32_t* ids,
                   int64_t ids_stride, int n_ids, void* out, uint64_t stream) {
    DC_REQUIRE(store && ids && out, "dc_gather_rows: null pointer");
    DC_REQUIRE(head_dim % 8 == 0 && head_dim >= 8 && head_dim <= 2048, "dc_gather_rows: head_dim %d", head_dim);
    DC_REQUIRE(n_prob >= 0 && n_prob <= 65535 && n_ids >= 0, "dc_gather_rows: bad sizes");
    return gather_rows(store, prob_stride, n_prob, head_dim, ids, ids_stride, n_ids, out, as_stream(stream));
}

int dc_pq_build_lut(const void* q, int q_mode, int group, int dtype, const float* centroids, int n_prob, int head_dim,
                    int n_sub, float* lut, uint64_t stream) {
    return pq_build_lut(q, q_mode, group, dtype, centroids, n_prob, head_dim, n_sub, lut, as_stream(stream));
}

int dc_pq_adc_scan(const uint8_t* codes, int64_t prob_stride, int n_prob, int64_t n, int n_sub, const float* lut,
                   uint32_t* scores, int64_t score_stride, uint32_t* minmax, uint64_t stream) {
    return pq_adc_scan(codes, prob_stride, n_prob, n, n_sub, lut, scores, score_stride, minmax, as_stream(stream));
}

int dc_rerank_scores(const void* keys, int64_t prob_stride, int n_prob, int head_dim, int dtype, const void* q,
                     int q_mode, int group, const uint32_t* ids, int64_t ids_stride, int n_ids, uint32_t* out_bits,
                     uint64_t stream) {
    return rerank_scores(keys, prob_stride, n_prob, head_dim, dtype, q, q_mode, group, ids, ids_stride, n_ids, out_bits,
                         as_stream(stream));
}

}  // extern "C"
