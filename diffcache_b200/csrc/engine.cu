// Engine object and the extern "C" boundary (declared in include/diffcache_b200.h).
//
// dc_engine is the HBM-resident counterpart of DataLayer<bf16> + Index<T>
// (diffcache_cpu/src/lib.rs:189-197, diffcache_cpu/src/nsw.rs:47-56): it owns the key and
// value stores K,V[bsz*kv_heads][max_ctx_len][head_dim] and every scratch buffer a decode
// step needs, all allocated once in dc_create so that the per-step calls only enqueue
// kernels (they can be captured in a CUDA graph).
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "exchange.cuh"

namespace dc {

// ---- kernels defined in the other translation units ----
int score_scan(const void* keys, int64_t prob_stride, int n_prob, int64_t n, int head_dim, int dtype, const void* q,
               int q_mode, int group, uint32_t* scores, int64_t score_stride, uint32_t* minmax, cudaStream_t stream,
               uint32_t* status = nullptr, int kv_heads = 1, int64_t q_stride_b = 0, const int32_t* n_dev = nullptr);
int topk_select(const uint32_t* bits, const uint32_t* ids, int64_t in_stride, int n_prob, int64_t n, int k,
                const uint32_t* minmax, uint32_t id_offset, uint32_t* out_bits, uint32_t* out_ids, int64_t out_stride,
                uint32_t* status, cudaStream_t stream, uint32_t* minmax_reset = nullptr, const int32_t* n_dev = nullptr,
                const XchgOut* xout = nullptr);
int select_prepare();
int64_t select_scratch_bytes(int n_prob);
int merge_sorted_count(const uint32_t* bits_all, int world, int n_prob, int k, int my_rank, int32_t* out_count,
                       cudaStream_t stream, const XchgLL* ll = nullptr, int64_t rank_stride = 0);
int sparse_attend(const void* k_store, const void* v_store, int64_t prob_stride, int64_t n_rows, int n_prob,
                  int kv_heads, int group, int head_dim, int dtype, const void* q, const uint32_t* sel,
                  int64_t sel_stride, int n_sel, int64_t sel_base, const void* k_new, const void* v_new, void* res_k,
                  void* res_v, int64_t res_stride_b, int64_t res_stride_h, int res_len, float scale, void* out,
                  float* out_lse, float* out_acc, float* out_ml, void* scratch, cudaStream_t stream,
                  const int32_t* sel_count = nullptr, int64_t q_stride_b = 0, int64_t new_stride_b = 0,
                  const int32_t* n_rows_dev = nullptr, const int32_t* res_len_dev = nullptr, const XchgOut* xout = nullptr,
                  const XchgFinal* fin = nullptr);
int adaptive_budget(const uint32_t* bits, int64_t stride, int n_prob, int k, int head_dim, const int* seq, int n_seq,
                    float threshold, int32_t* budget, cudaStream_t stream, const int32_t* n_dev = nullptr);
int64_t attend_scratch_bytes(int n_prob, int group, int head_dim);
int lse_combine(const float* acc, int64_t acc_ps, int64_t acc_rs, const float* ml, int64_t ml_ps, int64_t ml_rs,
                int n_part, int64_t rows, int head_dim, int dtype, void* out, float* out_lse, float* out_acc,
                float* out_ml, cudaStream_t stream, const XchgLL* ll = nullptr, const XchgOut* xout = nullptr,
                const XchgFinal* fin = nullptr);
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

// DC_PDL: "0" = never, "1" (default) = for launches that go straight to a stream, "2" = also for
// launches that are being captured into a CUDA graph.  Measured on B200: between stream launches the
// early scheduling hides launch latency; between the kernel nodes of a replayed graph, whose plain
// edges already cost about a microsecond, programmatic edges were slower (37 -> 42 us on the
// four-kernel step of a batch-1, 32K-token problem).
bool pdl_enabled(cudaStream_t stream) {
    static const int mode = [] {
        const char* v = std::getenv("DC_PDL");
        if (v == nullptr || v[0] == 0) return 1;
        return v[0] == '0' ? 0 : v[0] == '2' ? 2 : 1;
    }();
    if (mode != 1) return mode == 2;
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &st) != cudaSuccess) { cudaGetLastError(); return false; }
    return st == cudaStreamCaptureStatusNone;
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

// ---- row counts kept on the device ----
// len[0] = valid rows per problem.  The host keeps a mirror for sizing launches, but kernels read this
// word when they run, so launches replayed from a CUDA graph follow a store that grows between replays.
__global__ void set_len_kernel(int32_t* len, int32_t value) { len[0] = value; }

// Index::insert (diffcache_cpu/src/nsw.rs:544-557) on device words: row len[0] of every problem <- keys/vals
// (n_prob, dim), then len[0] += 1.  One CTA, so that every thread sees the old length.
__global__ void __launch_bounds__(1024)
append_rows_kernel(const uint16_t* __restrict__ keys, const uint16_t* __restrict__ vals, int n_prob, int dim,
                   uint16_t* __restrict__ k_store, uint16_t* __restrict__ v_store, int64_t prob_stride, int64_t max_ctx,
                   int32_t* len, uint32_t* status) {
    const int lanes = dim / 8;
    const int64_t n = len[0];
    if (n >= max_ctx) {  // full: nothing is written (the host-side call reports DC_ESTATE when it can tell)
        if (threadIdx.x == 0 && status) atomicMax(status, 301u);
        return;
    }
    for (int i = threadIdx.x; i < n_prob * 2 * lanes; i += blockDim.x) {
        const int p = i / (2 * lanes), which = (i / lanes) & 1, c = i % lanes;
        const uint16_t* src = (which ? vals : keys) + static_cast<int64_t>(p) * dim + c * 8;
        uint16_t* dst = (which ? v_store : k_store) + p * prob_stride + n * dim + c * 8;
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
    }
    __syncthreads();
    if (threadIdx.x == 0) len[0] = static_cast<int32_t>(n + 1);
}

// Window ring of the resident buffer, all state in device words so that the whole decode loop can be one
// replayed graph per layer.  win = {suffix_len, head, prefix_len, cap, res_len_now, steps, -, -} (int32):
// the resident rows of a (batch, kv head) are [prefix_len sink rows | cap window slots].  While the window
// is not full the new token goes to slot suffix_len; once it is full the OLDEST token (slot head) is first
// moved into the scanned store (row len[0], len[0] += 1: what DataLayer::insert would do,
// diffcache_cpu/src/lib.rs:352-369) and the new token takes its slot, instead of the reference's
// `assert kvbuf_suffix_len < kvbuf_suffix_maxlen` (src/diffcache/kvcache/diffcache.py:221).  Attention does
// not depend on the order of its rows, so the ring needs no unrolling.  win[4] receives the number of
// resident rows the attention of this step covers.  One CTA.  win[0..3] are advanced once per decode
// step (not per layer) by window_advance_kernel.
__global__ void __launch_bounds__(1024)
window_push_kernel(const uint16_t* __restrict__ k_new, const uint16_t* __restrict__ v_new, int64_t new_stride_b,
                   uint16_t* __restrict__ res_k, uint16_t* __restrict__ res_v, int64_t res_stride_b, int64_t res_stride_h,
                   int n_prob, int kv_heads, int dim, uint16_t* __restrict__ k_store, uint16_t* __restrict__ v_store,
                   int64_t prob_stride, int64_t max_ctx, int32_t* len, int32_t* win, uint32_t* status) {
    pdl_launch_dependents();
    pdl_wait();
    const int lanes = dim / 8;
    const int suffix_len = win[0], head = win[1], prefix_len = win[2], cap = win[3];
    const int64_t n = len[0];
    const bool full = suffix_len >= cap;
    const bool spill = full && n < max_ctx;
    const int slot = full ? head : suffix_len;
    if (full && !spill && threadIdx.x == 0 && status) atomicMax(status, 302u);  // store full: the oldest token is dropped
    for (int i = threadIdx.x; i < n_prob * 2 * lanes; i += blockDim.x) {
        const int p = i / (2 * lanes), which = (i / lanes) & 1, c = i % lanes;
        const int b = p / kv_heads, h = p % kv_heads;
        uint16_t* row = (which ? res_v : res_k) + b * res_stride_b + h * res_stride_h +
                        static_cast<int64_t>(prefix_len + slot) * dim + c * 8;
        if (spill) {
            uint16_t* dst = (which ? v_store : k_store) + p * prob_stride + n * dim + c * 8;
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(row);
        }
        const int64_t off = new_stride_b ? b * new_stride_b + static_cast<int64_t>(h) * dim : static_cast<int64_t>(p) * dim;
        *reinterpret_cast<uint4*>(row) = *reinterpret_cast<const uint4*>((which ? v_new : k_new) + off + c * 8);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (spill) len[0] = static_cast<int32_t>(n + 1);
        win[4] = prefix_len + min(suffix_len + 1, cap);
    }
}

__global__ void window_advance_kernel(int32_t* win) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) {
        if (win[0] < win[3]) win[0] += 1;
        else win[1] = (win[1] + 1) % max(win[3], 1);
        win[5] += 1;
    }
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
    int64_t max_ctx = 0, row_offset = 0;
    int64_t ctx_len = 0;           // host mirror of len[0]; exact unless len_on_device
    bool len_on_device = false;    // a device-side spill (dc_window_push) may have advanced len[0] since the last read
    int32_t* len = nullptr;        // device words: len[0] = valid rows per problem
    uint16_t* ins_stage = nullptr; // staging for host-side dc_insert rows: 2 x (n_prob, D)
    // sequence-sharded step over a peer exchange (allocated by the first dc_sharded_local call)
    uint32_t* shard_bits = nullptr;   // (n_prob, shard_k) this rank's sorted candidate keys
    uint32_t* shard_gidx = nullptr;   // (n_prob, shard_k) their global row ids
    int32_t* shard_count = nullptr;   // (n_prob) length of the globally winning prefix
    float* shard_part = nullptr;      // [acc (rows, D) | ml (rows, 2)] partial attention of this rank
    int shard_k = 0;
    dc_xchg* out_xchg = nullptr;      // dc_set_output_exchange: decode steps also fan their output slice out to it
    int out_xchg_channel = 0;
    void* out_dense = nullptr;         // dc_set_output_gather: where the step's last kernel unpacks all ranks' slices
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
    std::vector<cudaEvent_t> trace_events;  // dc_trace_begin / dc_trace_read: one event after every kernel of a step
    int trace_cap = 0, trace_n = 0;
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
// Rows per problem a launch on `s` must be sized for.  Kernels read the exact count from e->len when they
// run; the host mirror is exact for launches that execute once, but a launch captured into a graph is
// replayed later, when rows may have been appended, so it is sized for the whole store, and so is every
// launch after a device-side spill (whose count only the device knows).
int rows_bound(dc_engine* e, cudaStream_t s, int64_t* out) {
    *out = e->ctx_len;
    if (e->len_on_device) { *out = e->max_ctx; return DC_OK; }
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    DC_CUDA_TRY(cudaStreamIsCapturing(s, &st));
    if (st != cudaStreamCaptureStatusNone) *out = e->max_ctx;
    return DC_OK;
}

// Exact row count on the host: the mirror, refreshed from the device word after device-side spills
// (synchronises `s`; not usable while `s` is being captured).
int host_ctx_len(dc_engine* e, cudaStream_t s, int64_t* out) {
    if (e->len_on_device) {
        int32_t v = 0;
        DC_CUDA_TRY(cudaMemcpyAsync(&v, e->len, sizeof(v), cudaMemcpyDeviceToHost, s));
        DC_CUDA_TRY(cudaStreamSynchronize(s));
        e->ctx_len = v;
    }
    *out = e->ctx_len;
    return DC_OK;
}

// Records the next trace event on `s` while a trace is open (dc_trace_begin); does nothing otherwise.
int trace_mark(dc_engine* e, cudaStream_t s) {
    if (e->trace_n < e->trace_cap) {
        DC_CUDA_TRY(cudaEventRecord(e->trace_events[e->trace_n], s));
        e->trace_n += 1;
    }
    return DC_OK;
}

int scan_and_select(dc_engine* e, const void* q, int q_mode, int k, int64_t n_bound, uint32_t id_offset,
                    uint32_t* out_bits, uint32_t* out_ids, cudaStream_t s, cudaEvent_t* ev = nullptr,
                    int64_t q_stride_b = 0, const XchgOut* xout = nullptr) {
    // e->minmax is in its initial state here: set once in dc_create, and put back by every select
    if (ev) DC_CUDA_TRY(cudaEventRecord(ev[0], s));
    trace_mark(e, s);
    int rc = score_scan(e->k, e->prob_stride, e->n_prob, n_bound, e->head_dim, e->dtype, q, q_mode, e->group, e->scores,
                        e->score_stride, e->minmax, s, e->status, e->kv_heads, q_stride_b, e->len);
    if (rc) return rc;
    if (ev) DC_CUDA_TRY(cudaEventRecord(ev[1], s));
    trace_mark(e, s);
    rc = topk_select(e->scores, nullptr, e->score_stride, e->n_prob, n_bound, k, e->minmax, id_offset, out_bits,
                     out_ids, k, e->status, s, e->minmax, e->len, xout);
    if (rc) return rc;
    if (ev) DC_CUDA_TRY(cudaEventRecord(ev[2], s));
    trace_mark(e, s);
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

int decode_attend_impl(dc_engine* e, const void* q, int64_t q_stride_b, const void* k_new, const void* v_new,
                       int64_t new_stride_b, void* res_k, void* res_v, int64_t res_stride_b, int64_t res_stride_h,
                       int res_len, const int32_t* res_len_dev, int topk, float scale, void* out, int32_t* out_idx,
                       float* out_lse, cudaStream_t s);

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
    alloc(reinterpret_cast<void**>(&e->len), 256);
    alloc(reinterpret_cast<void**>(&e->ins_stage), 2 * static_cast<size_t>(e->n_prob) * head_dim * sizeof(uint16_t));
    if (err == cudaSuccess) err = cudaMemset(e->len, 0, 256);
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
    cudaFree(e->stage_k); cudaFree(e->stage_v); cudaFree(e->len); cudaFree(e->ins_stage);
    cudaFree(e->shard_bits); cudaFree(e->shard_gidx); cudaFree(e->shard_count); cudaFree(e->shard_part);
    for (cudaEvent_t ev : e->phase_events) cudaEventDestroy(ev);
    for (cudaEvent_t ev : e->trace_events) cudaEventDestroy(ev);
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
    set_len_kernel<<<1, 1, 0, s>>>(e->len, static_cast<int32_t>(seq_len));
    DC_CUDA_TRY(cudaGetLastError());
    e->ctx_len = seq_len;
    e->len_on_device = false;
    if (!is_device_ptr(keys) || !is_device_ptr(vals)) DC_CUDA_TRY(cudaStreamSynchronize(s));
    return DC_OK;
}

int dc_insert(dc_engine* e, const void* keys, const void* vals, uint64_t stream) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(keys && vals, "dc_insert: null keys/vals");
    cudaStream_t s = as_stream(stream);
    // the row lands at the position the DEVICE length word holds when the copy runs, so an insert captured
    // into a graph appends at the right place on every replay; the host mirror only feeds the full check
    if (!e->len_on_device && e->ctx_len >= e->max_ctx) {
        set_error("dc_insert: store is full (max_ctx_len=%lld)", static_cast<long long>(e->max_ctx));
        return DC_ESTATE;
    }
    const bool host_src = !is_device_ptr(keys) || !is_device_ptr(vals);
    const uint16_t* kd = static_cast<const uint16_t*>(keys);
    const uint16_t* vd = static_cast<const uint16_t*>(vals);
    if (host_src) {
        const size_t bytes = static_cast<size_t>(e->n_prob) * e->head_dim * sizeof(uint16_t);
        DC_CUDA_TRY(cudaMemcpyAsync(e->ins_stage, keys, bytes, cudaMemcpyDefault, s));
        DC_CUDA_TRY(cudaMemcpyAsync(e->ins_stage + static_cast<size_t>(e->n_prob) * e->head_dim, vals, bytes,
                                    cudaMemcpyDefault, s));
        kd = e->ins_stage;
        vd = e->ins_stage + static_cast<size_t>(e->n_prob) * e->head_dim;
    }
    DC_REQUIRE(((reinterpret_cast<uintptr_t>(kd) | reinterpret_cast<uintptr_t>(vd)) & 15) == 0,
               "dc_insert: keys/vals must be 16-byte aligned");
    append_rows_kernel<<<1, 1024, 0, s>>>(kd, vd, e->n_prob, e->head_dim, e->k, e->v, e->prob_stride, e->max_ctx, e->len,
                                          e->status);
    DC_CUDA_TRY(cudaGetLastError());
    if (e->ctx_len < e->max_ctx) e->ctx_len += 1;
    if (host_src) DC_CUDA_TRY(cudaStreamSynchronize(s));
    return DC_OK;
}

int dc_ctx_len(dc_engine* e, int64_t* out) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(out != nullptr, "dc_ctx_len: null out");
    return host_ctx_len(e, nullptr, out);
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
    cudaStream_t s = as_stream(stream);
    int64_t ctx = 0;
    int rc0 = host_ctx_len(e, s, &ctx);
    if (rc0) return rc0;
    const int k = static_cast<int>(std::min<int64_t>(ef, ctx));  // lib.rs:374
    DC_REQUIRE(k <= DC_MAX_TOPK, "dc_query: ef=%d exceeds DC_MAX_TOPK=%d", k, DC_MAX_TOPK);
    if (k == 0) return DC_OK;
    const int D = e->head_dim;
    const size_t es = sizeof(uint16_t);
    bool host_io = false;

    const void* q_dev = q_mean;
    if (!is_device_ptr(q_mean)) {
        host_io = true;
        DC_CUDA_TRY(cudaMemcpyAsync(e->q_dev, q_mean, static_cast<size_t>(e->n_prob) * D * es, cudaMemcpyHostToDevice, s));
        q_dev = e->q_dev;
    }
    int rc = scan_and_select(e, q_dev, 0, k, ctx, 0u, e->sel_bits, e->sel_idx, s);
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
    int64_t ctx = 0;
    int rc = host_ctx_len(e, nullptr, &ctx);
    if (rc) return rc;
    if (ctx == 0) return DC_OK;
    const size_t per_prob = static_cast<size_t>(ctx) * e->head_dim;
    auto convert = [&](int p0, int np, float* dst) {
        dim3 grid(256, np);
        const uint16_t* src = e->k + static_cast<int64_t>(p0) * e->prob_stride;
        if (e->dtype == DC_BF16) keys_to_f32_kernel<DC_BF16><<<grid, 256>>>(src, e->prob_stride, ctx, e->head_dim, dst);
        else keys_to_f32_kernel<DC_FP16><<<grid, 256>>>(src, e->prob_stride, ctx, e->head_dim, dst);
        return cudaGetLastError();
    };
    cudaError_t err = cudaSuccess;
    if (is_device_ptr(out)) {
        err = convert(0, e->n_prob, out);
    } else {
        // host destination: converted a few problems at a time through a bounded device buffer (<= 64 MB),
        // not through an fp32 copy of the whole store
        const int chunk = static_cast<int>(std::max<size_t>(1, std::min<size_t>(e->n_prob, (64u << 20) / (per_prob * sizeof(float)))));
        float* tmp = nullptr;
        DC_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&tmp), chunk * per_prob * sizeof(float)));
        for (int p0 = 0; p0 < e->n_prob && err == cudaSuccess; p0 += chunk) {
            const int np = std::min(chunk, e->n_prob - p0);
            err = convert(p0, np, tmp);
            if (err == cudaSuccess)
                err = cudaMemcpy(out + static_cast<size_t>(p0) * per_prob, tmp, np * per_prob * sizeof(float), cudaMemcpyDeviceToHost);
        }
        cudaFree(tmp);
    }
    if (err == cudaSuccess) err = cudaDeviceSynchronize();
    if (err != cudaSuccess) return cuda_fail(err, "dc_get_keys");
    return DC_OK;
}

int dc_export_rows(dc_engine* e, void* keys_out, void* vals_out) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(keys_out && vals_out, "dc_export_rows: null pointer");
    int64_t ctx = 0;
    int rc = host_ctx_len(e, nullptr, &ctx);
    if (rc) return rc;
    if (ctx == 0) return DC_OK;
    const size_t row_bytes = static_cast<size_t>(ctx) * e->head_dim * sizeof(uint16_t);
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
    cudaStream_t s = as_stream(stream);
    return decode_attend_impl(e, q, q_stride_b, k_new, v_new, new_stride_b, res_k, res_v, res_stride_b, res_stride_h,
                              res_len, nullptr, topk, scale, out, out_idx, out_lse, s);
}

}  // extern "C"

namespace {

// Shared by dc_decode_attend[_strided] (res_len known to the host, new token appended by the attention
// kernel) and dc_decode_attend_dyn (res_len_dev != NULL: the resident length is a device word, res_len its
// upper bound, the new token already sits in the window).
int decode_attend_impl(dc_engine* e, const void* q, int64_t q_stride_b, const void* k_new, const void* v_new,
                       int64_t new_stride_b, void* res_k, void* res_v, int64_t res_stride_b, int64_t res_stride_h,
                       int res_len, const int32_t* res_len_dev, int topk, float scale, void* out, int32_t* out_idx,
                       float* out_lse, cudaStream_t s) {
    int64_t bound = 0;
    int rc = rows_bound(e, s, &bound);
    if (rc) return rc;
    // Rows the store can hold when the launches run; the kernels clamp to the rows it does hold (pads in the
    // selection are skipped by the attention).
    const int k = static_cast<int>(std::min<int64_t>(topk, bound));
    DC_REQUIRE(k <= DC_MAX_TOPK, "dc_decode_attend: topk=%d exceeds DC_MAX_TOPK=%d", k, DC_MAX_TOPK);
    DC_REQUIRE(k + res_len + (k_new ? 1 : 0) >= 1, "dc_decode_attend: nothing to attend over");
    cudaEvent_t* ev = nullptr;
    if (k > 0 && e->phase_count < e->phase_cap) ev = &e->phase_events[4 * e->phase_count];
    if (k > 0) {
        rc = scan_and_select(e, q, 1, k, bound, 0u, e->sel_bits, e->sel_idx, s, ev, q_stride_b);
        if (rc) return rc;
    }
    const int32_t* sel_count = nullptr;
    if (k > 0 && e->budget_n > 0) {  // k-check epilogue of the select: rows beyond the budget are not attended
        rc = adaptive_budget(e->sel_bits, k, e->n_prob, k, e->head_dim, e->budget_seq, e->budget_n, e->budget_threshold,
                             e->budget, s, e->len);
        if (rc) return rc;
        sel_count = e->budget;
    }
    XchgOut xo;
    const XchgOut* xout = nullptr;
    XchgFinal fin;
    const XchgFinal* finp = nullptr;
    if (e->out_xchg != nullptr) {   // head-sharded layer: (bsz, q_heads, D) becomes (bsz, world, q_heads * D) on every rank
        xo = xchg_out_args(e->out_xchg, e->out_xchg_channel);
        const int64_t slice_words = static_cast<int64_t>(e->q_heads) * e->head_dim / 2;
        xo.rows_per_block = e->q_heads;
        xo.block_stride = xchg_world(e->out_xchg) * slice_words;
        xo.rank_off = xchg_rank(e->out_xchg) * slice_words;
        xo.row_words = e->head_dim / 2;
        xout = &xo;
        if (e->out_dense != nullptr) {   // the merge kernel also waits for all ranks' slices and unpacks them
            fin.ll = xchg_ll_args(e->out_xchg, e->out_xchg_channel);
            fin.out = e->out_dense;
            fin.out_lse = nullptr;
            finp = &fin;
        }
    }
    rc = sparse_attend(e->k, e->v, e->prob_stride, bound, e->n_prob, e->kv_heads, e->group, e->head_dim, e->dtype,
                       q, e->sel_idx, k, k, 0, k_new, v_new, res_k, res_v, res_stride_b, res_stride_h, res_len, scale,
                       out, out_lse, nullptr, nullptr, e->att_scratch, s, sel_count, q_stride_b, new_stride_b, e->len,
                       res_len_dev, xout, finp);
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

}  // namespace

extern "C" {

int dc_window_push(dc_engine* e, const void* k_new, const void* v_new, int64_t new_stride_b, void* res_k, void* res_v,
                   int64_t res_stride_b, int64_t res_stride_h, int32_t* window_state, uint64_t stream) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(k_new && v_new && res_k && res_v && window_state, "dc_window_push: null pointer");
    DC_REQUIRE(new_stride_b >= 0 && new_stride_b % 8 == 0 && res_stride_b % 8 == 0 && res_stride_h % 8 == 0,
               "dc_window_push: strides must be non-negative multiples of 8 elements");
    DC_REQUIRE(((reinterpret_cast<uintptr_t>(k_new) | reinterpret_cast<uintptr_t>(v_new) |
                 reinterpret_cast<uintptr_t>(res_k) | reinterpret_cast<uintptr_t>(res_v)) & 15) == 0,
               "dc_window_push: every row pointer must be 16-byte aligned");
    DC_REQUIRE(is_device_ptr(k_new) && is_device_ptr(v_new) && is_device_ptr(window_state),
               "dc_window_push: device pointers only");
    cudaStream_t s = as_stream(stream);
    e->len_on_device = true;  // from here on only the device knows how many rows the store holds
    DC_CUDA_TRY(launch_chained(window_push_kernel, dim3(1), dim3(1024), 0, s, 0u, static_cast<const uint16_t*>(k_new),
                               static_cast<const uint16_t*>(v_new), new_stride_b, static_cast<uint16_t*>(res_k),
                               static_cast<uint16_t*>(res_v), res_stride_b, res_stride_h, e->n_prob, e->kv_heads,
                               e->head_dim, e->k, e->v, e->prob_stride, e->max_ctx, e->len, window_state, e->status));
    return DC_OK;
}

int dc_window_advance(int32_t* window_state, uint64_t stream) {
    DC_REQUIRE(window_state != nullptr, "dc_window_advance: null pointer");
    DC_CUDA_TRY(launch_chained(window_advance_kernel, dim3(1), dim3(32), 0, as_stream(stream), 0u, window_state));
    return DC_OK;
}

int dc_decode_attend_dyn(dc_engine* e, const void* q, int64_t q_stride_b, void* res_k, void* res_v,
                         int64_t res_stride_b, int64_t res_stride_h, const int32_t* res_len_dev, int res_cap, int topk,
                         float scale, void* out, int32_t* out_idx, float* out_lse, uint64_t stream) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(q && out && res_k && res_v && res_len_dev, "dc_decode_attend_dyn: null pointer");
    DC_REQUIRE(q_stride_b >= 0 && q_stride_b % 8 == 0, "dc_decode_attend_dyn: q batch stride must be a multiple of 8 elements");
    DC_REQUIRE(q_stride_b == 0 || q_stride_b >= static_cast<int64_t>(e->q_heads) * e->head_dim,
               "dc_decode_attend_dyn: q batch stride smaller than one batch of query heads");
    DC_REQUIRE(res_cap >= 1 && topk >= 0, "dc_decode_attend_dyn: res_cap=%d topk=%d", res_cap, topk);
    return decode_attend_impl(e, q, q_stride_b, nullptr, nullptr, 0, res_k, res_v, res_stride_b, res_stride_h, res_cap,
                              res_len_dev, topk, scale, out, out_idx, out_lse, as_stream(stream));
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
                           as_stream(stream), nullptr);
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

int dc_trace_begin(dc_engine* e, int max_marks) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(max_marks >= 0 && max_marks <= 4096, "dc_trace_begin: max_marks=%d", max_marks);
    while (static_cast<int>(e->trace_events.size()) < max_marks) {
        cudaEvent_t ev;
        DC_CUDA_TRY(cudaEventCreate(&ev));
        e->trace_events.push_back(ev);
    }
    e->trace_cap = max_marks;
    e->trace_n = 0;
    return DC_OK;
}

int dc_trace_read(dc_engine* e, float* intervals_ms, int* n_marks) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(intervals_ms && n_marks, "dc_trace_read: null pointer");
    *n_marks = e->trace_n;
    e->trace_cap = 0;  // closes the trace
    if (e->trace_n == 0) return DC_OK;
    DC_CUDA_TRY(cudaEventSynchronize(e->trace_events[e->trace_n - 1]));
    for (int i = 0; i + 1 < e->trace_n; i++)
        DC_CUDA_TRY(cudaEventElapsedTime(&intervals_ms[i], e->trace_events[i], e->trace_events[i + 1]));
    return DC_OK;
}

static int local_topk_impl(dc_engine* e, const void* q, int topk, uint32_t* out_bits, uint32_t* out_gidx, uint64_t stream,
                          const XchgOut* xout, bool* fanned_out);

int dc_local_topk(dc_engine* e, const void* q, int topk, uint32_t* out_bits, uint32_t* out_gidx, uint64_t stream) {
    return local_topk_impl(e, q, topk, out_bits, out_gidx, stream, nullptr, nullptr);
}

// xout: also store the keys into every rank's exchange buffer; *fanned_out tells whether that happened (it does
// not when this engine holds no rows: the pads are then written by a memset, which cannot fan out).
static int local_topk_impl(dc_engine* e, const void* q, int topk, uint32_t* out_bits, uint32_t* out_gidx, uint64_t stream,
                          const XchgOut* xout, bool* fanned_out) {
    DC_ENGINE_ENTER(e);
    if (fanned_out) *fanned_out = false;
    DC_REQUIRE(q && out_bits && out_gidx, "dc_local_topk: null pointer");
    DC_REQUIRE(topk >= 1 && topk <= DC_MAX_TOPK, "dc_local_topk: topk=%d outside [1, %d]", topk, DC_MAX_TOPK);
    cudaStream_t s = as_stream(stream);
    int64_t bound = 0;
    int rc = rows_bound(e, s, &bound);
    if (rc) return rc;
    if (bound == 0) {
        DC_CUDA_TRY(cudaMemsetAsync(out_bits, 0xFF, static_cast<size_t>(e->n_prob) * topk * sizeof(uint32_t), s));
        DC_CUDA_TRY(cudaMemsetAsync(out_gidx, 0xFF, static_cast<size_t>(e->n_prob) * topk * sizeof(uint32_t), s));
        return DC_OK;
    }
    if (fanned_out) *fanned_out = xout != nullptr;
    return scan_and_select(e, q, 1, topk, bound, static_cast<uint32_t>(e->row_offset), out_bits, out_gidx, s, nullptr, 0, xout);
}

static int attend_owned_impl(dc_engine* e, const void* q, const uint32_t* sel_gidx, int n_sel, const void* k_new,
                            const void* v_new, void* res_k, void* res_v, int64_t res_stride_b, int64_t res_stride_h,
                            int res_len, float scale, float* out_acc, float* out_ml, const int32_t* sel_count,
                            uint64_t stream, const XchgOut* xout, const XchgFinal* fin = nullptr);

int dc_attend_owned(dc_engine* e, const void* q, const uint32_t* sel_gidx, int n_sel, const void* k_new,
                    const void* v_new, void* res_k, void* res_v, int64_t res_stride_b, int64_t res_stride_h,
                    int res_len, float scale, float* out_acc, float* out_ml, const int32_t* sel_count,
                    uint64_t stream) {
    return attend_owned_impl(e, q, sel_gidx, n_sel, k_new, v_new, res_k, res_v, res_stride_b, res_stride_h, res_len, scale,
                             out_acc, out_ml, sel_count, stream, nullptr);
}

static int attend_owned_impl(dc_engine* e, const void* q, const uint32_t* sel_gidx, int n_sel, const void* k_new,
                            const void* v_new, void* res_k, void* res_v, int64_t res_stride_b, int64_t res_stride_h,
                            int res_len, float scale, float* out_acc, float* out_ml, const int32_t* sel_count,
                            uint64_t stream, const XchgOut* xout, const XchgFinal* fin) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(q && out_acc && out_ml, "dc_attend_owned: null pointer");
    int64_t bound = 0;
    int rc = rows_bound(e, as_stream(stream), &bound);
    if (rc) return rc;
    return sparse_attend(e->k, e->v, e->prob_stride, bound, e->n_prob, e->kv_heads, e->group, e->head_dim,
                         e->dtype, q, sel_gidx, n_sel, n_sel, e->row_offset, k_new, v_new, res_k, res_v, res_stride_b,
                         res_stride_h, res_len, scale, nullptr, nullptr, out_acc, out_ml, e->att_scratch,
                         as_stream(stream), sel_count, 0, 0, e->len, nullptr, xout, fin);
}

// ---- sequence-sharded step with the two exchanges done by peer stores (exchange.cu) ----

// DC_XCHG_FUSED=0 keeps the exchange stores in separate copy kernels (for comparison); default: fused into the
// kernels that produce the values.
static bool fused_push() {
    static const bool on = [] {
        const char* v = std::getenv("DC_XCHG_FUSED");
        return !(v != nullptr && v[0] == '0');
    }();
    return on;
}

int dc_set_output_exchange(dc_engine* e, dc_xchg* x, int channel) {
    DC_ENGINE_ENTER(e);
    if (x != nullptr) {
        DC_REQUIRE(channel >= 0 && channel < kXchgChannels, "dc_set_output_exchange: channel %d", channel);
        DC_REQUIRE(xchg_slot_bytes(x, channel) == static_cast<int64_t>(e->bsz) * e->q_heads * e->head_dim * 2,
                   "dc_set_output_exchange: the channel's slot (%lld bytes) is not one (bsz, q_heads, head_dim) output slice",
                   static_cast<long long>(xchg_slot_bytes(x, channel)));
        DC_REQUIRE(e->head_dim % 4 == 0, "dc_set_output_exchange: head_dim");
        DC_REQUIRE(xchg_ready(x), "dc_set_output_exchange: not every peer buffer is mapped yet");
    }
    e->out_xchg = x;
    e->out_xchg_channel = channel;
    if (x == nullptr) e->out_dense = nullptr;
    return DC_OK;
}

int dc_set_output_gather(dc_engine* e, void* dense) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(dense == nullptr || e->out_xchg != nullptr, "dc_set_output_gather: dc_set_output_exchange comes first");
    DC_REQUIRE(dense == nullptr || (is_device_ptr(dense) && (reinterpret_cast<uintptr_t>(dense) & 15) == 0),
               "dc_set_output_gather: a 16-byte aligned device pointer is needed");
    e->out_dense = dense;
    return DC_OK;
}

static int64_t shard_part_bytes(const dc_engine* e) {
    const int64_t rows = static_cast<int64_t>(e->n_prob) * e->group;
    return (rows * (e->head_dim + 2) * static_cast<int64_t>(sizeof(float)) + 15) / 16 * 16;
}

int dc_sharded_slot_bytes(dc_engine* e, int topk, int64_t* out2) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(out2 != nullptr && topk >= 1 && topk <= DC_MAX_TOPK, "dc_sharded_slot_bytes: bad arguments");
    out2[0] = static_cast<int64_t>(e->n_prob) * topk * static_cast<int64_t>(sizeof(uint32_t));
    out2[0] = (out2[0] + 15) / 16 * 16;
    out2[1] = shard_part_bytes(e);
    return DC_OK;
}

int dc_sharded_local(dc_engine* e, dc_xchg* x, const void* q, int topk, uint64_t stream) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(x != nullptr && q != nullptr, "dc_sharded_local: null pointer");
    DC_REQUIRE(topk >= 2 && topk <= DC_MAX_TOPK && topk % 2 == 0, "dc_sharded_local: topk=%d must be even, in [2, %d]", topk,
               DC_MAX_TOPK);
    DC_REQUIRE(static_cast<int64_t>(xchg_world(x)) * topk * 4 <= 200 * 1024,
               "dc_sharded_local: world*topk=%lld keys do not fit the prefix-count kernel (200 KB of shared memory)",
               static_cast<long long>(xchg_world(x)) * topk);
    int64_t need[2];
    need[0] = (static_cast<int64_t>(e->n_prob) * topk * 4 + 15) / 16 * 16;
    need[1] = shard_part_bytes(e);
    DC_REQUIRE(xchg_slot_bytes(x, 0) >= need[0] && xchg_slot_bytes(x, 1) >= need[1],
               "dc_sharded_local: exchange slots (%lld, %lld bytes) are smaller than this step needs (%lld, %lld)",
               static_cast<long long>(xchg_slot_bytes(x, 0)), static_cast<long long>(xchg_slot_bytes(x, 1)),
               static_cast<long long>(need[0]), static_cast<long long>(need[1]));
    cudaStream_t s = as_stream(stream);
    if (e->shard_k != topk) {  // first call (or a new k): not a stream operation, so not inside a capture
        cudaFree(e->shard_bits); cudaFree(e->shard_gidx); cudaFree(e->shard_count); cudaFree(e->shard_part);
        e->shard_bits = e->shard_gidx = nullptr; e->shard_count = nullptr; e->shard_part = nullptr; e->shard_k = 0;
        DC_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&e->shard_bits), need[0]));
        DC_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&e->shard_gidx), need[0]));
        DC_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&e->shard_count), static_cast<size_t>(e->n_prob) * sizeof(int32_t) + 16));
        DC_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&e->shard_part), need[1]));
        DC_CUDA_TRY(cudaMemset(e->shard_part, 0, need[1]));
        e->shard_k = topk;
    }
    // the select writes the sorted keys into every rank's buffer itself; only an engine without rows (pads
    // written by a memset) needs the separate push
    const XchgOut xo = xchg_out_args(x, 0);
    bool fanned = false;
    int rc = local_topk_impl(e, q, topk, e->shard_bits, e->shard_gidx, stream, fused_push() ? &xo : nullptr, &fanned);
    if (rc) return rc;
    if (!fanned) {
        rc = dc_xchg_push(x, 0, e->shard_bits, need[0], stream);
        if (rc) return rc;
    }
    return trace_mark(e, s);
}

// fin (may be NULL): the split merge also does the final merge of all ranks' partials (one launch fewer); only for
// steps whose ranks run on different GPUs, since the kernel then waits for blocks the other ranks' kernels send
static int sharded_attend_impl(dc_engine* e, dc_xchg* x, const void* q, const void* k_new, const void* v_new, void* res_k,
                               void* res_v, int64_t res_stride_b, int64_t res_stride_h, int res_len, float scale,
                               uint64_t stream, const XchgFinal* fin) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(x != nullptr && q != nullptr, "dc_sharded_attend: null pointer");
    DC_REQUIRE(e->shard_k > 0, "dc_sharded_attend: dc_sharded_local has not run");
    cudaStream_t s = as_stream(stream);
    const int k = e->shard_k;
    const XchgLL w0 = xchg_ll_args(x, 0);
    int rc = merge_sorted_count(nullptr, xchg_world(x), e->n_prob, k, xchg_rank(x), e->shard_count, s, &w0, 0);
    if (rc) return rc;
    trace_mark(e, s);
    const int64_t rows = static_cast<int64_t>(e->n_prob) * e->group;
    // the split merge writes (acc, m, l) into every rank's buffer itself
    XchgOut xo = xchg_out_args(x, 1);
    xo.row_words = e->head_dim;
    rc = attend_owned_impl(e, q, e->shard_gidx, k, k_new, v_new, res_k, res_v, res_stride_b, res_stride_h, res_len, scale,
                           e->shard_part, e->shard_part + rows * e->head_dim, e->shard_count, stream,
                           fused_push() ? &xo : nullptr, fused_push() ? fin : nullptr);
    if (rc) return rc;
    trace_mark(e, s);
    if (!fused_push()) {
        rc = dc_xchg_push(x, 1, e->shard_part, shard_part_bytes(e), stream);
        if (rc) return rc;
    }
    return trace_mark(e, s);
}

int dc_sharded_attend(dc_engine* e, dc_xchg* x, const void* q, const void* k_new, const void* v_new, void* res_k,
                      void* res_v, int64_t res_stride_b, int64_t res_stride_h, int res_len, float scale, uint64_t stream) {
    return sharded_attend_impl(e, x, q, k_new, v_new, res_k, res_v, res_stride_b, res_stride_h, res_len, scale, stream,
                               nullptr);
}

int dc_sharded_combine(dc_engine* e, dc_xchg* x, void* out, float* out_lse, uint64_t stream) {
    DC_ENGINE_ENTER(e);
    DC_REQUIRE(x != nullptr && out != nullptr, "dc_sharded_combine: null pointer");
    const int64_t rows = static_cast<int64_t>(e->n_prob) * e->group;
    const XchgLL w1 = xchg_ll_args(x, 1);
    int rc = lse_combine(nullptr, 0, 0, nullptr, 0, 0, xchg_world(x), rows, e->head_dim, e->dtype, out, out_lse, nullptr,
                         nullptr, as_stream(stream), &w1);
    if (rc) return rc;
    return trace_mark(e, as_stream(stream));
}

int dc_sharded_decode_attend(dc_engine* e, dc_xchg* x, const void* q, const void* k_new, const void* v_new, void* res_k,
                             void* res_v, int64_t res_stride_b, int64_t res_stride_h, int res_len, int topk, float scale,
                             void* out, float* out_lse, uint64_t stream) {
    int rc = dc_sharded_local(e, x, q, topk, stream);
    if (rc) return rc;
    // All three phases in one call means the ranks run concurrently on their own GPUs, so the split merge may
    // wait for the other ranks' partials itself and write the final output (DC_XCHG_FUSED=0: separate kernels).
    static const bool fuse_final = [] {   // DC_XCHG_FUSED_FINAL=0: the final merge stays a kernel of its own
        const char* v = std::getenv("DC_XCHG_FUSED_FINAL");
        return !(v != nullptr && v[0] == '0');
    }();
    if (fuse_final && fused_push() && e != nullptr && x != nullptr && out != nullptr && e->trace_cap == 0) {
        XchgFinal fin;
        fin.ll = xchg_ll_args(x, 1);
        fin.out = out;
        fin.out_lse = out_lse;
        return sharded_attend_impl(e, x, q, k_new, v_new, res_k, res_v, res_stride_b, res_stride_h, res_len, scale, stream,
                                   &fin);
    }
    rc = dc_sharded_attend(e, x, q, k_new, v_new, res_k, res_v, res_stride_b, res_stride_h, res_len, scale, stream);
    if (rc) return rc;
    return dc_sharded_combine(e, x, out, out_lse, stream);
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
