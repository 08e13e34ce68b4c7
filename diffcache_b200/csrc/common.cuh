// Shared device/host helpers for the diffcache_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "../../include/diffcache_b200.h"

namespace dc {

// ---- error reporting across the C ABI -------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t err, const char* what);

#define DC_CUDA_TRY(expr)                                  \
    do {                                                   \
        cudaError_t _e = (expr);                           \
        if (_e != cudaSuccess) return dc::cuda_fail(_e, #expr); \
    } while (0)

#define DC_REQUIRE(cond, ...)            \
    do {                                 \
        if (!(cond)) {                   \
            dc::set_error(__VA_ARGS__);  \
            return DC_EINVAL;            \
        }                                \
    } while (0)

inline cudaStream_t as_stream(uint64_t s) { return reinterpret_cast<cudaStream_t>(s); }

int sm_count();  // SMs of the current device (cached per device)

// Runs a set-up step once per CUDA device (kernel attribute opt-ins, symbol address look-ups): the
// first caller on a device does the work under a lock, later callers only read an atomic flag, so
// first calls from several host threads do not race.  A step that fails is tried again next time.
struct PerDeviceOnce {
    static constexpr int kMaxDevices = 64;
    std::mutex mu;
    std::atomic<bool> done[kMaxDevices];
    PerDeviceOnce() { for (auto& d : done) d.store(false, std::memory_order_relaxed); }
    template <class F>
    int run(F&& step) {
        int dev = 0;
        cudaError_t err = cudaGetDevice(&dev);
        if (err != cudaSuccess) return cuda_fail(err, "cudaGetDevice");
        const bool tracked = dev >= 0 && dev < kMaxDevices;
        if (tracked && done[dev].load(std::memory_order_acquire)) return DC_OK;
        std::lock_guard<std::mutex> lock(mu);
        if (tracked && done[dev].load(std::memory_order_relaxed)) return DC_OK;
        const int rc = step(dev);
        if (rc == DC_OK && tracked) done[dev].store(true, std::memory_order_release);
        return rc;
    }
};

// ---- programmatic dependent launch --------------------------------------------------------------
// The kernels of a decode step run back to back on one stream, each consuming what the one before it
// wrote.  Launched with cudaLaunchAttributeProgrammaticStreamSerialization, a kernel may be scheduled
// while its predecessor is still draining: every kernel here first lets ITS successor be scheduled
// (pdl_launch_dependents), does the set-up that touches no global data, and then blocks in pdl_wait
// until the predecessor grid has completed and its writes are visible.  Both instructions do nothing
// in a kernel that was launched the ordinary way.  Every kernel of the chain executes pdl_wait, so
// "kernel N finished" still implies "kernels 1..N-1 finished".
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

// Whether a launch on `stream` gets the attribute: not while the stream is being captured into a graph
// (see the definition), never when the environment variable DC_PDL is "0".
bool pdl_enabled(cudaStream_t stream);

// cudaLaunchKernelEx with the programmatic-serialization attribute (and a cluster size when cluster_x > 0).
template <class... KArgs, class... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  unsigned cluster_x, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    unsigned n_attr = 0;
    if (pdl_enabled(stream)) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        n_attr++;
    }
    if (cluster_x > 0) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = cluster_x;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        n_attr++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- element-type helpers -------------------------------------------------------------------
// Unpack eight 16-bit elements held in a uint4 into fp32.
template <int DT>
__device__ __forceinline__ void unpack8(const uint4& w, float (&f)[8]);

template <>
__device__ __forceinline__ void unpack8<DC_BF16>(const uint4& w, float (&f)[8]) {
    // bf16 -> fp32 is a 16-bit shift: low element by shifting up, high element by masking.
    f[0] = __uint_as_float(w.x << 16);
    f[1] = __uint_as_float(w.x & 0xFFFF0000u);
    f[2] = __uint_as_float(w.y << 16);
    f[3] = __uint_as_float(w.y & 0xFFFF0000u);
    f[4] = __uint_as_float(w.z << 16);
    f[5] = __uint_as_float(w.z & 0xFFFF0000u);
    f[6] = __uint_as_float(w.w << 16);
    f[7] = __uint_as_float(w.w & 0xFFFF0000u);
}

template <>
__device__ __forceinline__ void unpack8<DC_FP16>(const uint4& w, float (&f)[8]) {
    float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w.x));
    float2 b = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
    float2 c = __half22float2(*reinterpret_cast<const __half2*>(&w.z));
    float2 d = __half22float2(*reinterpret_cast<const __half2*>(&w.w));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
    f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

template <int DT>
__device__ __forceinline__ float elem_to_float(uint16_t h) {
    if (DT == DC_BF16) return __uint_as_float(static_cast<uint32_t>(h) << 16);
    return __half2float(__ushort_as_half(h));
}

template <int DT>
__device__ __forceinline__ uint16_t float_to_elem(float f) {  // round to nearest even
    if (DT == DC_BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(f));
    return __half_as_ushort(__float2half_rn(f));
}

// Streaming 16-byte load: the key/value stores are read once per step, so they should
// not displace the (re-read) score and candidate buffers from L1/L2.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    return __ldcs(reinterpret_cast<const uint4*>(p));
}

// Streaming 32-byte load (sm_100 has 256-bit global loads): half the load instructions and L1/L2
// requests per byte of a 16-byte load; read-only path, no L1 allocation, evict-first in L2.
struct Wide32 { uint4 lo, hi; };
__device__ __forceinline__ Wide32 ld_stream32(const void* p) {
    unsigned long long a, b, c, d;
    asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.v4.b64 {%0,%1,%2,%3}, [%4];\n"
                 : "=l"(a), "=l"(b), "=l"(c), "=l"(d) : "l"(p));
    Wide32 w;
    w.lo = make_uint4(static_cast<uint32_t>(a), static_cast<uint32_t>(a >> 32), static_cast<uint32_t>(b),
                      static_cast<uint32_t>(b >> 32));
    w.hi = make_uint4(static_cast<uint32_t>(c), static_cast<uint32_t>(c >> 32), static_cast<uint32_t>(d),
                      static_cast<uint32_t>(d >> 32));
    return w;
}

// Eight query elements [col0, col0+8) of the retrieval query of one problem as fp32.
// Where the query rows of problem `prob` (= batch * kv_heads + kv head) start.
// q_mode 0: q holds one group-mean row per problem, densely.  q_mode 1: q holds the `group` query heads of
// every problem back to back; q_stride_b == 0 means the batches are dense too ((n_prob*group, dim)),
// otherwise q_stride_b elements separate two batches (a slice of a fused q/k/v projection output).
__device__ __forceinline__ const uint16_t* query_base(const uint16_t* q, int64_t prob, int dim, int q_mode, int group,
                                                     int kv_heads, int64_t q_stride_b) {
    if (q_mode == 0) return q + prob * dim;
    if (q_stride_b == 0) return q + prob * group * dim;
    return q + (prob / kv_heads) * q_stride_b + (prob % kv_heads) * group * dim;
}

// q_mode 0: qbase already holds the group mean.  q_mode 1: qbase holds the `group` query heads of
// the problem back to back; the mean is the fp32 sum in head order times 1/group, rounded
// once to the element type (what torch's mean over a bf16 tensor produces).
template <int DT>
__device__ __forceinline__ void load_query8(const uint16_t* qbase, int dim, int q_mode, int group, int col0,
                                            float (&out)[8]) {
    if (q_mode == 0) {
        uint4 w = *reinterpret_cast<const uint4*>(qbase + col0);
        unpack8<DT>(w, out);
    } else {
        float s[8];
#pragma unroll
        for (int j = 0; j < 8; j++) s[j] = 0.0f;
        for (int g = 0; g < group; g++) {
            uint4 w = *reinterpret_cast<const uint4*>(qbase + g * dim + col0);
            float f[8];
            unpack8<DT>(w, f);
#pragma unroll
            for (int j = 0; j < 8; j++) s[j] += f[j];
        }
        float inv = 1.0f / static_cast<float>(group);
#pragma unroll
        for (int j = 0; j < 8; j++) out[j] = elem_to_float<DT>(float_to_elem<DT>(s[j] * inv));
    }
}


// Transposing butterfly reduction.  Every lane holds NV partial values; the LPR lanes
// that share a row (consecutive lanes, LPR a power of two) must be summed.  Instead of NV
// full butterflies (NV*log2(LPR) shuffles) each exchange step halves the number of live
// values per lane (lanes in the upper half of the exchange keep the upper half of the
// values), so the cost is NV-1 shuffles while values remain, then plain butterfly steps.
// Afterwards lane `l` holds treduce_count<NV,LPR>() fully reduced values v[0..count) whose
// original indices start at treduce_base<NV,LPR>(l); lanes that differ only in the low
// treduce_plain_bits<NV,LPR>() bits of their position hold identical copies.
template <int NV, int LPR>
__device__ __forceinline__ void treduce(float (&v)[NV], int lane) {
    constexpr unsigned kFull = 0xFFFFFFFFu;
    int nv = NV;
#pragma unroll
    for (int off = LPR / 2; off >= 1; off >>= 1) {
        if (nv > 1) {
            const int half = nv / 2;
            const bool up = (lane & off) != 0;
#pragma unroll
            for (int j = 0; j < NV / 2; j++) {
                if (j < half) {
                    float send = up ? v[j] : v[j + half];
                    float keep = up ? v[j + half] : v[j];
                    v[j] = keep + __shfl_xor_sync(kFull, send, off);
                }
            }
            nv = half;
        } else {
            v[0] += __shfl_xor_sync(kFull, v[0], off);
        }
    }
}

__host__ __device__ constexpr int ilog2(int x) { return x <= 1 ? 0 : 1 + ilog2(x / 2); }

template <int NV, int LPR>
__host__ __device__ constexpr int treduce_count() { return NV >= LPR ? NV / LPR : 1; }

template <int NV, int LPR>
__host__ __device__ constexpr int treduce_plain_bits() { return NV >= LPR ? 0 : ilog2(LPR) - ilog2(NV); }

template <int NV, int LPR>
__device__ __forceinline__ int treduce_base(int lane) {
    int base = 0, half = NV / 2;
#pragma unroll
    for (int off = LPR / 2; off >= 1; off >>= 1) {
        if (half >= 1) {
            if (lane & off) base += half;
            half /= 2;
        }
    }
    return base;
}


// ---- asynchronous bulk copies (TMA engine, untiled form) completing on a shared-memory mbarrier ----
__device__ __forceinline__ unsigned smem_u32(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n}\n"
                 ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after kMbarSpinLimit polls (each poll itself blocks for a hardware-defined
// time slice), so a copy that never completes cannot hang the GPU; the caller reports the failure.
constexpr int kMbarSpinLimit = 1 << 20;
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* bar, unsigned parity) {
    for (int i = 0; i < kMbarSpinLimit; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// One thread copies `bytes` (a multiple of 16; both addresses 16-byte aligned) global -> shared;
// completion is signalled on `bar` as `bytes` transaction bytes.
__device__ __forceinline__ void bulk_copy_g2s(void* smem_dst, const void* gmem_src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Orders this thread's earlier generic-proxy shared-memory accesses before later async-proxy ones.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// Ranking key of the reference: raw bits of fp32 (65536 - dot).
__device__ __forceinline__ uint32_t dist_bits(float dot) { return __float_as_uint(65536.0f - dot); }

}  // namespace dc
