// Score scan on the 5th-generation tensor cores (tcgen05), selected with DC_SCAN_VARIANT=tcgen05.
//
// Same result as the kernels of scan.cu — the loop body of Index::search_bruteforce
// (diffcache_cpu/src/nsw.rs:601-607) with Index::distance QKDist (nsw.rs:129-139) — computed as a
// swapped-operand contraction: 128 key rows are the M dimension of one MMA tile, the query is the N
// dimension (16 columns, the minimum for M = 128; column 0 holds the group-mean query, the others are
// zero), head_dim = 128 is K:
//
//     S[128 keys x 16] = Ktile[128 x 128] . Qt[128 x 16]        fp32 accumulators in tensor memory
//
// Per (batch, kv head) the reference scores with ONE vector, so this is a GEMV dressed as a GEMM: 15 of
// the 16 columns are padding and the tensor pipe is nearly idle; the kernel exists to measure exactly
// that, and because it takes the multiply-adds off the CUDA cores.  Data movement is what matters:
//   * key tiles arrive by TMA (cp.async.bulk.tensor.2d, two 64-column boxes per 128-row tile, 128-byte
//     swizzle) into a ring of 32 KB shared-memory stages, each completing on an mbarrier;
//   * one elected thread issues eight tcgen05.mma (K = 16 each) per tile and commits them to two
//     mbarriers: "stage free" for the TMA producer and "accumulator ready" for the epilogue;
//   * four epilogue warps read column 0 of the accumulator (tcgen05.ld 32x32b: lane = key row), turn it
//     into the ranking key bits(65536 - dot) and write 128 consecutive keys per tile.  Accumulators are handed
//     over in pairs (two tiles per barrier round trip), four pairs rotate, and two groups of four epilogue warps
//     take alternate pairs: with one group reading one tile per round trip, the read-out (barrier wake-up,
//     tcgen05.ld, release) took about 1 us per tile and held the kernel at 4.9 TB/s whatever the number of
//     accumulators.
// Persistent CTAs (one per SM) each take a contiguous range of tiles.  Every mbarrier wait is bounded: a
// wait that runs out records 211..215 in the status word, the roles drain, tensor memory is freed and
// the kernel returns.  No multicast, one CTA per cluster.
//
// Arithmetic: the products of two 16-bit values are exact in fp32; the tensor core's fp32 accumulation
// order differs from the CUDA-core kernels', so ranking keys can differ from theirs in the last bit
// (within the one ulp of dist that the selection-parity rule allows), never more.
#include <cuda.h>

#include <cstring>

#include "common.cuh"

namespace dc {

namespace {

constexpr int kTcThreads = 384;                      // producer, MMA, allocator, query warps + two groups of 4 epilogue warps
constexpr int kTcStages = 5;
constexpr int kTileRows = 128;
constexpr int kTileDim = 128;
constexpr int kHalfBytes = kTileRows * 128;          // one 64-column box: 128 rows x 128 bytes
constexpr int kStageBytes = 2 * kHalfBytes;          // 32 KB
constexpr int kQTileBytes = 2 * 16 * 128;            // 16 rows x 128 dims, two 64-column halves
constexpr int kPairs = 4;                            // accumulator pairs in flight: a pair = two tiles, read out together
constexpr int kTmemCols = kPairs * 32;               // 16 fp32 columns per tile; a power of two >= 32
constexpr int kTcSmemBytes = kTcStages * kStageBytes + 2 * kQTileBytes + 1024;

__device__ __forceinline__ void mbar_arrive_plain(unsigned long long* bar) {
    asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.shared::cta.b64 st, [%0];\n}\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// Shared-memory matrix descriptor of a K-major operand stored as rows of 128 bytes with the 128-byte swizzle
// (what the TMA box above produces): start address, leading offset 1 (unused for swizzled K-major), 1024
// bytes between 8-row groups, descriptor version 1, layout type 2 = SWIZZLE_128B.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// Instruction descriptor of kind::f16: fp32 accumulate, A and B both K-major, 16-bit inputs of the given
// format (0 = f16, 1 = bf16), N = 16, M = 128.
__host__ __device__ constexpr uint32_t instr_desc(int fmt) {
    return (1u << 4) | (static_cast<uint32_t>(fmt) << 7) | (static_cast<uint32_t>(fmt) << 10) | ((16u >> 3) << 17) |
           ((128u >> 4) << 24);
}

struct TcShared {
    unsigned long long full[kTcStages], empty[kTcStages];
    unsigned long long acc_full[kPairs], acc_empty[kPairs];
    unsigned long long q_full[2], q_empty[2];
    uint32_t tmem_base;
    uint32_t s_lo, s_hi;
};

// grid = (#SMs).  Tile t of the launch covers rows [r0, r0 + 128) of problem t / tiles_per_prob.
template <int DT>
__global__ void __launch_bounds__(kTcThreads, 1)
score_scan_tc_kernel(const __grid_constant__ CUtensorMap kmap, int64_t rows_per_prob, int64_t n,
                     const int32_t* __restrict__ n_dev, int n_prob, const uint16_t* __restrict__ q, int q_mode, int group,
                     int kv_heads, int64_t q_stride_b, uint32_t* __restrict__ scores, int64_t score_stride,
                     uint32_t* __restrict__ minmax, uint32_t* __restrict__ status) {
    pdl_launch_dependents();
    pdl_wait();
    if (n_dev != nullptr) n = *n_dev;
    extern __shared__ unsigned char tc_smem_raw[];
    __shared__ TcShared sh;
    const uint32_t raw = smem_u32(tc_smem_raw);
    unsigned char* ring = tc_smem_raw + (((raw + 1023u) & ~1023u) - raw);   // 1024-byte aligned: the swizzle unit
    unsigned char* qtile = ring + kTcStages * kStageBytes;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int64_t tiles_per_prob = (n + kTileRows - 1) / kTileRows;
    const int64_t total = tiles_per_prob * n_prob;
    const int64_t t_begin = total * blockIdx.x / gridDim.x, t_end = total * (blockIdx.x + 1) / gridDim.x;
    const int64_t my_tiles = t_end - t_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTcStages; s++) { mbar_init(&sh.full[s], 1); mbar_init(&sh.empty[s], 1); }
        for (int a = 0; a < kPairs; a++) { mbar_init(&sh.acc_full[a], 1); mbar_init(&sh.acc_empty[a], 4); }
        for (int a = 0; a < 2; a++) { mbar_init(&sh.q_full[a], 1); mbar_init(&sh.q_empty[a], 1); }
        mbar_init_fence();
    }
    for (int i = threadIdx.x; i < 2 * kQTileBytes / 16; i += kTcThreads)   // rows 1..15 of both query tiles stay zero
        reinterpret_cast<uint4*>(qtile)[i] = make_uint4(0, 0, 0, 0);
    fence_proxy_async();   // the MMAs read these zeros through the async proxy
    if (warp == 2) {   // tensor-memory allocation is a warp-wide operation; this warp frees it at the end
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sh.tmem_base)), "n"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;

    if (warp == 0) {
        // ---- TMA producer ----
        if (lane == 0) {
            for (int64_t i = 0; i < my_tiles; i++) {
                const int s = static_cast<int>(i % kTcStages);
                if (i >= kTcStages && !mbar_wait_bounded(&sh.empty[s], static_cast<unsigned>((i / kTcStages - 1) & 1))) {
                    if (status) atomicMax(status, 211u);
                    break;
                }
                const int64_t t = t_begin + i;
                const int64_t p = t / tiles_per_prob, r0 = (t % tiles_per_prob) * kTileRows;
                const int y = static_cast<int>(p * rows_per_prob + r0);
                unsigned char* dst = ring + static_cast<size_t>(s) * kStageBytes;
                mbar_arrive_expect_tx(&sh.full[s], kStageBytes);
                tma_load_2d(dst, &kmap, 0, y, &sh.full[s]);                 // columns 0..63   (x * 2 bytes = 0)
                tma_load_2d(dst + kHalfBytes, &kmap, 64, y, &sh.full[s]);   // columns 64..127 (x * 2 bytes = 128)
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: one thread ----
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(DT == DC_BF16 ? 1 : 0);
            int64_t cur_p = -1, prob_ord = -1;
            for (int64_t i = 0; i < my_tiles; i++) {
                const int s = static_cast<int>(i % kTcStages);
                const int64_t pair = i / 2;                       // tiles 2*pair and 2*pair+1 share a read-out
                const int a = static_cast<int>(pair % kPairs);
                const int64_t t = t_begin + i, p = t / tiles_per_prob;
                bool ok = true;
                if (p != cur_p) {   // first tile of a problem in this CTA: its query tile must be ready
                    cur_p = p; prob_ord++;
                    ok = mbar_wait_bounded(&sh.q_full[prob_ord & 1], static_cast<unsigned>((prob_ord >> 1) & 1));
                    if (!ok && status) atomicMax(status, 212u);
                }
                if (ok && (i & 1) == 0 && pair >= kPairs) {
                    ok = mbar_wait_bounded(&sh.acc_empty[a], static_cast<unsigned>((pair / kPairs - 1) & 1));
                    if (!ok && status) atomicMax(status, 213u);
                }
                if (ok) {
                    ok = mbar_wait_bounded(&sh.full[s], static_cast<unsigned>((i / kTcStages) & 1));
                    if (!ok && status) atomicMax(status, 214u);
                }
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_base = smem_u32(ring + static_cast<size_t>(s) * kStageBytes);
                const uint32_t b_base = smem_u32(qtile + static_cast<size_t>(prob_ord & 1) * kQTileBytes);
#pragma unroll
                for (int k = 0; k < kTileDim / 16; k++) {
                    // k-step k covers dims [16k, 16k+16): half k/4 of the tile, 32 bytes into its 128-byte rows
                    const uint64_t ad = smem_desc_sw128(a_base + (k / 4) * kHalfBytes + (k % 4) * 32);
                    const uint64_t bd = smem_desc_sw128(b_base + (k / 4) * (kQTileBytes / 2) + (k % 4) * 32);
                    tc_mma_f16(tmem + static_cast<uint32_t>(a * 32 + (i & 1) * 16), ad, bd, idesc, k > 0 ? 1u : 0u);
                }
                tc_commit(&sh.empty[s]);       // the stage may be refilled once these MMAs have read it
                if ((i & 1) == 1 || i + 1 == my_tiles) tc_commit(&sh.acc_full[a]);    // ... and the pair is complete
                const bool last_of_prob = (i + 1 == my_tiles) || ((t + 1) / tiles_per_prob != p);
                if (last_of_prob) tc_commit(&sh.q_empty[prob_ord & 1]);
            }
        }
    } else if (warp == 3) {
        // ---- query tiles: row 0 of a 16 x 128 K-major tile = the group-mean query of the problem (16-byte
        // chunk c of row 0 sits at chunk c of its 128-byte row: the swizzle XORs with the row index, 0) ----
        int64_t first_p = my_tiles > 0 ? t_begin / tiles_per_prob : 0;
        int64_t last_p = my_tiles > 0 ? (t_end - 1) / tiles_per_prob : -1;
        for (int64_t p = first_p; p <= last_p; p++) {
            const int64_t ord = p - first_p;
            const int buf = static_cast<int>(ord & 1);
            bool ok = true;
            if (ord >= 2) ok = mbar_wait_bounded(&sh.q_empty[buf], static_cast<unsigned>((ord / 2 - 1) & 1));
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) { if (lane == 0 && status) atomicMax(status, 215u); break; }
            if (lane < kTileDim / 8) {
                float f[8];
                load_query8<DT>(query_base(q, p, kTileDim, q_mode, group, kv_heads, q_stride_b), kTileDim, q_mode, group, lane * 8, f);
                uint4 w;
                w.x = float_to_elem<DT>(f[0]) | (static_cast<uint32_t>(float_to_elem<DT>(f[1])) << 16);
                w.y = float_to_elem<DT>(f[2]) | (static_cast<uint32_t>(float_to_elem<DT>(f[3])) << 16);
                w.z = float_to_elem<DT>(f[4]) | (static_cast<uint32_t>(float_to_elem<DT>(f[5])) << 16);
                w.w = float_to_elem<DT>(f[6]) | (static_cast<uint32_t>(float_to_elem<DT>(f[7])) << 16);
                unsigned char* dst = qtile + static_cast<size_t>(buf) * kQTileBytes + (lane / 8) * (kQTileBytes / 2) + (lane % 8) * 16;
                *reinterpret_cast<uint4*>(dst) = w;
            }
            fence_proxy_async();   // the MMA reads shared memory through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive_plain(&sh.q_full[buf]);
        }
    } else if (warp >= 4) {
        // ---- epilogue: two groups of four warps take alternate accumulator pairs; warp w reads tensor-memory
        // lanes [32 (w % 4), +32) = key rows of the tile ----
        const int quarter = warp & 3;
        const int group_id = (warp - 4) >> 2;
        uint32_t lo = 0xFFFFFFFFu, hi = 0u;
        int64_t cur_p = -1;
        auto flush_minmax = [&]() {
            lo = __reduce_min_sync(0xFFFFFFFFu, lo);
            hi = __reduce_max_sync(0xFFFFFFFFu, hi);
            if (minmax != nullptr && lane == 0 && lo <= hi) {
                atomicMin(&minmax[2 * cur_p], lo);
                atomicMax(&minmax[2 * cur_p + 1], hi);
            }
            lo = 0xFFFFFFFFu; hi = 0u;
        };
        const int64_t n_pairs = (my_tiles + 1) / 2;
        for (int64_t pair = group_id; pair < n_pairs; pair += 2) {
            const int a = static_cast<int>(pair % kPairs);
            if (!__all_sync(0xFFFFFFFFu, mbar_wait_bounded(&sh.acc_full[a], static_cast<unsigned>((pair / kPairs) & 1)))) {
                if (lane == 0 && status) atomicMax(status, 216u);
                break;
            }
            tc_fence_after();
            const bool two = 2 * pair + 1 < my_tiles;
            uint32_t v[2] = {0u, 0u};
            const uint32_t taddr = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(a * 32);
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];\n" : "=r"(v[0]) : "r"(taddr) : "memory");
            if (two) asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];\n" : "=r"(v[1]) : "r"(taddr + 16u) : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_plain(&sh.acc_empty[a]);   // the pair may be overwritten
#pragma unroll
            for (int h = 0; h < 2; h++) {
                if (h == 1 && !two) break;
                const int64_t t = t_begin + 2 * pair + h, p = t / tiles_per_prob, r0 = (t % tiles_per_prob) * kTileRows;
                if (p != cur_p) {
                    if (cur_p >= 0) flush_minmax();
                    cur_p = p;
                }
                const int64_t r = r0 + quarter * 32 + lane;
                if (r < n) {
                    const uint32_t b = dist_bits(__uint_as_float(v[h]));
                    scores[p * score_stride + r] = b;
                    lo = min(lo, b);
                    hi = max(hi, b);
                }
            }
        }
        if (cur_p >= 0) flush_minmax();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "n"(kTmemCols) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

}  // namespace

// Returns DC_OK when the launch was made, DC_ESTATE when this variant does not apply (the caller then uses the
// default kernel), another code on a real failure.
int score_scan_tc(const void* keys, int64_t prob_stride, int n_prob, int64_t n, const int32_t* n_dev, int head_dim, int dtype,
                  const void* q, int q_mode, int group, int kv_heads, int64_t q_stride_b, uint32_t* scores,
                  int64_t score_stride, uint32_t* minmax, uint32_t* status, cudaStream_t stream) {
    if (head_dim != kTileDim || prob_stride % kTileDim != 0 || (reinterpret_cast<uintptr_t>(keys) & 127) != 0) return DC_ESTATE;
    EncodeTiledFn encode = encode_tiled_fn();
    if (encode == nullptr) return DC_ESTATE;
    const int64_t rows_per_prob = prob_stride / kTileDim;
    const int64_t rows_total = static_cast<int64_t>(n_prob - 1) * rows_per_prob + n;   // rows that exist; beyond: zero fill
    CUtensorMap map;
    std::memset(&map, 0, sizeof(map));
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(kTileDim), static_cast<cuuint64_t>(rows_total)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(kTileDim) * 2};
    const cuuint32_t box[2] = {64, kTileRows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = encode(&map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(keys), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) {
        set_error("score_scan_tc: cuTensorMapEncodeTiled failed with %d", static_cast<int>(cr));
        return DC_ECUDA;
    }
    static PerDeviceOnce once_bf16, once_fp16;
    PerDeviceOnce& once = dtype == DC_BF16 ? once_bf16 : once_fp16;
    int rc = once.run([dtype](int) {
        if (dtype == DC_BF16)
            DC_CUDA_TRY(cudaFuncSetAttribute(score_scan_tc_kernel<DC_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes));
        else
            DC_CUDA_TRY(cudaFuncSetAttribute(score_scan_tc_kernel<DC_FP16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes));
        return DC_OK;
    });
    if (rc != DC_OK) return rc;
    const dim3 grid(sm_count()), block(kTcThreads);
    if (dtype == DC_BF16)
        DC_CUDA_TRY(launch_chained(score_scan_tc_kernel<DC_BF16>, grid, block, kTcSmemBytes, stream, 0u, map, rows_per_prob, n,
                                   n_dev, n_prob, static_cast<const uint16_t*>(q), q_mode, group, kv_heads, q_stride_b, scores,
                                   score_stride, minmax, status));
    else
        DC_CUDA_TRY(launch_chained(score_scan_tc_kernel<DC_FP16>, grid, block, kTcSmemBytes, stream, 0u, map, rows_per_prob, n,
                                   n_dev, n_prob, static_cast<const uint16_t*>(q), q_mode, group, kv_heads, q_stride_b, scores,
                                   score_stride, minmax, status));
    return DC_OK;
}

}  // namespace dc
