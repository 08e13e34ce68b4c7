// Sparse gather-attention with split-K and log-sum-exp merge.
//
// Replaces, for one decode step, the gather loop of Index::search_bruteforce
// (diffcache_cpu/src/nsw.rs:623-629), the host->device copy of the gathered rows
// (src/diffcache/kvcache/diffcache.py:196-209) and flash_attn_with_kvcache over
// [retrieved | prefix | suffix | new token] (src/diffcache/base.py:134-142).
// The selected rows are read in place from the HBM store: every row is one contiguous
// 2*head_dim-byte segment copied asynchronously (16 bytes per lane) into a shared-memory ring,
// all query heads of the kv head are served from the same copy with tensor-core MMAs, and the
// row list of a problem is split over several CTAs whose (max, sum, accumulator) partials are
// merged by log-sum-exp in a second small kernel.
#include <cmath>
#include <cstdlib>

#include "exchange.cuh"

namespace dc {

namespace {

constexpr int kAttThreads = 128;
constexpr int kAttWarps = kAttThreads / 32;
constexpr float kLog2e = 1.4426950408889634f;

struct AttendArgs {
    const uint16_t* k_store;
    const uint16_t* v_store;
    int64_t prob_stride;   // elements between problems in the store
    int64_t n_rows;        // valid rows per problem in the store
    int kv_heads;
    int group;             // query heads per kv head
    const uint16_t* q;     // (n_prob*group, D), or batches q_stride_b elements apart when q_stride_b != 0
    int64_t q_stride_b;
    int64_t new_stride_b;  // k_new / v_new: 0 = dense (n_prob, D), else elements between batches
    const uint32_t* sel;   // (n_prob, sel_stride) row ids, or nullptr
    int64_t sel_stride;
    int n_sel;
    int64_t sel_base;      // id - sel_base = local row; ids outside [0, n_rows) are skipped
    const int32_t* sel_count;  // optional per-problem budget: only the first sel_count[p] ids are attended
    const uint16_t* k_new; // (n_prob, D) or nullptr
    const uint16_t* v_new;
    uint16_t* res_k;       // resident rows
    uint16_t* res_v;
    int64_t res_stride_b, res_stride_h;
    int res_len;
    const int32_t* n_rows_dev;   // optional device words overriding n_rows / res_len when the kernel runs
    const int32_t* res_len_dev;  // (launches replayed from a graph while the lengths change)
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

// ---- warp-level tensor-core primitives (m16n8k16, fp32 accumulate) ----
// Only rows 0..7 of the 16-row A/C tiles are used (query heads of one kv head), so the A registers of
// rows 8..15 are zero and the matching accumulator halves are discarded.
template <int DT>
__device__ __forceinline__ void mma_16816(float& d0, float& d1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    float z2, z3;
    if (DT == DC_BF16) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%10,%10};\n"
            : "+f"(d0), "+f"(d1), "=f"(z2), "=f"(z3)
            : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(0.0f));
    } else {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%10,%10};\n"
            : "+f"(d0), "+f"(d1), "=f"(z2), "=f"(z3)
            : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(0.0f));
    }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// Two fp32 values -> packed 16-bit pair (first value in the low half) plus the packed rounding
// residue, so that hi + lo reproduces the fp32 values to ~2^-17 when both feed the MMA.
template <int DT>
__device__ __forceinline__ void pack_hi_lo(float x, float y, uint32_t& hi, uint32_t& lo) {
    if (DT == DC_BF16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
        float2 hf = __bfloat1622float2(h);
        __nv_bfloat162 l = __floats2bfloat162_rn(x - hf.x, y - hf.y);
        hi = *reinterpret_cast<uint32_t*>(&h);
        lo = *reinterpret_cast<uint32_t*>(&l);
    } else {
        __half2 h = __floats2half2_rn(x, y);
        float2 hf = __half22float2(h);
        __half2 l = __floats2half2_rn(x - hf.x, y - hf.y);
        hi = *reinterpret_cast<uint32_t*>(&h);
        lo = *reinterpret_cast<uint32_t*>(&l);
    }
}

constexpr int kHeadsPerCta = 8;   // query heads of one kv head handled by one CTA (rows 0..7 of the MMA tile)

// Per head_dim: rows per tile and ring depth.  A tile is kAttWarps x 16 x RB rows; every warp owns
// 16*RB rows of it for BOTH Q.K^T and P.V (split-K across warps, merged once at the end), so the
// main loop needs no block barrier except the hand-over of ring slots.
template <int LPR> struct AttCfg;
template <> struct AttCfg<8>  { static constexpr int RB = 2; static constexpr int NS = 3; };  // D = 64:  128-row tiles, 32 KB
template <> struct AttCfg<16> { static constexpr int RB = 1; static constexpr int NS = 2; };  // D = 128:  64-row tiles, 32 KB
template <> struct AttCfg<32> { static constexpr int RB = 1; static constexpr int NS = 3; };  // D = 256:  64-row tiles, 64 KB

template <int LPR>
constexpr size_t att_smem_bytes() {
    return static_cast<size_t>(AttCfg<LPR>::NS) * 2 * (kAttWarps * 16 * AttCfg<LPR>::RB) * (LPR * 8) * sizeof(uint16_t);
}

// Byte offset of 16-byte chunk `chunk` of row `row` inside a [rows][D] tile: the chunk index is XORed
// with the low row bits so that the 8 rows of an ldmatrix 8x8 block fall into 8 different bank groups.
template <int D>
__device__ __forceinline__ int swz(int row, int chunk) { return row * (D * 2) + ((chunk ^ (row & 7)) << 4); }

// grid = (n_split, n_prob, ceil(group / 8)).
//
// The rows of a split are processed in tiles staged through a ring of shared-memory buffers filled
// with asynchronous 16-byte copies issued NS-1 tiles ahead (row ids are fetched one iteration before
// that), so bytes in flight are set by shared memory, not registers.  Q.K^T and P.V run on the tensor
// cores: K rows are the "col-major" B operand of S = Q.K^T as they lie in memory, V rows become the B
// operand of O = P.V through ldmatrix.trans, and the S accumulator fragments are re-used in place as
// the A fragments of P (split into a 16-bit value and its rounding residue so that P keeps ~17 bits).
template <int DT, int LPR>
__global__ void __launch_bounds__(kAttThreads)
sparse_attend_kernel(const AttendArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t n_rows = a.n_rows_dev != nullptr ? static_cast<int64_t>(*a.n_rows_dev) : a.n_rows;
    const int res_len = a.res_len_dev != nullptr ? *a.res_len_dev : a.res_len;
    constexpr int D = LPR * 8;
    constexpr int RB = AttCfg<LPR>::RB;
    constexpr int NS = AttCfg<LPR>::NS;
    constexpr int RW = 16 * RB;                 // rows per warp per tile
    constexpr int TILE = kAttWarps * RW;        // rows per CTA tile
    constexpr int R = 32 / LPR;                 // rows covered by one warp-wide copy instruction
    constexpr int NCOPY = RW / R;               // copy instructions per lane per tile and tensor
    constexpr int STAGE_BYTES = 2 * TILE * D * 2;
    constexpr int KSTEPS = D / 16;
    constexpr int NT = D / 8;                   // 8-column output tiles

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int col = lane % LPR, sub = lane / LPR;
    const int gq = lane >> 2, tq = lane & 3;    // MMA fragment coordinates: row (head) and column pair
    const int64_t prob = blockIdx.y;
    const int split = blockIdx.x;
    const int g0 = blockIdx.z * kHeadsPerCta;   // first query head of this chunk
    const int n_heads = min(kHeadsPerCta, a.group - g0);
    const int b = static_cast<int>(prob / a.kv_heads), h = static_cast<int>(prob % a.kv_heads);

    extern __shared__ __align__(128) unsigned char att_smem[];
    __shared__ unsigned char s_valid[NS][TILE];
    __shared__ float s_ml[kAttWarps][kHeadsPerCta][2];

    const int has_new = a.k_new != nullptr ? 1 : 0;
    const int64_t new_off = a.new_stride_b ? b * a.new_stride_b + static_cast<int64_t>(h) * D : prob * D;
    const int total = a.n_sel + res_len + has_new;
    const int per = (total + a.n_split - 1) / a.n_split;
    const int j0 = min(total, split * per);
    const int j1 = min(total, j0 + per);
    const int n_tiles = (j1 - j0 + TILE - 1) / TILE;

    // A fragments of Q for every k-step: rows = heads of this chunk (zero beyond), raw 16-bit pairs
    uint32_t qa[KSTEPS][2];
    {
        const uint16_t* qrow = a.q_stride_b ? a.q + b * a.q_stride_b + (static_cast<int64_t>(h) * a.group + g0 + gq) * D
                                            : a.q + (prob * a.group + g0 + gq) * D;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
            qa[ks][0] = gq < n_heads ? *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * tq) : 0u;
            qa[ks][1] = gq < n_heads ? *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * tq + 8) : 0u;
        }
    }

    const uint16_t* kst = a.k_store + prob * a.prob_stride;
    const uint16_t* vst = a.v_store + prob * a.prob_stride;
    uint16_t* rk = a.res_k ? a.res_k + b * a.res_stride_b + h * a.res_stride_h : nullptr;
    uint16_t* rv = a.res_v ? a.res_v + b * a.res_stride_b + h * a.res_stride_h : nullptr;
    const uint32_t* selp = a.sel ? a.sel + prob * a.sel_stride : nullptr;
    const int n_sel_eff = a.sel_count ? min(a.n_sel, a.sel_count[prob]) : a.n_sel;  // rows beyond it are skipped

    // flash-attn's in-place append of the new token (base.py:134-142): one CTA per problem
    if (has_new && split == 0 && blockIdx.z == 0 && rk != nullptr && tid < LPR) {
        reinterpret_cast<uint4*>(rk + static_cast<int64_t>(res_len) * D)[tid] =
            reinterpret_cast<const uint4*>(a.k_new + new_off)[tid];
        reinterpret_cast<uint4*>(rv + static_cast<int64_t>(res_len) * D)[tid] =
            reinterpret_cast<const uint4*>(a.v_new + new_off)[tid];
    }

    // Row id of ONE of the NCOPY rows this lane group copies in tile `t`: lane `col` (< NCOPY) of a group
    // holds the id of row i = col; the copy loop fetches it with a shuffle (0xFFFFFFFF where the slot is
    // not a store row).  One global load per lane and tile instead of NCOPY.
    auto fetch_id = [&](int t) -> uint32_t {
        const int j = j0 + t * TILE + warp * RW + col * R + sub;
        return (col < NCOPY && t < n_tiles && j < j1 && j < n_sel_eff) ? selp[j] : 0xFFFFFFFFu;
    };
    // Issue the copies of tile `t` into its ring slot (one commit group per call, possibly empty).
    // Fast path: every row of the tile is a selected store row, so a row address is one multiply-add
    // from its id and the V address is the K address plus a constant.
    int soff[NCOPY];  // swizzled byte offset of this lane's chunk of each of its rows inside a K (or V) tile
#pragma unroll
    for (int i = 0; i < NCOPY; i++) soff[i] = swz<D>(warp * RW + i * R + sub, col);
    const uint16_t* kst_col = kst + col * 8;
    const int64_t v_minus_k = vst - kst;  // elements
    auto issue_tile = [&](int t, uint32_t my_id) {
        if (t < n_tiles) {
            unsigned char* ks = att_smem + (t % NS) * STAGE_BYTES;
            unsigned char* vs = ks + TILE * D * 2;
            const int jt = j0 + t * TILE;
            if (jt + TILE <= min(j1, a.n_sel)) {
#pragma unroll
                for (int i = 0; i < NCOPY; i++) {
                    const uint32_t id = __shfl_sync(0xFFFFFFFFu, my_id, sub * LPR + i);
                    const int64_t row = static_cast<int64_t>(id) - a.sel_base;
                    const bool ok = row >= 0 && row < n_rows;  // ids of other shards and pads are skipped
                    const uint16_t* kp = ok ? kst_col + row * D : a.q;
                    cp_async16(ks + soff[i], kp, ok ? 16 : 0);
                    cp_async16(vs + soff[i], ok ? kp + v_minus_k : a.q, ok ? 16 : 0);
                    if (col == 0) s_valid[t % NS][warp * RW + i * R + sub] = ok ? 1 : 0;
                }
            } else if (jt >= a.n_sel && jt + TILE <= min(j1, a.n_sel + res_len)) {
                // a tile of resident (sink / window) rows: consecutive rows of the caller's buffer
                const uint16_t* kp0 = rk + static_cast<int64_t>(jt - a.n_sel + warp * RW + sub) * D + col * 8;
                const int64_t rv_minus_rk = rv - rk;
#pragma unroll
                for (int i = 0; i < NCOPY; i++) {
                    const uint16_t* kp = kp0 + i * R * D;
                    cp_async16(ks + soff[i], kp, 16);
                    cp_async16(vs + soff[i], kp + rv_minus_rk, 16);
                    if (col == 0) s_valid[t % NS][warp * RW + i * R + sub] = 1;
                }
            } else {
#pragma unroll
                for (int i = 0; i < NCOPY; i++) {
                    const int r = warp * RW + i * R + sub;
                    const int j = jt + r;
                    const uint16_t* kp = nullptr;
                    const uint16_t* vp = nullptr;
                    const uint32_t id = __shfl_sync(0xFFFFFFFFu, my_id, sub * LPR + i);
                    if (j < j1) {
                        if (j < a.n_sel) {
                            const int64_t row = static_cast<int64_t>(id) - a.sel_base;
                            if (row >= 0 && row < n_rows) { kp = kst + row * D; vp = vst + row * D; }
                        } else if (j < a.n_sel + res_len) {
                            const int64_t row = j - a.n_sel;
                            kp = rk + row * D; vp = rv + row * D;
                        } else {
                            kp = a.k_new + new_off; vp = a.v_new + new_off;
                        }
                    }
                    const bool ok = kp != nullptr;
                    // a skipped slot is zero-filled (source size 0) from any valid address
                    cp_async16(ks + soff[i], ok ? kp + col * 8 : a.q, ok ? 16 : 0);
                    cp_async16(vs + soff[i], ok ? vp + col * 8 : a.q, ok ? 16 : 0);
                    if (col == 0) s_valid[t % NS][r] = ok ? 1 : 0;
                }
            }
        }
        cp_async_commit();
    };

    // per-lane softmax state of head gq over this warp's rows (identical in the 4 lanes of a head,
    // except l_run which is each lane's partial sum) and the output accumulators O[gq][8*nt + 2*tq, +1]
    float m_run = -INFINITY, l_run = 0.0f;
    float o_acc[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) { o_acc[nt][0] = 0.0f; o_acc[nt][1] = 0.0f; }

    uint32_t my_id;
#pragma unroll
    for (int t = 0; t < NS - 1; t++) {  // prologue: tiles 0 .. NS-2
        my_id = fetch_id(t);
        issue_tile(t, my_id);
    }
    my_id = fetch_id(NS - 1);

    // ldmatrix addresses: 32-bit shared addresses, lane-dependent parts computed once.  A chunk index c
    // XORed with (row & 7) = (lane & 7) splits into a part that depends on the k-step / output tile
    // (compile-time constant XOR a lane constant) and a low part that is a lane constant.
    const unsigned smem_base = smem_u32(att_smem);
    const unsigned x7 = lane & 7;
    const unsigned lane_row_qk = (warp * RW + x7) * (D * 2);                               // + (rb*16 + grp*8) rows
    const unsigned lane_row_pv = (warp * RW + ((lane >> 3) & 1) * 8 + x7) * (D * 2);       // + rb*16 rows
    const unsigned xq = (x7 & 4u) << 4, lowq = (((lane >> 3) ^ x7) & 3u) << 4;             // chunk = 4*kk + (lane>>3)
    const unsigned xp = (x7 & 6u) << 4, lowp = (((lane >> 4) ^ x7) & 1u) << 4;             // chunk = 2*n2 + (lane>>4)

    for (int t = 0; t < n_tiles; t++) {
        cp_async_wait<NS - 2>();  // this thread's copies of tile t have landed (newer tiles may be in flight)
        __syncthreads();          // ... and everyone's; everyone is also done with tile t-1, whose slot is reused now
        issue_tile(t + NS - 1, my_id);
        my_id = fetch_id(t + NS);

        const unsigned ks = smem_base + (t % NS) * STAGE_BYTES;
        const unsigned vs = ks + TILE * D * 2;
        const unsigned char* valid = s_valid[t % NS];

#pragma unroll
        for (int rb = 0; rb < RB; rb++) {
            const int row0 = warp * RW + rb * 16;  // this warp's 16 rows
            // ---- S = Q.K^T for two 8-row groups: sc[2*grp + {0,1}] = rows row0 + 8*grp + 2*tq + {0,1} ----
            // mma.sync has a long issue-to-result latency here, so the k-steps are spread over four
            // independent accumulator chains (2 groups x even/odd k-step) instead of one chain per group.
            float sc[4];
            {
                float acc[2][2][2];
#pragma unroll
                for (int grp = 0; grp < 2; grp++)
#pragma unroll
                    for (int e = 0; e < 2; e++) { acc[grp][e][0] = 0.0f; acc[grp][e][1] = 0.0f; }
#pragma unroll
                for (int kk = 0; kk < KSTEPS / 2; kk++) {
#pragma unroll
                    for (int grp = 0; grp < 2; grp++) {
                        uint32_t bk[4];  // B fragments of k-steps 2kk (bk[0], bk[1]) and 2kk+1 (bk[2], bk[3])
                        ldmatrix_x4(bk, ks + lane_row_qk + (rb * 16 + grp * 8) * (D * 2) +
                                            ((static_cast<unsigned>(4 * kk) << 4) ^ xq) + lowq);
                        mma_16816<DT>(acc[grp][0][0], acc[grp][0][1], qa[2 * kk][0], qa[2 * kk][1], bk[0], bk[1]);
                        mma_16816<DT>(acc[grp][1][0], acc[grp][1][1], qa[2 * kk + 1][0], qa[2 * kk + 1][1], bk[2], bk[3]);
                    }
                }
#pragma unroll
                for (int grp = 0; grp < 2; grp++) {
                    const int r = row0 + grp * 8 + 2 * tq;
                    sc[2 * grp] = valid[r] ? (acc[grp][0][0] + acc[grp][1][0]) * a.scale_log2 : -INFINITY;
                    sc[2 * grp + 1] = valid[r + 1] ? (acc[grp][0][1] + acc[grp][1][1]) * a.scale_log2 : -INFINITY;
                }
            }
            // ---- online softmax over the 16 rows (the 4 lanes of a head hold 4 rows each) ----
            float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
            mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
            const float m_new = fmaxf(m_run, mx);
            const float alpha = (m_run == -INFINITY) ? 0.0f : exp2f(m_run - m_new);
            float p[4];
#pragma unroll
            for (int i = 0; i < 4; i++) p[i] = (sc[i] == -INFINITY) ? 0.0f : exp2f(sc[i] - m_new);
            l_run = l_run * alpha + (p[0] + p[1]) + (p[2] + p[3]);
            m_run = m_new;
            if (__any_sync(0xFFFFFFFFu, alpha != 1.0f)) {  // the running maximum rarely moves after the first tiles
#pragma unroll
                for (int nt = 0; nt < NT; nt++) { o_acc[nt][0] *= alpha; o_acc[nt][1] *= alpha; }
            }
            // ---- O += P.V: the S fragments are the A fragments of P (k = row within the 16) ----
            uint32_t p_hi[2], p_lo[2];
            pack_hi_lo<DT>(p[0], p[1], p_hi[0], p_lo[0]);  // rows 2tq, 2tq+1      (k = 2tq, 2tq+1)
            pack_hi_lo<DT>(p[2], p[3], p_hi[1], p_lo[1]);  // rows 8+2tq, 8+2tq+1  (k = 2tq+8, 2tq+9)
            // Each output tile takes two MMAs (value and residue of P) on the same accumulator; they are
            // issued four tiles apart so that the second never waits for the first.
#pragma unroll
            for (int n4 = 0; n4 < NT / 8; n4++) {
                uint32_t bv[4][4];  // V^T fragments of 8 output tiles: (bv[j][0], bv[j][1]) tile 2*(4*n4+j), (bv[j][2], bv[j][3]) the next
#pragma unroll
                for (int j = 0; j < 4; j++)
                    ldmatrix_x4_trans(bv[j], vs + lane_row_pv + (rb * 16) * (D * 2) +
                                                 ((static_cast<unsigned>(2 * (4 * n4 + j)) << 4) ^ xp) + lowp);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int n2 = 4 * n4 + j;
                    mma_16816<DT>(o_acc[2 * n2][0], o_acc[2 * n2][1], p_hi[0], p_hi[1], bv[j][0], bv[j][1]);
                    mma_16816<DT>(o_acc[2 * n2 + 1][0], o_acc[2 * n2 + 1][1], p_hi[0], p_hi[1], bv[j][2], bv[j][3]);
                }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int n2 = 4 * n4 + j;
                    mma_16816<DT>(o_acc[2 * n2][0], o_acc[2 * n2][1], p_lo[0], p_lo[1], bv[j][0], bv[j][1]);
                    mma_16816<DT>(o_acc[2 * n2 + 1][0], o_acc[2 * n2 + 1][1], p_lo[0], p_lo[1], bv[j][2], bv[j][3]);
                }
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();  // the ring is idle: reuse it to merge the warps' partial results

    // ---- merge the kAttWarps row slices (log-sum-exp) and write this split's partial ----
    float (*s_o)[kHeadsPerCta][D + 4] = reinterpret_cast<float (*)[kHeadsPerCta][D + 4]>(att_smem);
    l_run += __shfl_xor_sync(0xFFFFFFFFu, l_run, 1);
    l_run += __shfl_xor_sync(0xFFFFFFFFu, l_run, 2);
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
        *reinterpret_cast<float2*>(&s_o[warp][gq][8 * nt + 2 * tq]) = make_float2(o_acc[nt][0], o_acc[nt][1]);
    if (tq == 0) { s_ml[warp][gq][0] = m_run; s_ml[warp][gq][1] = l_run; }
    __syncthreads();
    for (int e = tid; e < n_heads * D; e += kAttThreads) {
        const int g = e / D, d = e % D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttWarps; w++) m = fmaxf(m, s_ml[w][g][0]);
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < kAttWarps; w++) {
            const float mw = s_ml[w][g][0];
            if (mw != -INFINITY) o += s_o[w][g][d] * exp2f(mw - m);
        }
        a.part_acc[((prob * a.group + g0 + g) * a.n_split + split) * D + d] = o;
    }
    if (tid < n_heads) {
        float m = -INFINITY, l = 0.0f;
#pragma unroll
        for (int w = 0; w < kAttWarps; w++) m = fmaxf(m, s_ml[w][tid][0]);
#pragma unroll
        for (int w = 0; w < kAttWarps; w++) {
            const float mw = s_ml[w][tid][0];
            if (mw != -INFINITY) l += s_ml[w][tid][1] * exp2f(mw - m);
        }
        float* ml = a.part_ml + ((prob * a.group + g0 + tid) * a.n_split + split) * 2;
        ml[0] = m;
        ml[1] = l;
    }
}

// Merge partials: part s of row r is acc[s*acc_ps + r*acc_rs .. +dim), (m, l) at ml[s*ml_ps + r*ml_rs].
// Split-K layout (rows, n_part, D): acc_ps = D, acc_rs = n_part*D.  All-gather layout
// (n_part, rows, D): acc_ps = part stride, acc_rs = D.  Writes either the normalised output in the
// element type (+ optional natural-log LSE) or the merged un-normalised (acc, m, l).
constexpr int kCombineThreads = 128;
constexpr int kCombineMaxParts = 1024;

// One row (blockIdx.x) of a merge.  xepoch: epoch the fan-out stores carry (xo.world != 0); want: epoch the polled
// parts must carry (ll.chan != nullptr).  Uses static shared memory: a kernel that calls it twice separates the
// calls with a block barrier.
template <int DT>
__device__ __forceinline__ void
combine_row(const float* __restrict__ part_acc, int64_t acc_ps, int64_t acc_rs, const float* __restrict__ part_ml,
            int64_t ml_ps, int64_t ml_rs, int n_part, int dim, uint16_t* __restrict__ out, float* __restrict__ out_lse,
            float* __restrict__ out_acc, float* __restrict__ out_ml, const XchgLL& ll, int64_t ll_ml_off, uint32_t want,
            const XchgOut& xo, int64_t xo_ml_off, uint32_t xepoch) {
    const int64_t row = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    __shared__ float s_w[kCombineMaxParts];   // weight of every part: exp2(m_s - M)
    __shared__ float s_red[kCombineThreads / 32];
    __shared__ float s_M, s_L;
    const float* ml = part_ml + row * ml_rs;
    const float* acc = part_acc + row * acc_rs;
    // Parts delivered by peer stores as {word, epoch} pairs into this rank's exchange buffer (slot s = part s,
    // holding [acc (rows, dim) | ml (rows, 2)]): this row's words are polled until they carry the current epoch
    // and staged in shared memory, which then takes the place of the global arrays.
    __shared__ __align__(16) float s_stage[kXchgMaxWorld * (256 + 4)];
    if (ll.chan != nullptr) {
        const int row_stride = dim + 4;   // dim accumulators, (m, l), padding that keeps rows 16-byte aligned
        const unsigned long long t0 = global_timer_ns();
        bool fail = false;
        const int per = dim / 2 + 1;      // pair vectors per part: dim / 2 of accumulators, one of (m, l)
        // four vectors per thread are loaded before the first is examined (one round trip for all of them);
        // only vectors that have not arrived yet are polled one by one
        const int total = n_part * per;
        for (int i0 = tid; i0 < total; i0 += 4 * kCombineThreads) {
            uint4 w[4];
            const uint4* src[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int i = i0 + j * kCombineThreads;
                if (i >= total) continue;
                const int s = i / per, v = i % per;
                const int64_t word = v < dim / 2 ? row * dim + 2 * v : ll_ml_off + row * 2;
                src[j] = ll.chan + s * ll.slot_vecs + word / 2;
                w[j] = ld_volatile16(src[j]);
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int i = i0 + j * kCombineThreads;
                if (i >= total) continue;
                const int s = i / per, v = i % per;
                uint2 d = make_uint2(w[j].x, w[j].z);
                if (w[j].y != want || w[j].w != want) d = xchg_poll(src[j], want, ll, t0, fail);
                float* dst = s_stage + s * row_stride + (v < dim / 2 ? 2 * v : dim);
                dst[0] = __uint_as_float(d.x);
                dst[1] = __uint_as_float(d.y);
            }
        }
        __syncthreads();
        acc = s_stage; acc_ps = row_stride;
        ml = s_stage + dim; ml_ps = row_stride;
    }
    // M = max_s m_s
    float m = -INFINITY;
    for (int s = tid; s < n_part; s += kCombineThreads) m = fmaxf(m, ml[s * ml_ps]);
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
    if (lane == 0) s_red[warp] = m;
    __syncthreads();
    if (tid == 0) {
        float mm = s_red[0];
        for (int w = 1; w < kCombineThreads / 32; w++) mm = fmaxf(mm, s_red[w]);
        s_M = mm;
    }
    __syncthreads();
    const float M = s_M;
    // weights and L = sum_s w_s * l_s
    float l = 0.0f;
    for (int s = tid; s < n_part; s += kCombineThreads) {
        const float ms = ml[s * ml_ps];
        const float w = (ms == -INFINITY) ? 0.0f : exp2f(ms - M);
        s_w[s] = w;
        l += w * ml[s * ml_ps + 1];
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) l += __shfl_xor_sync(0xFFFFFFFFu, l, off);
    __syncthreads();  // s_M consumed by everyone before s_red is reused; s_w complete
    if (lane == 0) s_red[warp] = l;
    __syncthreads();
    if (tid == 0) {
        float ll = 0.0f;
        for (int w = 0; w < kCombineThreads / 32; w++) ll += s_red[w];
        s_L = ll;
    }
    __syncthreads();
    const float L = s_L;
    const bool vec_ok = (dim % 4 == 0) && (dim / 4 <= kCombineThreads) && (kCombineThreads % (dim / 4) == 0) &&
                        (acc_ps % 4 == 0) && ((reinterpret_cast<uintptr_t>(acc) & 15) == 0);
    if (vec_ok) {
        // 16-byte loads; the parts are dealt round-robin to dim/4-lane groups so that their loads are
        // in flight together, and the groups' sums are added through shared memory
        __shared__ __align__(16) float s_part[kCombineThreads * 4];
        const int lanes = dim / 4, groups = kCombineThreads / lanes;
        const int g = tid / lanes, l = tid % lanes;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = g; s < n_part; s += groups) {
            const float4 a4 = *reinterpret_cast<const float4*>(acc + s * acc_ps + 4 * l);
            const float w = s_w[s];
            o.x += a4.x * w; o.y += a4.y * w; o.z += a4.z * w; o.w += a4.w * w;
        }
        *reinterpret_cast<float4*>(&s_part[(g * lanes + l) * 4]) = o;
        __syncthreads();
        if (tid < lanes) {
            float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int gg = 0; gg < groups; gg++) {
                const float4 p4 = *reinterpret_cast<const float4*>(&s_part[(gg * lanes + tid) * 4]);
                t.x += p4.x; t.y += p4.y; t.z += p4.z; t.w += p4.w;
            }
            const float v4[4] = {t.x, t.y, t.z, t.w};
            uint16_t e4[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int d = 4 * tid + j;
                e4[j] = float_to_elem<DT>(L > 0.0f ? v4[j] / L : 0.0f);
                if (out) out[row * dim + d] = e4[j];
                if (out_acc) out_acc[row * dim + d] = v4[j];
            }
            if (xo.world) {
                if (out_acc) {   // four fp32 accumulators = four words
                    const int64_t w = xchg_word_index(xo, row, 4 * tid);
                    xchg_put2(xo, xepoch, w, __float_as_uint(v4[0]), __float_as_uint(v4[1]));
                    xchg_put2(xo, xepoch, w + 2, __float_as_uint(v4[2]), __float_as_uint(v4[3]));
                } else {         // four 16-bit outputs = two words
                    xchg_put2(xo, xepoch, xchg_word_index(xo, row, 2 * tid), e4[0] | (static_cast<uint32_t>(e4[1]) << 16),
                              e4[2] | (static_cast<uint32_t>(e4[3]) << 16));
                }
            }
        }
    } else {
        for (int d = tid; d < dim; d += kCombineThreads) {
            float o = 0.0f;
            for (int s = 0; s < n_part; s++) o += acc[s * acc_ps + d] * s_w[s];
            if (out) out[row * dim + d] = float_to_elem<DT>(L > 0.0f ? o / L : 0.0f);
            if (out_acc) out_acc[row * dim + d] = o;
            if (xo.world && out_acc) xchg_put(xo, xepoch, xchg_word_index(xo, row, d), __float_as_uint(o));
        }
        // (the host only asks for a fan-out of 16-bit outputs when the vector path above is taken)
    }
    if (tid == 0) {
        if (out_lse) out_lse[row] = L > 0.0f ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
        if (out_ml) { out_ml[row * 2] = M; out_ml[row * 2 + 1] = L; }
        if (xo.world && out_ml) xchg_put2(xo, xepoch, xo.rank_off + xo_ml_off + row * 2, __float_as_uint(M), __float_as_uint(L));
    }
}

template <int DT>
__global__ void __launch_bounds__(kCombineThreads)
lse_combine_kernel(const float* __restrict__ part_acc, int64_t acc_ps, int64_t acc_rs,
                   const float* __restrict__ part_ml, int64_t ml_ps, int64_t ml_rs, int n_part, int dim,
                   uint16_t* __restrict__ out, float* __restrict__ out_lse, float* __restrict__ out_acc,
                   float* __restrict__ out_ml, const XchgLL ll, int64_t ll_ml_off, const XchgOut xo, int64_t xo_ml_off) {
    pdl_launch_dependents();
    pdl_wait();
    // results that other ranks need go straight into every rank's exchange buffer as well (pair format):
    // (acc, m, l) of a sequence-sharded step, or the 16-bit output slice of a head-sharded layer
    const uint32_t xepoch = xo.world ? xchg_next_epoch(xo) : 0u;
    const uint32_t want = ll.chan != nullptr ? ll.epoch[ll.channel] : 0u;
    combine_row<DT>(part_acc, acc_ps, acc_rs, part_ml, ml_ps, ml_rs, n_part, dim, out, out_lse, out_acc, out_ml, ll,
                    ll_ml_off, want, xo, xo_ml_off, xepoch);
    if (xo.world) xchg_finish(xo, xepoch, gridDim.x);
}

// Sequence-sharded step, both sides of the second exchange in one launch: the CTA of a row merges this rank's
// split partials, stores (acc, m, l) into every rank's copy of the channel, then waits for the other ranks' (acc,
// m, l) of the same row in its own copy and merges those into the final output.  The second half polls for the
// epoch the first half has just written with, so it needs no kernel boundary in between; what it waits for is
// written by the same kernel on the OTHER GPUs, never by a later launch on this one.
template <int DT>
__global__ void __launch_bounds__(kCombineThreads)
lse_combine_exchange_kernel(const float* __restrict__ part_acc, int64_t acc_ps, int64_t acc_rs,
                            const float* __restrict__ part_ml, int64_t ml_ps, int64_t ml_rs, int n_part, int dim,
                            float* __restrict__ out_acc, float* __restrict__ out_ml, const XchgOut xo, int64_t ml_off,
                            const XchgLL ll, uint16_t* __restrict__ out, float* __restrict__ out_lse) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t xepoch = xchg_next_epoch(xo);
    const XchgLL none = {};
    combine_row<DT>(part_acc, acc_ps, acc_rs, part_ml, ml_ps, ml_rs, n_part, dim, nullptr, nullptr, out_acc, out_ml, none,
                    0, 0u, xo, ml_off, xepoch);
    xchg_finish(xo, xepoch, gridDim.x);   // starts with a block barrier: the shared arrays are free again
    XchgOut off = xo;
    off.world = 0;
    combine_row<DT>(nullptr, 0, 0, nullptr, 0, 0, ll.world, dim, out, out_lse, nullptr, nullptr, ll, ml_off, xepoch, off, 0,
                    0u);
}

template <int DT, int LPR>
int launch_attend(const AttendArgs& a, int n_prob, cudaStream_t stream) {
    // > 48 KB of dynamic shared memory needs an opt-in per kernel and device (not a stream operation)
    static PerDeviceOnce once;
    int rc0 = once.run([](int) {
        DC_CUDA_TRY(cudaFuncSetAttribute(sparse_attend_kernel<DT, LPR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(att_smem_bytes<LPR>())));
        return DC_OK;
    });
    if (rc0 != DC_OK) return rc0;
    const int chunks = (a.group + kHeadsPerCta - 1) / kHeadsPerCta;
    dim3 grid(static_cast<unsigned>(a.n_split), static_cast<unsigned>(n_prob), static_cast<unsigned>(chunks));
    DC_CUDA_TRY(launch_chained(sparse_attend_kernel<DT, LPR>, grid, dim3(kAttThreads), att_smem_bytes<LPR>(), stream, 0u, a));
    return DC_OK;
}

// Head-sharded layer, both sides of the all-gather in one launch: the CTA of output row (b, h) merges the splits,
// stores its 16-bit output row into every rank's copy of the channel (xo: rows interleaved by rank, so that the
// channel reads (bsz, world, q_heads * dim)), then waits in its own copy for row (b, h) of EVERY rank and writes those
// `world` rows densely to `dense` (bsz, world * q_heads * dim) - what a separate wait-and-unpack kernel did before.
template <int DT>
__global__ void __launch_bounds__(kCombineThreads)
lse_combine_allgather_kernel(const float* __restrict__ part_acc, int64_t acc_ps, int64_t acc_rs,
                             const float* __restrict__ part_ml, int64_t ml_ps, int64_t ml_rs, int n_part, int dim,
                             uint16_t* __restrict__ out, float* __restrict__ out_lse, const XchgOut xo, const XchgLL ll,
                             uint32_t* __restrict__ dense) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t xepoch = xchg_next_epoch(xo);
    const XchgLL none = {};
    combine_row<DT>(part_acc, acc_ps, acc_rs, part_ml, ml_ps, ml_rs, n_part, dim, out, out_lse, nullptr, nullptr, none, 0,
                    0u, xo, 0, xepoch);
    xchg_finish(xo, xepoch, gridDim.x);
    // words of row (b, h) of rank r: block b, rank offset r * slice, row h of the slice (the layout of xo)
    const int64_t row = blockIdx.x;
    const int64_t b = row / xo.rows_per_block, h = row % xo.rows_per_block;
    const int64_t slice = xo.rows_per_block * xo.row_words;
    const int vec_per_row = static_cast<int>(xo.row_words / 2);   // 16-byte pair vectors (2 words) per row
    const unsigned long long t0 = global_timer_ns();
    bool fail = false;
    const int total = ll.world * vec_per_row;
    for (int i0 = threadIdx.x; i0 < total; i0 += 4 * kCombineThreads) {
        uint4 w[4];
        const uint4* src[4];
        int64_t word[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int i = i0 + j * kCombineThreads;
            if (i >= total) continue;
            const int r = i / vec_per_row, v = i % vec_per_row;
            word[j] = b * xo.block_stride + r * slice + h * xo.row_words + 2 * v;
            src[j] = ll.chan + word[j] / 2;
            w[j] = ld_volatile16(src[j]);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int i = i0 + j * kCombineThreads;
            if (i >= total) continue;
            uint2 d = make_uint2(w[j].x, w[j].z);
            if (w[j].y != xepoch || w[j].w != xepoch) d = xchg_poll(src[j], xepoch, ll, t0, fail);
            *reinterpret_cast<uint2*>(dense + word[j]) = d;
        }
    }
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
                float* out_ml, cudaStream_t stream, const XchgLL* ll, const XchgOut* xout, const XchgFinal* fin) {
    // fin (may be NULL; needs xout and out_acc / out_ml): after the fan-out the same launch waits for the other
    // ranks' blocks and writes the merge of all ranks' parts to fin->out
    // ll (may be NULL): the parts arrive in pair format in an exchange channel instead of acc / ml
    // xout (may be NULL): the results are also stored into every rank's copy of an exchange channel, either
    // (out_acc, out_ml) as [acc (rows, dim) | ml (rows, 2)] words or `out` as 16-bit pairs, laid out by xout
    DC_REQUIRE(xout == nullptr || out_acc != nullptr ||
                   (head_dim % 4 == 0 && head_dim / 4 <= kCombineThreads && kCombineThreads % (head_dim / 4) == 0),
               "lse_combine: fan-out of 16-bit outputs needs head_dim a multiple of 4 that divides %d", 4 * kCombineThreads);
    DC_REQUIRE(((acc && ml) || ll) && n_part >= 1 && rows >= 0, "lse_combine: bad arguments");
    DC_REQUIRE(ll == nullptr || (n_part <= kXchgMaxWorld && head_dim <= 256 && head_dim % 2 == 0),
               "lse_combine: parts from the peer exchange: at most %d parts, even head_dim <= 256", kXchgMaxWorld);
    DC_REQUIRE(dtype == DC_BF16 || dtype == DC_FP16, "lse_combine: dtype %d not supported", dtype);
    DC_REQUIRE(n_part <= kCombineMaxParts, "lse_combine: n_part=%d exceeds %d", n_part, kCombineMaxParts);
    if (rows == 0) return DC_OK;
    const dim3 grid(static_cast<unsigned>(rows)), block(kCombineThreads);
    XchgLL w = {};
    if (ll != nullptr) w = *ll;
    XchgOut xo = {};
    if (xout != nullptr) xo = *xout;
    const int64_t ml_off = rows * head_dim;   // word offset of the (m, l) block inside a part's slot
    if (fin != nullptr && out_acc == nullptr) {   // head-sharded layer: fan-out of the 16-bit rows + gather of all ranks' rows
        DC_REQUIRE(xout != nullptr && out != nullptr && ll == nullptr && fin->out != nullptr && fin->ll.chan != nullptr &&
                       fin->ll.world == xo.world && fin->ll.channel == xo.channel && xo.row_words % 2 == 0,
                   "lse_combine: the in-kernel gather needs the fan-out of `out` on the same channel");
        if (dtype == DC_BF16)
            DC_CUDA_TRY(launch_chained(lse_combine_allgather_kernel<DC_BF16>, grid, block, 0, stream, 0u, acc, acc_ps, acc_rs,
                                       ml, ml_ps, ml_rs, n_part, head_dim, static_cast<uint16_t*>(out), out_lse, xo, fin->ll,
                                       static_cast<uint32_t*>(fin->out)));
        else
            DC_CUDA_TRY(launch_chained(lse_combine_allgather_kernel<DC_FP16>, grid, block, 0, stream, 0u, acc, acc_ps, acc_rs,
                                       ml, ml_ps, ml_rs, n_part, head_dim, static_cast<uint16_t*>(out), out_lse, xo, fin->ll,
                                       static_cast<uint32_t*>(fin->out)));
        return DC_OK;
    }
    if (fin != nullptr) {
        DC_REQUIRE(xout != nullptr && out_acc != nullptr && out_ml != nullptr && ll == nullptr && fin->out != nullptr &&
                       fin->ll.chan != nullptr && fin->ll.world == xo.world && fin->ll.channel == xo.channel,
                   "lse_combine: the in-kernel final merge needs the fan-out of (acc, m, l) on the same channel");
        DC_REQUIRE(fin->ll.world <= kXchgMaxWorld && head_dim <= 256 && head_dim % 2 == 0,
                   "lse_combine: parts from the peer exchange: at most %d parts, even head_dim <= 256", kXchgMaxWorld);
        if (dtype == DC_BF16)
            DC_CUDA_TRY(launch_chained(lse_combine_exchange_kernel<DC_BF16>, grid, block, 0, stream, 0u, acc, acc_ps, acc_rs,
                                       ml, ml_ps, ml_rs, n_part, head_dim, out_acc, out_ml, xo, ml_off, fin->ll,
                                       static_cast<uint16_t*>(fin->out), fin->out_lse));
        else
            DC_CUDA_TRY(launch_chained(lse_combine_exchange_kernel<DC_FP16>, grid, block, 0, stream, 0u, acc, acc_ps, acc_rs,
                                       ml, ml_ps, ml_rs, n_part, head_dim, out_acc, out_ml, xo, ml_off, fin->ll,
                                       static_cast<uint16_t*>(fin->out), fin->out_lse));
        return DC_OK;
    }
    if (dtype == DC_BF16)
        DC_CUDA_TRY(launch_chained(lse_combine_kernel<DC_BF16>, grid, block, 0, stream, 0u, acc, acc_ps, acc_rs, ml, ml_ps,
                                   ml_rs, n_part, head_dim, static_cast<uint16_t*>(out), out_lse, out_acc, out_ml, w, ml_off,
                                   xo, ml_off));
    else
        DC_CUDA_TRY(launch_chained(lse_combine_kernel<DC_FP16>, grid, block, 0, stream, 0u, acc, acc_ps, acc_rs, ml, ml_ps,
                                   ml_rs, n_part, head_dim, static_cast<uint16_t*>(out), out_lse, out_acc, out_ml, w, ml_off,
                                   xo, ml_off));
    return DC_OK;
}

int sparse_attend(const void* k_store, const void* v_store, int64_t prob_stride, int64_t n_rows, int n_prob,
                  int kv_heads, int group, int head_dim, int dtype, const void* q, const uint32_t* sel,
                  int64_t sel_stride, int n_sel, int64_t sel_base, const void* k_new, const void* v_new, void* res_k,
                  void* res_v, int64_t res_stride_b, int64_t res_stride_h, int res_len, float scale, void* out,
                  float* out_lse, float* out_acc, float* out_ml, void* scratch, cudaStream_t stream,
                  const int32_t* sel_count, int64_t q_stride_b, int64_t new_stride_b, const int32_t* n_rows_dev,
                  const int32_t* res_len_dev, const XchgOut* xout, const XchgFinal* fin) {
    // n_rows_dev / res_len_dev (may be NULL): device words read when the kernel runs, overriding n_rows and
    // res_len, which then only size the launch (res_len = the most resident rows there can be)
    DC_REQUIRE(q != nullptr && scratch != nullptr, "sparse_attend: null q/scratch");
    DC_REQUIRE(q_stride_b % 8 == 0 && new_stride_b % 8 == 0, "sparse_attend: batch strides must be multiples of 8 elements");
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
    a.q_stride_b = q_stride_b;
    a.new_stride_b = new_stride_b;
    a.sel = sel;
    a.sel_stride = sel_stride;
    a.n_sel = n_sel;
    a.sel_base = sel_base;
    a.sel_count = sel_count;
    a.k_new = static_cast<const uint16_t*>(k_new);
    a.v_new = static_cast<const uint16_t*>(v_new);
    a.res_k = static_cast<uint16_t*>(res_k);
    a.res_v = static_cast<uint16_t*>(res_v);
    a.res_stride_b = res_stride_b;
    a.res_stride_h = res_stride_h;
    a.res_len = res_len;
    a.n_rows_dev = n_rows_dev;
    a.res_len_dev = res_len_dev;
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
                       dtype, out, out_lse, out_acc, out_ml, stream, nullptr, xout, fin);
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
// The look-up runs once per device under a lock, so first calls from several host threads are safe.
int noalloc_scratch_ptr(void** out) {
    static void* ptrs[PerDeviceOnce::kMaxDevices] = {};
    static PerDeviceOnce once;
    *out = nullptr;
    int dev = 0;
    DC_CUDA_TRY(cudaGetDevice(&dev));
    DC_REQUIRE(dev >= 0 && dev < PerDeviceOnce::kMaxDevices, "dc_sparse_attend_noalloc: device ordinal %d not supported",
               dev);
    int rc = once.run([](int d) {
        void* p = nullptr;
        DC_CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        DC_REQUIRE(p != nullptr, "dc_sparse_attend_noalloc: no device address for the static scratch array");
        ptrs[d] = p;
        return DC_OK;
    });
    if (rc != DC_OK) return rc;
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
                         scale, out, out_lse, out_acc, out_ml, scratch, as_stream(stream), nullptr, 0, 0, nullptr, nullptr,
                         nullptr, nullptr);
}
