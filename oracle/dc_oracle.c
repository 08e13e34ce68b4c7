/*
 * CPU oracle for the decode-time retrieval-attention path of DiffCache.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * against and the timed CPU baseline; the product never links or calls it.
 *
 * PARITY UNPINNED: the reference holds no test, fixture or golden vector for
 * its scan / top-k / attention path (its only unit tests cover DualHeap,
 * diffcache_cpu/src/dualheap.rs:109-359), and its Rust crate cannot be built
 * where this oracle runs.  What is pinned: the top-k ordering semantics against
 * the DualHeap tests' sequences (tests/golden/select_kat.json).  Everything
 * else is a line-by-line restatement of the cited reference code.
 *
 * Element types cross as uint16 bit patterns (bf16 = 0, fp16 = 1), as in
 * diffcache_cpu/src/lib.rs:528-544.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define DCO_BF16 0
#define DCO_FP16 1

static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static inline float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

static inline float fp16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        /* subnormal: value = man * 2^-24 */
        float v = (float)man * 5.9604644775390625e-08f;
        return sign ? -v : v;
    }
    if (exp == 31) return bits_f32(sign | 0x7F800000u | (man << 13));
    return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

static inline float elem_to_f32(uint16_t h, int dtype) {
    return dtype == DCO_BF16 ? bf16_to_f32(h) : fp16_to_f32(h);
}

/* round-to-nearest-even fp32 -> bf16 (NaN kept quiet) */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u = f32_bits(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40u);
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7FFFu + lsb;
    return (uint16_t)(u >> 16);
}

/* round-to-nearest-even fp32 -> fp16 */
static inline uint16_t f32_to_fp16(float f) {
    uint32_t u = f32_bits(f);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t au = u & 0x7FFFFFFFu;
    if (au > 0x7F800000u) return (uint16_t)(sign | 0x7E00u);
    if (au >= 0x47800000u) return (uint16_t)(sign | 0x7C00u); /* >= 65536 -> inf (65520 rounds up too) */
    if (au >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);
    if (au < 0x33000000u) return (uint16_t)sign;              /* < 2^-25 -> 0 */
    int32_t e = (int32_t)(au >> 23) - 127;
    uint32_t m = (au & 0x7FFFFFu) | 0x800000u;
    if (e < -14) {
        int shift = -14 - e + 13; /* bits to drop from the 24-bit significand */
        uint32_t q = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1u);
        uint32_t half = 1u << (shift - 1);
        if (rem > half || (rem == half && (q & 1u))) q++;
        return (uint16_t)(sign | q);
    }
    uint32_t q = ((uint32_t)(e + 15) << 10) | ((m >> 13) & 0x3FFu);
    uint32_t rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) q++;
    return (uint16_t)(sign | q);
}

static inline uint16_t f32_to_elem(float f, int dtype) {
    return dtype == DCO_BF16 ? f32_to_bf16(f) : f32_to_fp16(f);
}

void dco_convert_to_f32(const uint16_t* in, int64_t n, int dtype, float* out) {
    for (int64_t i = 0; i < n; i++) out[i] = elem_to_f32(in[i], dtype);
}

void dco_convert_from_f32(const float* in, int64_t n, int dtype, uint16_t* out) {
    for (int64_t i = 0; i < n; i++) out[i] = f32_to_elem(in[i], dtype);
}

/*
 * Retrieval query = mean of the `group` query heads of each kv head, rounded to
 * the element type: src/diffcache/kvcache/diffcache.py:191-194
 * (`queries.view(B,Hkv,G,D).mean(dim=2)` on a bf16 tensor: fp32 sum in head
 * order, times 1/G, one rounding).  q: (n_prob*group, dim); out: (n_prob, dim).
 */
void dco_group_mean(const uint16_t* q, int n_prob, int group, int dim, int dtype, uint16_t* out) {
    float inv = 1.0f / (float)group;
    for (int p = 0; p < n_prob; p++)
        for (int d = 0; d < dim; d++) {
            float s = 0.0f;
            for (int g = 0; g < group; g++) s += elem_to_f32(q[((int64_t)p * group + g) * dim + d], dtype);
            out[(int64_t)p * dim + d] = f32_to_elem(s * inv, dtype);
        }
}

/*
 * Index::distance, QKDist: diffcache_cpu/src/nsw.rs:129-139 with
 * InnerProduct for bf16 (diffcache_cpu/src/lib.rs:65-69).
 * exact != 0: dot = the exact sum of the exact products, rounded once to fp32
 *             (the parity definition; the reference's simsimd accumulation
 *             order is ISA dependent).
 * exact == 0: fp32 accumulation in 16 independent lanes, the shape of a SIMD
 *             bf16 dot kernel; used for the timed CPU baseline only.
 */
static inline uint32_t dist_bits_one(const uint16_t* k, const float* qf, int dim, int dtype, int exact) {
    float dot;
    if (exact) {
        double acc = 0.0;
        for (int d = 0; d < dim; d++) acc += (double)(elem_to_f32(k[d], dtype) * qf[d]); /* product exact in fp32 */
        dot = (float)acc;
    } else {
        float lane[16] = {0};
        int d = 0;
        if (dtype == DCO_BF16) {
            for (; d + 16 <= dim; d += 16)
                for (int j = 0; j < 16; j++) lane[j] += bits_f32((uint32_t)k[d + j] << 16) * qf[d + j];
        } else {
            for (; d + 16 <= dim; d += 16)
                for (int j = 0; j < 16; j++) lane[j] += fp16_to_f32(k[d + j]) * qf[d + j];
        }
        for (; d < dim; d++) lane[0] += elem_to_f32(k[d], dtype) * qf[d];
        float s8[8], s4[4];
        for (int j = 0; j < 8; j++) s8[j] = lane[j] + lane[j + 8];
        for (int j = 0; j < 4; j++) s4[j] = s8[j] + s8[j + 4];
        dot = (s4[0] + s4[2]) + (s4[1] + s4[3]);
    }
    float dist = 65536.0f - dot; /* nsw.rs:138 */
    return f32_bits(dist);
}

/* dist bits of every row of one problem (the scan of nsw.rs:601-607). */
void dco_score_rows(const uint16_t* keys, int64_t n, int dim, int dtype, const uint16_t* q, int exact,
                    uint32_t* out_bits) {
    float qf[1024];
    for (int d = 0; d < dim; d++) qf[d] = elem_to_f32(q[d], dtype);
    for (int64_t i = 0; i < n; i++) out_bits[i] = dist_bits_one(keys + i * dim, qf, dim, dtype, exact);
}

/* ---- binary max-heap of u64 keys (std::collections::BinaryHeap<u64>, nsw.rs:600) ---- */
typedef struct { uint64_t* a; int64_t len; } heap_t;

static inline void heap_sift_up(heap_t* h, int64_t i) {
    uint64_t v = h->a[i];
    while (i > 0) {
        int64_t p = (i - 1) / 2;
        if (h->a[p] >= v) break;
        h->a[i] = h->a[p];
        i = p;
    }
    h->a[i] = v;
}

static inline void heap_sift_down(heap_t* h, int64_t i) {
    uint64_t v = h->a[i];
    int64_t n = h->len;
    for (;;) {
        int64_t c = 2 * i + 1;
        if (c >= n) break;
        if (c + 1 < n && h->a[c + 1] > h->a[c]) c++;
        if (h->a[c] <= v) break;
        h->a[i] = h->a[c];
        i = c;
    }
    h->a[i] = v;
}

static int cmp_u64(const void* x, const void* y) {
    uint64_t a = *(const uint64_t*)x, b = *(const uint64_t*)y;
    return a < b ? -1 : (a > b ? 1 : 0);
}

/*
 * Heap top-`ef` over a stream of (dist bits, id) exactly as nsw.rs:600-615:
 * push while the heap is not full, afterwards replace the maximum only when
 * the new dist is strictly smaller (float compare, nsw.rs:612).  ids == NULL
 * means id = position.  Returns the number kept (min(ef, n)); out_bits/out_ids
 * ascending by (bits << 32 | id) = BinaryHeap::into_sorted_vec (nsw.rs:621).
 */
int64_t dco_topk_heap(const uint32_t* bits, const uint32_t* ids, int64_t n, int64_t ef, uint32_t* out_bits,
                      uint32_t* out_ids) {
    if (ef <= 0) return 0;
    heap_t h;
    h.a = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)ef);
    h.len = 0;
    for (int64_t i = 0; i < n; i++) {
        uint32_t id = ids ? ids[i] : (uint32_t)i;
        uint64_t key = ((uint64_t)bits[i] << 32) | id; /* nsw.rs:74-80 */
        if (h.len < ef) {
            h.a[h.len++] = key;
            heap_sift_up(&h, h.len - 1);
        } else {
            float top = bits_f32((uint32_t)(h.a[0] >> 32));
            if (bits_f32(bits[i]) < top) {
                h.a[0] = key;
                heap_sift_down(&h, 0);
            }
        }
    }
    qsort(h.a, (size_t)h.len, sizeof(uint64_t), cmp_u64);
    for (int64_t i = 0; i < h.len; i++) {
        if (out_bits) out_bits[i] = (uint32_t)(h.a[i] >> 32);
        if (out_ids) out_ids[i] = (uint32_t)(h.a[i] & 0xFFFFFFFFu);
    }
    int64_t kept = h.len;
    free(h.a);
    return kept;
}

/*
 * "ef smallest under the total order (bits, id)" by sorting everything — the
 * definition the heap above must agree with when ids ascend with position.
 */
int64_t dco_topk_sort(const uint32_t* bits, const uint32_t* ids, int64_t n, int64_t ef, uint32_t* out_bits,
                      uint32_t* out_ids) {
    uint64_t* a = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)(n > 0 ? n : 1));
    for (int64_t i = 0; i < n; i++) a[i] = ((uint64_t)bits[i] << 32) | (ids ? ids[i] : (uint32_t)i);
    qsort(a, (size_t)n, sizeof(uint64_t), cmp_u64);
    int64_t kept = ef < n ? ef : n;
    for (int64_t i = 0; i < kept; i++) {
        if (out_bits) out_bits[i] = (uint32_t)(a[i] >> 32);
        if (out_ids) out_ids[i] = (uint32_t)(a[i] & 0xFFFFFFFFu);
    }
    free(a);
    return kept;
}

/*
 * DataLayer::query with use_bruteforce (diffcache_cpu/src/lib.rs:373-404) →
 * Index::search_bruteforce (diffcache_cpu/src/nsw.rs:592-630): per problem one
 * serial scan + heap + gather, a thread pool across the problems (rayon
 * par_iter, lib.rs:387-401).
 *   keys/vals : n_prob problems, problem stride `prob_stride` elements, n valid rows
 *   q_mean    : (n_prob, dim)
 *   out_keys/out_vals : (n_prob, ef, dim) (may be NULL), out_idx/out_bits (n_prob, ef)
 * ef is clamped to n (lib.rs:374).  Returns the clamped ef.
 */
int64_t dco_query(const uint16_t* keys, const uint16_t* vals, int64_t prob_stride, int n_prob, int64_t n, int dim,
                  int dtype, const uint16_t* q_mean, int64_t ef, int exact, int n_threads, uint16_t* out_keys,
                  uint16_t* out_vals, uint32_t* out_idx, uint32_t* out_bits) {
    if (ef > n) ef = n;
    if (ef <= 0) return 0;
#ifdef _OPENMP
    if (n_threads > 0) omp_set_num_threads(n_threads);
#endif
#pragma omp parallel for schedule(dynamic, 1)
    for (int p = 0; p < n_prob; p++) {
        const uint16_t* kp = keys + (int64_t)p * prob_stride;
        const uint16_t* vp = vals ? vals + (int64_t)p * prob_stride : NULL;
        float qf[1024];
        for (int d = 0; d < dim; d++) qf[d] = elem_to_f32(q_mean[(int64_t)p * dim + d], dtype);
        heap_t h;
        h.a = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)ef);
        h.len = 0;
        for (int64_t i = 0; i < n; i++) {
            uint32_t b = dist_bits_one(kp + i * dim, qf, dim, dtype, exact);
            if (h.len < ef) {
                h.a[h.len++] = ((uint64_t)b << 32) | (uint32_t)i;
                heap_sift_up(&h, h.len - 1);
            } else if (bits_f32(b) < bits_f32((uint32_t)(h.a[0] >> 32))) {
                h.a[0] = ((uint64_t)b << 32) | (uint32_t)i;
                heap_sift_down(&h, 0);
            }
        }
        qsort(h.a, (size_t)h.len, sizeof(uint64_t), cmp_u64);
        for (int64_t i = 0; i < h.len; i++) { /* gather, nsw.rs:623-629 */
            uint32_t id = (uint32_t)(h.a[i] & 0xFFFFFFFFu);
            if (out_keys) memcpy(out_keys + ((int64_t)p * ef + i) * dim, kp + (int64_t)id * dim, sizeof(uint16_t) * dim);
            if (out_vals && vp) memcpy(out_vals + ((int64_t)p * ef + i) * dim, vp + (int64_t)id * dim, sizeof(uint16_t) * dim);
            if (out_idx) out_idx[(int64_t)p * ef + i] = id;
            if (out_bits) out_bits[(int64_t)p * ef + i] = (uint32_t)(h.a[i] >> 32);
        }
        free(h.a);
    }
    return ef;
}

/*
 * Softmax attention of every query head over a gathered row set, the semantics
 * of flash_attn_with_kvcache as called at src/diffcache/base.py:134-142:
 * rows = [selected | resident | new token], GQA head hq -> kv head hq / group,
 * score = scale * <q, k>, output = softmax(score) . V.
 *   k_rows/v_rows : (n_prob, n_rows, dim) already gathered (element type)
 *   q             : (n_prob*group, dim)
 *   out_f32       : (n_prob*group, dim) fp64-accumulated result as fp32 (may be NULL)
 *   out_elem      : same, rounded to the element type (may be NULL)
 *   out_lse       : (n_prob*group) natural-log sum-exp of scaled scores (may be NULL)
 */
void dco_attend(const uint16_t* k_rows, const uint16_t* v_rows, int n_prob, int64_t n_rows, int group, int dim,
                int dtype, const uint16_t* q, float scale, int n_threads, float* out_f32, uint16_t* out_elem,
                float* out_lse) {
#ifdef _OPENMP
    if (n_threads > 0) omp_set_num_threads(n_threads);
#endif
#pragma omp parallel for schedule(dynamic, 1)
    for (int pg = 0; pg < n_prob * group; pg++) {
        int p = pg / group;
        const uint16_t* kp = k_rows + (int64_t)p * n_rows * dim;
        const uint16_t* vp = v_rows + (int64_t)p * n_rows * dim;
        double* s = (double*)malloc(sizeof(double) * (size_t)(n_rows > 0 ? n_rows : 1));
        double* acc = (double*)calloc((size_t)dim, sizeof(double));
        double m = -INFINITY;
        for (int64_t j = 0; j < n_rows; j++) {
            double dot = 0.0;
            for (int d = 0; d < dim; d++)
                dot += (double)elem_to_f32(kp[j * dim + d], dtype) * (double)elem_to_f32(q[(int64_t)pg * dim + d], dtype);
            s[j] = dot * (double)scale;
            if (s[j] > m) m = s[j];
        }
        double l = 0.0;
        for (int64_t j = 0; j < n_rows; j++) {
            double w = exp(s[j] - m);
            l += w;
            for (int d = 0; d < dim; d++) acc[d] += w * (double)elem_to_f32(vp[j * dim + d], dtype);
        }
        for (int d = 0; d < dim; d++) {
            float o = n_rows > 0 ? (float)(acc[d] / l) : 0.0f;
            if (out_f32) out_f32[(int64_t)pg * dim + d] = o;
            if (out_elem) out_elem[(int64_t)pg * dim + d] = f32_to_elem(o, dtype);
        }
        if (out_lse) out_lse[pg] = n_rows > 0 ? (float)(m + log(l)) : -INFINITY;
        free(s);
        free(acc);
    }
}

/* ---- product-quantisation baseline (no counterpart in the reference) ---- */

/* lut[p][m][c] = <q_p[m*ds .. (m+1)*ds), centroid[p][m][c][:]>, fp32, dims in order. */
void dco_pq_build_lut(const uint16_t* q_mean, int dtype, const float* centroids, int n_prob, int dim, int n_sub,
                      float* lut) {
    int ds = dim / n_sub;
    for (int p = 0; p < n_prob; p++)
        for (int m = 0; m < n_sub; m++)
            for (int c = 0; c < 256; c++) {
                const float* cen = centroids + (((int64_t)p * n_sub + m) * 256 + c) * ds;
                float s = 0.0f;
                for (int d = 0; d < ds; d++) s = fmaf(elem_to_f32(q_mean[(int64_t)p * dim + m * ds + d], dtype), cen[d], s);
                lut[((int64_t)p * n_sub + m) * 256 + c] = s;
            }
}

/* ADC: score = sum_m lut[m][code[m]] in increasing m (fp32); bits(65536 - score). */
void dco_pq_adc_scores(const uint8_t* codes, int64_t n, int n_sub, const float* lut, uint32_t* out_bits) {
    for (int64_t i = 0; i < n; i++) {
        float s = 0.0f;
        for (int m = 0; m < n_sub; m++) s += lut[m * 256 + codes[i * n_sub + m]];
        out_bits[i] = f32_bits(65536.0f - s);
    }
}

/* Exact re-scoring of candidates: bits(65536 - <q, K[ids[i]]>). */
void dco_rerank_scores(const uint16_t* keys, int dim, int dtype, const uint16_t* q, const uint32_t* ids, int64_t n_ids,
                       int exact, uint32_t* out_bits) {
    float qf[1024];
    for (int d = 0; d < dim; d++) qf[d] = elem_to_f32(q[d], dtype);
    for (int64_t i = 0; i < n_ids; i++) out_bits[i] = dist_bits_one(keys + (int64_t)ids[i] * dim, qf, dim, dtype, exact);
}

int dco_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ---- adaptive budget ("k-check"): power-law estimate of the attention mass of the top-h keys ---- */

/*
 * fit_alpha_from_logits (diffcache_cpu/src/nsw.rs:198-246): least-squares fit of
 * logit = a + b*ln(rank) over ranks min_rank..h (1-based), alpha = -b.  Sums in
 * double, alpha returned as float.  Returns 0 where the reference returns None.
 */
int dco_fit_alpha(const float* logits_sorted, int h, int min_rank, float* alpha_out) {
    if (h == 0 || min_rank == 0 || min_rank >= h) return 0;
    double n = (double)(h - min_rank + 1);
    if (n < 2.0) return 0;
    double sx = 0, sy = 0, sxx = 0, sxy = 0;
    for (int idx = min_rank - 1; idx < h; idx++) {
        double x = log((double)(idx + 1));
        double y = (double)logits_sorted[idx];
        sx += x; sy += y; sxx += x * x; sxy += x * y;
    }
    double denom = n * sxx - sx * sx;
    if (fabs(denom) < 1e-12) return 0;
    double b = (n * sxy - sx * sy) / denom;
    *alpha_out = (float)(-b);
    return 1;
}

/*
 * estimate_top_h_mass (nsw.rs:248-283): head = sum_{i<h} exp(z_i - max), tail =
 * exp(z_h - max) * h / (alpha - 1), mass = head / (head + tail); fp32 arithmetic.
 */
int dco_top_h_mass(const float* logits_sorted, int n, int h, float alpha, float* mass_out) {
    if (h == 0 || h > n) return 0;
    if (alpha <= 1.0f) return 0;
    float mx = logits_sorted[0];
    for (int i = 1; i < h; i++) if (logits_sorted[i] > mx) mx = logits_sorted[i];
    float head = 0.0f;
    for (int i = 0; i < h; i++) head += expf(logits_sorted[i] - mx);
    float vh = expf(logits_sorted[h - 1] - mx);
    float tail = vh * (float)h / (alpha - 1.0f);
    float denom = head + tail;
    if (denom <= 0.0f) return 0;
    *mass_out = head / denom;
    return 1;
}

/*
 * k_check_early_stoppable (nsw.rs:285-300) on the h best ranking keys (ascending dist):
 * logit = (65536 - dist) / sqrt(dim), fit from rank 5, stoppable iff mass >= threshold.
 * alpha_out / mass_out (may be NULL) receive the intermediate values (NaN where undefined).
 */
int dco_k_check(const uint32_t* dist_bits_sorted, int h, int dim, float threshold, float* alpha_out, float* mass_out) {
    float* z = (float*)malloc(sizeof(float) * (size_t)(h > 0 ? h : 1));
    float sq = sqrtf((float)dim);
    for (int i = 0; i < h; i++) z[i] = (65536.0f - bits_f32(dist_bits_sorted[i])) / sq;
    float alpha = NAN, mass = NAN;
    int ok = dco_fit_alpha(z, h, 5, &alpha);
    if (ok) ok = dco_top_h_mass(z, h, h, alpha, &mass);
    if (alpha_out) *alpha_out = alpha;
    if (mass_out) *mass_out = mass;
    free(z);
    return ok && mass >= threshold;
}

/*
 * The budget the reference's search would stop at (nsw.rs:339-376): the first
 * checkpoint h of k_check_seq (h < k) whose top-h keys pass the k-check; k otherwise.
 */
int dco_adaptive_budget(const uint32_t* dist_bits_sorted, int k, int dim, const int* seq, int n_seq, float threshold) {
    for (int e = 0; e < n_seq; e++) {
        int h = seq[e];
        if (h >= k) break;
        if (dco_k_check(dist_bits_sorted, h, dim, threshold, NULL, NULL)) return h;
    }
    return k;
}
