/*
 * diffcache_b200 — C ABI of the B200 (sm_100a) retrieval-attention engine.
 *
 * This is the boundary a maintainer of DiffCache binds instead of the Rust/pyo3
 * module `diffcache._cpu` (diffcache_cpu/src/lib.rs:523-672).  Every entry point
 * is plain C: opaque handle, raw pointers, sizes, and a CUDA stream passed as a
 * 64-bit integer (the same convention the reference uses for `query_streaming`,
 * diffcache_cpu/src/lib.rs:626-636).
 *
 * Conventions
 *  - Every function returns 0 on success and a negative DC_E* code on failure;
 *    nothing aborts, traps or throws across this boundary.  `dc_last_error()`
 *    returns a thread-local, human readable description of the last failure.
 *    (The reference reports the same conditions as Rust panics:
 *    diffcache_cpu/src/lib.rs:332-333,353-354,376,579.)
 *  - Element types cross the boundary as 16-bit patterns (bf16 or fp16), exactly
 *    as the reference passes numpy uint16 views (diffcache_cpu/src/lib.rs:528-544).
 *  - Unless stated otherwise a function only enqueues work on `stream` and
 *    returns; device buffers must stay alive until that work completed.
 *  - "problem" p = b * kv_heads + h is one (batch, kv-head) pair: one
 *    `nsw::Index` of the reference (diffcache_cpu/src/lib.rs:296-313).
 *  - Ranking key: dist = 65536.0f - dot(q, k) in fp32, compared by its raw bit
 *    pattern, ties broken by the smaller row id
 *    (diffcache_cpu/src/nsw.rs:74-91,129-139,600-615).
 */
#ifndef DIFFCACHE_B200_H
#define DIFFCACHE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DC_OK 0
#define DC_EINVAL (-1)   /* bad argument / shape (reference: assert!/panic!) */
#define DC_ECUDA (-2)    /* a CUDA runtime call failed */
#define DC_ENOMEM (-3)   /* device allocation failed */
#define DC_ESTATE (-4)   /* call not valid in the engine's current state */
#define DC_EDEVICE (-5)  /* a kernel reported an internal error status */

#define DC_BF16 0
#define DC_FP16 1

/* Largest top-k / ef a select call accepts (reference: MAX_EF, diffcache_cpu/src/nsw.rs:14-20). */
#define DC_MAX_TOPK 16384

typedef struct dc_engine dc_engine;

/* Description of the last failure on the calling thread ("" if none). */
const char* dc_last_error(void);

/* Library/ABI version (major*10000 + minor*100 + patch). */
int dc_version(void);

/* ------------------------------------------------------------------------- *
 * Engine object: one per layer, as in src/diffcache/kvcache/diffcache.py:87-100
 * ------------------------------------------------------------------------- */

/*
 * Replaces DiffCacheCPU.__new__ (diffcache_cpu/src/lib.rs:553-589) and
 * DataLayer::new / Index::new (lib.rs:293-324, nsw.rs:680-698).
 * Allocates the engine-owned HBM store K,V[bsz*kv_heads][max_ctx_len][head_dim]
 * plus all per-step scratch, on CUDA device `device`.  head_dim must be 64, 128
 * or 256; q_heads must be a multiple of kv_heads (lib.rs:294).
 */
int dc_create(int bsz, int q_heads, int kv_heads, int head_dim, int64_t max_ctx_len,
              int dtype, int device, dc_engine** out);

/* Frees everything dc_create allocated.  Synchronises the device first. */
int dc_destroy(dc_engine* e);

/*
 * Sequence-sharded engines: the rows this engine holds are rows
 * [row_offset, row_offset + ctx_len) of a longer logical sequence.  Row ids
 * reported by dc_local_topk are local + row_offset.  Default 0.  No counterpart
 * in the reference (it is single-process, src/diffcache/base.py:28).
 */
int dc_set_row_offset(dc_engine* e, int64_t row_offset);

/*
 * Replaces DiffCacheCPU.prefill (lib.rs:601-611) → DataLayer::prefill
 * (lib.rs:329-347) → Index::prefill (nsw.rs:497-528): copies seq_len rows per
 * problem into the store and sets ctx_len = seq_len.  `keys`/`vals` may be host
 * or device memory; strides are in elements for the (batch, kv-head, row) axes,
 * the head_dim axis must be contiguous.  The reference layout (B,Hkv,S,D)
 * contiguous is stride_b = Hkv*S*D, stride_h = S*D, stride_s = D; the model's
 * native (B,S,Hkv,D) layout is stride_b = S*Hkv*D, stride_h = D, stride_s = Hkv*D.
 * The reference's `neighbours` argument only feeds the NSW graph and has no
 * meaning for an exact scan, so it is not part of this ABI.
 */
int dc_prefill(dc_engine* e, const void* keys, const void* vals, int64_t seq_len,
               int64_t stride_b, int64_t stride_h, int64_t stride_s, uint64_t stream);

/*
 * Replaces DiffCacheCPU.insert (lib.rs:591-599) → Index::insert (nsw.rs:544-557):
 * appends one row per problem; keys/vals are (bsz, kv_heads, head_dim)
 * contiguous, host or device.  Fails with DC_ESTATE when the store is full.
 * The row index is read from the engine's device length word when the copy runs
 * (and the word is advanced there), so an insert captured into a CUDA graph
 * appends at the right place on every replay.
 */
int dc_insert(dc_engine* e, const void* keys, const void* vals, uint64_t stream);

/* Number of valid rows per problem (DataLayer.ctx_len, lib.rs:191).  Synchronises the device after
 * dc_window_push has been used (only the device knows how many rows were spilled into the store). */
int dc_ctx_len(dc_engine* e, int64_t* out);

/*
 * Replaces DiffCacheCPU.query (lib.rs:613-624) with use_bruteforce semantics:
 * DataLayer::query (lib.rs:373-404) → Index::search_bruteforce (nsw.rs:592-630).
 * q_mean is (bsz, kv_heads, head_dim); ef is clamped to ctx_len; row i of
 * out_keys/out_vals (bsz, kv_heads, ef, head_dim) is the i-th best row (smallest
 * (dist bits, row id) first).  out_idx (int32) and out_bits (uint32), each
 * (bsz, kv_heads, ef), are optional (NULL to skip).  All pointers may be host or
 * device memory; when any of them is host memory the call synchronises `stream`
 * before returning, as the reference call is synchronous.
 */
int dc_query(dc_engine* e, const void* q_mean, int ef, void* out_keys, void* out_vals,
             int32_t* out_idx, uint32_t* out_bits, uint64_t stream);

/*
 * Synchronises `stream` and reports DC_EDEVICE if a kernel of an earlier
 * asynchronous call on this engine flagged an internal inconsistency (the
 * kernels never trap; they record a status word and produce padded output).
 * The reference surfaces such conditions as Rust panics (e.g. nsw.rs:622).
 */
int dc_check_status(dc_engine* e, uint64_t stream);

/*
 * Replaces DiffCacheCPU.get_keys (lib.rs:646-649): fp32 copy of the stored keys,
 * (bsz, kv_heads, ctx_len, head_dim), host or device destination; synchronous.
 */
int dc_get_keys(dc_engine* e, float* out);

/*
 * Raw copy of the stored rows, keys_out/vals_out (bsz, kv_heads, ctx_len,
 * head_dim) 16-bit patterns, host or device; synchronous.  Feeds the snapshot
 * that replaces DiffCacheCPU.save (lib.rs:638-640, nsw.rs:704-733); the way
 * back is dc_prefill (DiffCacheCPU.load, lib.rs:642-644).
 */
int dc_export_rows(dc_engine* e, void* keys_out, void* vals_out);

/*
 * Replaces DiffCacheCPU.update_r_sq (lib.rs:651-659).  r_sq only enters the
 * graph-construction metric (nsw.rs:141-146), never the query ranking
 * (nsw.rs:129-139), so an exact scan only validates n == kv_heads.
 */
int dc_update_r_sq(dc_engine* e, const float* r_sq, int n);

/*
 * The fused decode step.  Replaces, for one layer, the chain
 *   DiffCache.decode_pre_query_operation  (src/diffcache/kvcache/diffcache.py:191-194)
 *   DiffCache.decode_query_kvcache        (diffcache.py:211-223)
 *   DiffCache.decode_post_query_operation (diffcache.py:196-209)
 *   flash_attn_with_kvcache(...)          (src/diffcache/base.py:134-142)
 * without leaving HBM: group-mean query → score scan over the store → exact
 * top-k → softmax attention of every query head over
 * [top-k rows | resident rows | new token].
 *
 *  q        (bsz, q_heads, head_dim) device
 *  k_new, v_new  (bsz, kv_heads, head_dim) device, or both NULL.  When given,
 *           the new token takes part in attention as the last row and is also
 *           appended to the resident buffers at row res_len (what flash-attn's
 *           in-place append does), so res_k/res_v need room for res_len+1 rows.
 *  res_k, res_v  resident (sink + local window) rows on the device,
 *           element strides res_stride_b / res_stride_h, row stride head_dim;
 *           in the reference layout this is kbuf[:, :, budget:, :]
 *           (diffcache.py:48-66).  May be NULL when res_len == 0 and k_new == NULL.
 *  topk     clamped to ctx_len; 0 skips retrieval.
 *  scale    softmax scale; <= 0 selects head_dim^-0.5 (flash-attn default).
 *  out      (bsz, q_heads, head_dim) device, engine dtype.
 *  out_idx  optional (bsz, kv_heads, k) int32 selected rows, best first, k = min(topk, rows), where rows is
 *           ctx_len — or max_ctx_len when the call is being captured into a CUDA graph or follows
 *           dc_window_push (the launches are then sized for the whole store; entries beyond the rows the
 *           store holds are 0xFFFFFFFF).
 *  out_lse  optional (bsz, q_heads) fp32 natural-log sum-exp of scaled scores.
 */
int dc_decode_attend(dc_engine* e, const void* q, const void* k_new, const void* v_new,
                     void* res_k, void* res_v, int64_t res_stride_b, int64_t res_stride_h,
                     int res_len, int topk, float scale, void* out, int32_t* out_idx,
                     float* out_lse, uint64_t stream);

/*
 * dc_decode_attend for inputs that are slices of a fused q/k/v projection output (what a model's
 * attention block holds at this point, src/diffcache/llama.py:181-195): inside a batch the heads are
 * dense, but q_stride_b (new_stride_b) elements separate two batches of q (of k_new and v_new, which
 * must share it).  0 means dense, i.e. dc_decode_attend.  Strides are multiples of 8 elements.
 */
int dc_decode_attend_strided(dc_engine* e, const void* q, int64_t q_stride_b, const void* k_new,
                             const void* v_new, int64_t new_stride_b, void* res_k, void* res_v,
                             int64_t res_stride_b, int64_t res_stride_h, int res_len, int topk, float scale,
                             void* out, int32_t* out_idx, float* out_lse, uint64_t stream);

/*
 * Decode loop with every length on the device, so that ONE captured CUDA graph per
 * layer serves the whole generation (the reference captures two graphs per layer,
 * src/diffcache/base.py:116-155, and updates `cache_seqlens` between replays).
 *
 * window_state is 8 int32 device words shared by all layers of a model:
 *   {suffix_len, head, prefix_len, cap, res_len_now, steps, 0, 0}
 * The resident buffer of a (batch, kv head) holds prefix_len sink rows followed by
 * `cap` window slots (the reference's kvbuf suffix region of kvbuf_suffix_maxlen
 * rows, src/diffcache/kvcache/diffcache.py:48-66).  The caller initialises
 * suffix_len, prefix_len and cap (head = 0) after prefill.
 *
 * dc_window_push: appends the step's new token to this layer's window.  While the
 * window is not full it goes to slot suffix_len.  Once it is full the oldest token
 * (slot head) is first appended to the scanned store — DataLayer::insert
 * (diffcache_cpu/src/lib.rs:352-369, Index::insert nsw.rs:544-557), which the
 * reference never calls: it stops at `assert kvbuf_suffix_len < kvbuf_suffix_maxlen`
 * (diffcache.py:221) — and the new token takes its slot.  Writes res_len_now =
 * prefix_len + min(suffix_len + 1, cap).  If the store is full too, the oldest
 * token is dropped and status 302 is recorded (dc_check_status).
 * dc_window_advance: once per decode step, after the last layer's push: suffix_len
 * grows until cap, then head moves round the ring (diffcache.py:222-223).
 * dc_decode_attend_dyn: dc_decode_attend_strided without a new token (it already
 * sits in the window) and with the resident length read from *res_len_dev when the
 * kernels run; res_cap (>= any value that word takes) only sizes the launch.  The
 * number of stored rows is likewise read from the engine's device word.
 * After dc_window_push the host no longer knows the row count without asking the
 * device: dc_ctx_len synchronises, and launches are sized for max_ctx_len.
 */
int dc_window_push(dc_engine* e, const void* k_new, const void* v_new, int64_t new_stride_b, void* res_k, void* res_v,
                   int64_t res_stride_b, int64_t res_stride_h, int32_t* window_state, uint64_t stream);
int dc_window_advance(int32_t* window_state, uint64_t stream);
int dc_decode_attend_dyn(dc_engine* e, const void* q, int64_t q_stride_b, void* res_k, void* res_v,
                         int64_t res_stride_b, int64_t res_stride_h, const int32_t* res_len_dev, int res_cap, int topk,
                         float scale, void* out, int32_t* out_idx, float* out_lse, uint64_t stream);

/*
 * Adaptive retrieval budget.  Replaces the k-check early stop of the reference's
 * search (fit_alpha_from_logits / estimate_top_h_mass / k_check_early_stoppable,
 * diffcache_cpu/src/nsw.rs:198-300, applied at the checkpoints of `k_check_seq`,
 * nsw.rs:339-376; options `k_check_seq`, `attn_mass_threshold`, lib.rs:565-566):
 * after the exact top-k, per problem the first checkpoint h < topk whose top-h
 * logits (65536 - dist) / sqrt(head_dim) pass the power-law mass test becomes the
 * budget, and dc_decode_attend attends only over the h best rows (plus resident
 * rows and the new token).  n_seq = 0 switches it off (default).  The test runs
 * on the device; dc_get_budget copies the (bsz*kv_heads) int32 budgets of the
 * last step (host or device destination).
 */
int dc_set_adaptive_budget(dc_engine* e, const int32_t* k_check_seq, int n_seq, float attn_mass_threshold);
int dc_get_budget(dc_engine* e, int32_t* out, uint64_t stream);

/*
 * Per-phase device timing of dc_decode_attend, the counterpart of the reference's
 * `{name}_search_latency` / `{name}_collect_latency` / `{name}_total_query_latency`
 * counters (diffcache_cpu/src/nsw.rs:618,660, diffcache_cpu/src/lib.rs:403).
 * dc_set_phase_timing(e, n) makes the next n calls of dc_decode_attend record CUDA
 * events on their stream around the scan, select and attend phases (n = 0 turns
 * it off; not usable while the stream is being captured into a graph).
 * dc_get_phase_times synchronises those events and returns the SUM in milliseconds
 * of each phase over the `*steps` recorded calls.
 */
int dc_set_phase_timing(dc_engine* e, int max_steps);
int dc_get_phase_times(dc_engine* e, float* scan_ms, float* select_ms, float* attend_ms, int* steps);

/*
 * Kernel-by-kernel trace of the sequence-sharded step (dc_local_topk / dc_sharded_*): after
 * dc_trace_begin(e, n) the next calls record a CUDA event on their stream before the scan and after
 * every kernel they launch (scan, select, key push, prefix count, attention + split merge, partial
 * push, final merge), up to n events; dc_trace_read synchronises the last one, returns the
 * *n_marks - 1 intervals between consecutive events in milliseconds and closes the trace.  Same
 * purpose as dc_set_phase_timing; not usable during graph capture.
 */
int dc_trace_begin(dc_engine* e, int max_marks);
int dc_trace_read(dc_engine* e, float* intervals_ms, int* n_marks);

/* ------------------------------------------------------------------------- *
 * Sequence-sharded decode (one engine per GPU holds a contiguous row range).
 * No counterpart in the reference (single GPU); the semantics are those of the
 * single-engine path applied to the concatenated rows.
 * ------------------------------------------------------------------------- */

/*
 * Local half of a sharded step: group-mean query, scan of this engine's rows,
 * local top-k.  out_bits/out_gidx are (bsz*kv_heads, topk) uint32, best first;
 * out_gidx = local row + row_offset.  When ctx_len < topk the tail is padded
 * with bits = 0xFFFFFFFF, gidx = 0xFFFFFFFF (never selected by a merge).
 */
int dc_local_topk(dc_engine* e, const void* q, int topk, uint32_t* out_bits,
                  uint32_t* out_gidx, uint64_t stream);

/*
 * Second half: attention of every query head over the rows of `sel_gidx`
 * ((bsz*kv_heads, n_sel) uint32, global ids) that this engine owns, plus the
 * resident rows / new token given (pass res_len = 0 and NULLs on ranks that hold
 * neither sink nor window).  Writes un-normalised partial results:
 *   out_acc (bsz, q_heads, head_dim) fp32 = sum_j exp(s_j - m) v_j
 *   out_ml  (bsz, q_heads, 2) fp32 = (m in log2 units, l = sum_j exp2(s_j - m))
 * which dc_lse_combine merges.  sel_count (may be NULL): per problem, only the
 * first sel_count[p] entries of its id list are attended (what
 * dc_merge_sorted_count returns for this rank's own candidate list).
 */
int dc_attend_owned(dc_engine* e, const void* q, const uint32_t* sel_gidx, int n_sel,
                    const void* k_new, const void* v_new, void* res_k, void* res_v,
                    int64_t res_stride_b, int64_t res_stride_h, int res_len, float scale,
                    float* out_acc, float* out_ml, const int32_t* sel_count, uint64_t stream);

/* ------------------------------------------------------------------------- *
 * Peer exchange: the two all-gathers of a sequence-sharded step done by plain
 * stores over NVLink into buffers the ranks have mapped from one another, fused
 * with the kernels that consume the data (no collective library, no Python).
 * No counterpart in the reference (single process, single GPU).
 *
 * Set-up, once: every rank calls dc_xchg_create (its own buffer: per channel
 * `world` slots of slot_bytes[c] payload bytes, multiples of 16), hands the
 * dc_xchg_handle_bytes()-byte handle of dc_xchg_get_handle to every other rank
 * over any side channel (it is a cudaIpcMemHandle_t), and maps each peer with
 * dc_xchg_open_peer; ranks that live in the same process use dc_xchg_set_peer
 * with dc_xchg_local() of the peer instead.  All ranks must have finished this
 * before the first push (a host barrier).
 *
 * Wire format: every 32-bit word is stored as an 8-byte pair {word, epoch}; a
 * reader that finds the epoch it expects has the word that came with it, so
 * arrival needs no fence and no separate flag.
 * dc_xchg_push(channel, src, bytes): sends `bytes` (multiple of 16) from device
 * memory `src` into slot `rank` of the channel in EVERY rank's buffer, tagged
 * with the channel's next epoch.
 * dc_xchg_push_rows(channel, src, rows, row_bytes): the same for a (rows,
 * row_bytes) block that is to be interleaved with the other ranks' blocks row by
 * row: the channel then holds (rows, world, row_bytes), i.e. the concatenation
 * along the last axis (an all-gather of head slices).
 * dc_xchg_collect(channel, dst, bytes): a kernel that waits until the first
 * `bytes` payload bytes of this rank's copy of the channel carry the current
 * epoch (every one of them must have been pushed in this exchange) and writes
 * them densely to device memory `dst`.  The sharded step below does not need it:
 * its consumer kernels read the pairs themselves.
 * Every rank must issue the same sequence of pushes.  Waits are bounded (2 s by
 * default, dc_xchg_set_timeout_ms or the environment variable
 * DC_XCHG_TIMEOUT_MS): when one runs out, the kernel records a status, finishes
 * on zeros, and dc_xchg_check (synchronises `stream`) returns DC_EDEVICE — a
 * missing peer never hangs the GPU.
 * ------------------------------------------------------------------------- */
typedef struct dc_xchg dc_xchg;
int dc_xchg_create(int rank, int world, int device, const int64_t* slot_bytes, int n_channels, dc_xchg** out);
int dc_xchg_destroy(dc_xchg* x);
int dc_xchg_handle_bytes(void);
int dc_xchg_get_handle(dc_xchg* x, void* handle_out);
int dc_xchg_open_peer(dc_xchg* x, int peer_rank, const void* handle);
int dc_xchg_set_peer(dc_xchg* x, int peer_rank, void* peer_base);
void* dc_xchg_local(dc_xchg* x);
int dc_xchg_set_timeout_ms(dc_xchg* x, int ms);
int dc_xchg_push(dc_xchg* x, int channel, const void* src, int64_t bytes, uint64_t stream);
int dc_xchg_push_rows(dc_xchg* x, int channel, const void* src, int64_t rows, int64_t row_bytes, uint64_t stream);
int dc_xchg_collect(dc_xchg* x, int channel, void* dst, int64_t bytes, uint64_t stream);
int dc_xchg_check(dc_xchg* x, uint64_t stream);

/*
 * One rank's share of a sequence-sharded decode step over a peer exchange whose
 * channel 0 / channel 1 slots hold at least the two sizes dc_sharded_slot_bytes
 * reports (candidate keys; partial attention results):
 *   dc_sharded_local    scan + local top-k of this engine's rows, keys pushed to every rank;
 *   dc_sharded_attend   waits for all ranks' keys, counts the prefix of this rank's own list that is
 *                       globally selected (dc_merge_sorted_count), attends over it (dc_attend_owned;
 *                       resident rows / new token as given there) and pushes the partial result;
 *   dc_sharded_combine  waits for all ranks' partials and merges them by log-sum-exp into `out`
 *                       (bsz, q_heads, head_dim), identical on every rank.
 * dc_sharded_decode_attend is the whole step as one call and five kernels on `stream` (scan; select,
 * which also stores the keys into every rank's buffer; prefix count; attention; split merge, which
 * also stores the partials into every rank's buffer and then waits for the other ranks' partials and
 * writes the final merge; topk must be even), capturable in a CUDA graph once the first call has
 * allocated the per-engine buffers.  Its last kernel waits for data that the same kernel of the
 * OTHER ranks sends, so every rank must run on its own GPU; ranks that share a GPU (tests) call
 * the three phase functions, all ranks' phase n before any rank's phase n + 1.
 * Results are those of dc_decode_attend on the concatenated rows (same ranking keys, ties to the
 * smaller global row id: nsw.rs:74-91,612).
 */
int dc_sharded_slot_bytes(dc_engine* e, int topk, int64_t* out2);
/*
 * Head-sharded layers (every rank holds some kv heads of a layer and needs all ranks' attention outputs for
 * the output projection): after dc_set_output_exchange(e, x, channel) every dc_decode_attend* call of this
 * engine also stores its (bsz, q_heads, head_dim) output into every rank's copy of the channel, interleaved so
 * that the channel holds (bsz, world, q_heads * head_dim) — the stores are part of the kernel that produces
 * the output.  The consumer gets it with dc_xchg_collect.  The channel's slot must be bsz * q_heads * head_dim
 * * 2 bytes; x = NULL switches it off.  Consecutive exchanges must use different channels (one per layer,
 * round-robin) unless something else orders the ranks between them.
 */
int dc_set_output_exchange(dc_engine* e, dc_xchg* x, int channel);
/*
 * With dc_set_output_gather(e, dense) the kernel that stores the slice also does the consumer's side: it then
 * waits, in this rank's copy of the channel, for the same output rows of every rank and writes all slices
 * densely to `dense` ((bsz, world * q_heads * head_dim) elements, device memory) - the all-gather is complete
 * when the decode call's kernels are, without dc_xchg_collect.  Every rank must run on its own GPU (the kernel
 * waits for what the same kernel of the other ranks sends).  dense = NULL switches it off;
 * dc_set_output_exchange(e, NULL, ..) does too.
 */
int dc_set_output_gather(dc_engine* e, void* dense);
int dc_sharded_local(dc_engine* e, dc_xchg* x, const void* q, int topk, uint64_t stream);
int dc_sharded_attend(dc_engine* e, dc_xchg* x, const void* q, const void* k_new, const void* v_new, void* res_k,
                      void* res_v, int64_t res_stride_b, int64_t res_stride_h, int res_len, float scale, uint64_t stream);
int dc_sharded_combine(dc_engine* e, dc_xchg* x, void* out, float* out_lse, uint64_t stream);
int dc_sharded_decode_attend(dc_engine* e, dc_xchg* x, const void* q, const void* k_new, const void* v_new, void* res_k,
                             void* res_v, int64_t res_stride_b, int64_t res_stride_h, int res_len, int topk, float scale,
                             void* out, float* out_lse, uint64_t stream);

/* ------------------------------------------------------------------------- *
 * Stateless kernels (device pointers only).  The engine calls are compositions
 * of these; they are exported for sharded drivers and for parity tests.
 * ------------------------------------------------------------------------- */

/*
 * Score scan = the loop body of Index::search_bruteforce (nsw.rs:601-607) with
 * Index::distance QKDist (nsw.rs:129-139).  keys: n_prob problems of n rows,
 * problem stride `prob_stride` elements, row stride head_dim.  q_mode 0: q is
 * (n_prob, head_dim) already group-averaged; q_mode 1: q is (n_prob*group,
 * head_dim) query heads and the group mean (fp32 sum in head order, times
 * 1/group, rounded to the element type — torch's `.mean(dim=2)` of
 * diffcache.py:193) is formed in the kernel prologue.  Writes
 * scores[p*score_stride + i] = bits(65536.0f - dot) and, if minmax != NULL,
 * atomically folds (min, max) of those bits into minmax[2p], minmax[2p+1]
 * (caller initialises to 0xFFFFFFFF, 0).
 */
int dc_score_scan(const void* keys, int64_t prob_stride, int n_prob, int64_t n, int head_dim,
                  int dtype, const void* q, int q_mode, int group, uint32_t* scores,
                  int64_t score_stride, uint32_t* minmax, uint64_t stream);

/*
 * Exact top-k select = the BinaryHeap<u64> of search_bruteforce
 * (nsw.rs:600-615,621): the k smallest 64-bit keys (bits << 32 | id), ascending.
 * bits: (n_prob, n) with row stride in_stride.  ids == NULL means id = position.
 * minmax (2 per problem) may be NULL (computed in the kernel).  out_bits /
 * out_ids: (n_prob, k) with row stride out_stride; either may be NULL.  When
 * k > n the tail beyond n is padded with 0xFFFFFFFF (bits and ids).  `scratch` must hold dc_select_scratch_bytes(n_prob) zeroed bytes (a status
 * word: a non-zero value after the call reports an internal inconsistency).
 */
int dc_topk_select(const uint32_t* bits, const uint32_t* ids, int64_t in_stride, int n_prob,
                   int64_t n, int k, const uint32_t* minmax, uint32_t* out_bits,
                   uint32_t* out_ids, int64_t out_stride, void* scratch, uint64_t stream);
int64_t dc_select_scratch_bytes(int n_prob);

/*
 * Sparse gather-attention + split-K merge = flash_attn_with_kvcache over the
 * gathered buffer (base.py:134-142), reading rows in place.  Store pointers as in
 * dc_score_scan; sel (n_prob, sel_stride) uint32 row ids minus `sel_base`; only
 * ids with sel_base <= id < sel_base + n_rows are attended (others are skipped).
 * Exactly one of (out, out_acc/out_ml) must be given: `out` is the normalised
 * result in the element type, out_acc/out_ml the un-normalised partials.
 * `scratch` must hold dc_attend_scratch_bytes(n_prob, group, head_dim) bytes.
 */
int dc_sparse_attend(const void* k_store, const void* v_store, int64_t prob_stride, int64_t n_rows,
                     int n_prob, int kv_heads, int group, int head_dim, int dtype, const void* q,
                     const uint32_t* sel, int64_t sel_stride, int n_sel, int64_t sel_base,
                     const void* k_new, const void* v_new, void* res_k, void* res_v,
                     int64_t res_stride_b, int64_t res_stride_h, int res_len, float scale,
                     void* out, float* out_lse, float* out_acc, float* out_ml, void* scratch,
                     uint64_t stream);
int64_t dc_attend_scratch_bytes(int n_prob, int group, int head_dim);

/*
 * dc_sparse_attend for callers that cannot allocate device memory (no
 * counterpart in the reference).  A host that gives all of HBM to its own pool
 * at start-up, or that may not call cudaMalloc while serving because it
 * synchronises the device, has no buffer to pass as `scratch`; here the split-K
 * scratch is a fixed DC_NOALLOC_SCRATCH_BYTES array inside the library image
 * (held by every GPU that loads the library until the process exits), and the
 * call allocates nothing.  Arguments and results are those of dc_sparse_attend
 * without `scratch`.  Problems whose partials do not fit are rejected with
 * DC_EINVAL and a message naming both sizes (the need is
 * n_prob * splits * group * (head_dim + 2) * 4 bytes, with splits chosen so that
 * n_prob * splits is about two CTAs per SM, the same rule dc_sparse_attend uses;
 * the environment variable DC_ATTEND_CTAS_PER_SM can raise that to at most four).
 * The first call on a device looks the array's device address up (once, under
 * a lock, so concurrent first calls are safe) and should therefore come before
 * any stream capture.  All calls on a device share the array: calls whose
 * kernels overlap on the GPU race and must be serialised by the caller; stale
 * contents from an earlier call are harmless (every slot is written before it
 * is read).
 */
#define DC_NOALLOC_SCRATCH_BYTES (4 * 1024 * 1024)
int dc_sparse_attend_noalloc(const void* k_store, const void* v_store, int64_t prob_stride, int64_t n_rows,
                             int n_prob, int kv_heads, int group, int head_dim, int dtype, const void* q,
                             const uint32_t* sel, int64_t sel_stride, int n_sel, int64_t sel_base,
                             const void* k_new, const void* v_new, void* res_k, void* res_v,
                             int64_t res_stride_b, int64_t res_stride_h, int res_len, float scale,
                             void* out, float* out_lse, float* out_acc, float* out_ml, uint64_t stream);

/*
 * Merge of per-rank candidate lists for a sequence-sharded search, without
 * moving row ids.  bits_all: (world, n_prob, k) uint32, the ascending ranking
 * keys that dc_local_topk wrote on every rank (0xFFFFFFFF pads), as an
 * all-gather delivers them.  Ranks own contiguous, ascending row ranges, so on
 * equal keys a lower rank's rows come first (the reference's tie rule, smaller
 * row id wins: nsw.rs:74-91,612).  The global k best that `my_rank` owns are a
 * prefix of its own list; out_count[p] (int32, n_prob) receives its length, to
 * be passed to dc_attend_owned as sel_count together with this rank's own id
 * list.  Requires world * k * 4 bytes <= 200 KB (DC_EINVAL otherwise: merge
 * (bits, id) pairs with dc_topk_select instead).  No counterpart in the
 * reference, which is single-process.
 */
int dc_merge_sorted_count(const uint32_t* bits_all, int world, int n_prob, int k, int my_rank,
                          int32_t* out_count, uint64_t stream);

/*
 * Log-sum-exp merge of `n_part` partial results (split-K partials of one GPU, or
 * the per-rank partials an all-gather delivers): part i holds
 * acc_i = acc + i*acc_part_stride, (rows, head_dim) fp32, and
 * ml_i = ml + i*ml_part_stride, (rows, 2) fp32 = (max in log2 units, sum); strides
 * in floats.  Writes out (rows, head_dim) in the element type and optional
 * lse (rows) fp32.  No counterpart in the reference (flash-attn merges its own
 * splits internally, src/diffcache/base.py:134-142).
 */
int dc_lse_combine(const float* acc, int64_t acc_part_stride, const float* ml, int64_t ml_part_stride,
                   int n_part, int64_t rows, int head_dim, int dtype, void* out, float* out_lse,
                   uint64_t stream);

/*
 * The k-check on its own: sel_bits (n_prob, stride) best-first ranking keys as
 * written by dc_topk_select, k of them valid per problem; out_budget (n_prob)
 * int32 on the device; k_check_seq is a host array (nsw.rs:198-300,339-376).
 */
int dc_adaptive_budget(const uint32_t* sel_bits, int64_t stride, int n_prob, int k, int head_dim,
                       const int32_t* k_check_seq, int n_seq, float attn_mass_threshold, int32_t* out_budget,
                       uint64_t stream);

/* Gather rows: out[p][i][:] = store[p][ids[p][i]][:]  (nsw.rs:623-629). */
int dc_gather_rows(const void* store, int64_t prob_stride, int n_prob, int head_dim,
                   const uint32_t* ids, int64_t ids_stride, int n_ids, void* out, uint64_t stream);

/* ------------------------------------------------------------------------- *
 * Product-quantisation baseline (asymmetric distance + exact rerank).
 * No counterpart in the reference: evaluation/impl/pqcache is an empty
 * directory.  Definition: M subspaces of head_dim/M dims, 256 centroids each;
 * lut[m][c] = <q_m, centroid[m][c]> (fp32, dims in order), score =
 * sum_m lut[m][code[m]] in increasing m, ranking key = bits(65536.0f - score).
 * ------------------------------------------------------------------------- */

/* lut (n_prob, M, 256) fp32 from q (n_prob, head_dim, element type; q_mode as in
 * dc_score_scan) and centroids (n_prob, M, 256, head_dim/M) fp32. */
int dc_pq_build_lut(const void* q, int q_mode, int group, int dtype, const float* centroids,
                    int n_prob, int head_dim, int n_sub, float* lut, uint64_t stream);

/* ADC scan over codes (n_prob, n, M) uint8 → scores/minmax as dc_score_scan. */
int dc_pq_adc_scan(const uint8_t* codes, int64_t prob_stride, int n_prob, int64_t n, int n_sub,
                   const float* lut, uint32_t* scores, int64_t score_stride, uint32_t* minmax,
                   uint64_t stream);

/* Exact re-scoring of candidate rows: out_bits[p][i] = bits(65536 - <q_p, K[p][ids[p][i]]>). */
int dc_rerank_scores(const void* keys, int64_t prob_stride, int n_prob, int head_dim, int dtype,
                     const void* q, int q_mode, int group, const uint32_t* ids, int64_t ids_stride,
                     int n_ids, uint32_t* out_bits, uint64_t stream);

#ifdef __cplusplus
}
#endif
#endif /* DIFFCACHE_B200_H */
