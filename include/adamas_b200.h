/*
 * adamas_b200 -- C ABI of the B200 (sm_100a) implementation of the Adamas decode hot path.
 *
 * Every entry point takes raw device pointers, plain integers and a CUDA stream, and returns an
 * int status (0 = ADAMAS_OK).  No entry point synchronises the stream.  On failure a
 * human-readable message is available from adamas_last_error() (thread-local).
 *
 * Each declaration cites the reference interface it replaces as <file>:<line> relative to the
 * root of the FibonaccciYan/Adamas checkout.
 *
 * Memory layouts (identical to the reference's KvPool, adamas/utils/kv_cache.py:21-24, layout NHD):
 *   KV cache of one layer    [pages, 2, page_size, H, D]   fp16 or bf16   (item 0 = K, item 1 = V)
 *   code cache of one layer  [pages, 1, page_size, H, D/8] 16-bit words   (2-bit codes, 32 B per key)
 * A page table is an int32 array of physical page numbers in logical order.  Token t of a
 * sequence lives at page page_table[t / page_size], entry t % page_size.
 * Packed code word w of a (token, head) holds dimensions 8w..8w+7, dimension 8w+i at bits
 * [2i, 2i+1] (kernels/include/decode/decode_page.cuh:380-398).
 */
#ifndef ADAMAS_B200_H_
#define ADAMAS_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ADAMAS_ABI_VERSION 4

/* status codes */
#define ADAMAS_OK 0
#define ADAMAS_ERR_INVALID 1     /* bad argument (null pointer, unsupported shape, size out of range) */
#define ADAMAS_ERR_CUDA 2        /* a CUDA runtime call or kernel launch failed */
#define ADAMAS_ERR_STATE 3       /* call order violated (forward before begin_forward) */

/* element types of q/k/v and the KV cache (the reference dispatches fp16 only,
 * adamas/ops/csrc/pytorch_extension_utils.h:25-35; bf16 is an extension) */
#define ADAMAS_F16 0
#define ADAMAS_BF16 1

/* distance metric of the estimate */
#define ADAMAS_METRIC_L1 0       /* sum |qc - kc|: evaluation/adamas_attention.py:222 */
#define ADAMAS_METRIC_XOR 1      /* lowbit + 2*highbit of qc^kc: kernels/include/decode/decode_attn.cuh:192-193 */

/* value formats of distances / top-k keys */
#define ADAMAS_VAL_F16 0         /* IEEE fp16 (the reference's format) */
#define ADAMAS_VAL_U16 1         /* unsigned 16-bit integer */

typedef void* adamas_stream_t;   /* a cudaStream_t */

/* Grouped-query attention.  Where a function takes num_heads AND num_q_heads, num_heads is the head
 * count of the caches (KV heads) and num_q_heads that of the query side: q, o, q_code, lse, the
 * distance rows, the histogram scratch and the index lists have num_q_heads rows, and query head r
 * reads cache head r / (num_q_heads / num_heads).  num_q_heads must be a multiple of num_heads;
 * num_q_heads == num_heads is multi-head attention, the only case the reference supports
 * (kernels/include/decode/decode_handler.cuh:83 asserts num_qo_heads == num_kv_heads; its kernels
 * carry a group-size parameter, kernels/include/decode/decode_attn.cuh:706,873, that is always 1).  Functions with num_heads alone (the stand-alone append
 * forms that take a pre-transformed h, adamas_append_estimate, adamas_decode_forward_static) are
 * multi-head only. */

/* Scratch of the fused decode step ("histogram scratch"): 32-bit words per head.  The estimate launch
 * of a step counts the distances of every head into its first 16 * 512 words (one 512-bin histogram
 * per slice of the row, up to 16 slices); the select+attend launch reads the counts, passes the thread
 * blocks' partial attention results through the remaining words, and clears the counts and its
 * arrival counter again.  The caller allocates num_heads * ADAMAS_HIST_WORDS_PER_HEAD words and zeroes
 * them ONCE; every call that uses the table leaves it ready for the next one (histogram part all
 * zero).  Calls that may overlap on the GPU need separate tables. */
#define ADAMAS_HIST_WORDS_PER_HEAD (16 * 512 + 16 * 132)

int adamas_abi_version(void);
const char* adamas_last_error(void);

/* Reads (and optionally clears) the current device's error flags.  Kernels never spin without a
 * limit: one that gives up on a wait (bit 0: the estimate kernel's copy pipeline; bit 1: the decode
 * kernel's; bit 2: the gather of select+attend) sets a flag here and
 * finishes, leaving wrong results behind.  Bit 3: select+attend was given a histogram table that does
 * not describe its distance rows (not zeroed before the step, or shared by overlapping calls).  Synchronises with the device.  No counterpart in the
 * reference, whose kernels have no waits of this kind. */
int adamas_device_error(unsigned* flags, int clear);

/* Turns programmatic dependent launch of the decode-step kernels (append, estimate, top-k, sparse
 * decode) on or off for this process; on by default, ADAMAS_PDL=0 in the environment turns it off.
 * With it a kernel's set-up overlaps the tail of the kernel before it on the same stream; every
 * kernel still waits for its predecessor to complete before it reads that kernel's results.  The
 * reference launches everything on the legacy default stream (e.g. adamas/ops/csrc/page.cu:99). */
int adamas_set_pdl(int enable);

/* Chooses how the decode-step entry points launch a step of 16, 32 or 64 heads (multi-head attention):
 * with the append, and the rotary embedding if one is asked for, folded into the estimate launch (two
 * launches; the default) or as three launches (append, estimate, select+attend;
 * ADAMAS_FUSED_APPEND=0 in the environment selects it).  Other head counts and grouped queries always
 * take three.  Results are identical.  No counterpart in the reference. */
int adamas_set_fused_append(int enable);

/* How many blocks of the estimate kernel may be resident per SM: 2 (default; fastest for one sequence)
 * or 1, which leaves half of every SM's registers and shared memory to kernels running on other
 * streams, so that the select+attend of one sequence overlaps the estimate of another (a batch of
 * independent sequences, one stream each).  ADAMAS_EST_BLOCKS_PER_SM in the environment sets the initial
 * value.  No counterpart in the reference (batch 1 only). */
int adamas_set_estimate_blocks_per_sm(int blocks);

/* Upper bound (1, 2, 4 or 8; default 8, or ADAMAS_MAX_CLUSTER in the environment) on the number of
 * thread blocks that share one head in adamas_select_attend / adamas_decode_step.  8 means automatic:
 * eight blocks per head, or up to sixteen while all blocks of the launch are resident at once (the
 * shortest single call); fewer take longer per call but leave room on the
 * GPU for calls of other sequences running on other streams (a batch of independent sequences).  Rows
 * longer than 32768 x the bound are rejected.  No counterpart in the reference (batch 1 only). */
int adamas_set_max_cluster(int blocks);

/* ---- stage 1: Hadamard transform, bucketize, pack, append -------------------------------- */

/* y[r, :] = round_to_dtype(scale * WHT_D(x[r, :])) for r < rows; D = head_dim = 128; x == y allowed.
 * Replaces faster_hadamard_transform.hadamard_transform(x, inplace) (external module;
 * call sites adamas/models/Adamas.py:120,150). */
int adamas_hadamard_transform(const void* x, void* y, int64_t rows, int head_dim, float scale,
                              int dtype, adamas_stream_t stream);

/* Bucketize (thresholds[3], strict >) and pack rows of already-transformed values:
 * h [rows, D] -> codes [rows, D/8] 16-bit words.
 * Replaces pack_2bit / vec_bucketize_and_pack_2bit (kernels/include/decode/decode_page.cuh:380-398;
 * reference test helper adamas/tests/test_estimate.py:12-24). */
int adamas_bucketize_pack(const void* h, void* codes, int64_t rows, int head_dim,
                          const float* thresholds3_host, int dtype, adamas_stream_t stream);

/* Decode append of one token.  k, v [1,H,D]; h [2,H,D] with row 0 = transformed q, row 1 =
 * transformed k; q_code_out [1,H,D/8].  The token's position is
 * (kv_num_pages-1)*page_size + kv_last_page_len - 1; its code goes to entry code_last_page_len-1
 * of the last code page.
 * Replaces append_kv_cache_decode (adamas/ops/csrc/page.cu:6-109,
 * kernels/include/decode/decode_page.cuh:415-469,566-590). */
int adamas_append_decode(const void* k, const void* v, const void* h, void* q_code_out,
                         void* kv_data, const int32_t* kv_page_table, int kv_num_pages,
                         int kv_last_page_len,
                         void* code_data, const int32_t* code_page_table, int code_num_pages,
                         int code_last_page_len,
                         int num_heads, int head_dim, int page_size,
                         const float* thresholds3_host, int dtype, adamas_stream_t stream);

/* Same, with the Hadamard transform done inside: takes q and k (after RoPE) instead of h.
 * Replaces the torch.cat + hadamard_transform + append_kvh sequence of
 * adamas/models/Adamas.py:145-161 with one launch.
 * Ordering (all decode appends): the launch lets the kernel that follows it in the stream start its
 * input-independent part early (programmatic dependent launch), and an adamas_estimate that follows
 * streams the cached codes AS THEY WERE BEFORE this append while the append runs (it excludes the
 * newest token).  One append per cache between two estimates, as a decode step does, is always safe; two
 * appends to the same cache back to back followed by an estimate that is to see the first of them need
 * adamas_set_pdl(0) or an intervening launch. */
int adamas_append_decode_fused(const void* q, const void* k, const void* v, void* q_code_out,
                               void* kv_data, const int32_t* kv_page_table, int kv_num_pages,
                               int kv_last_page_len,
                               void* code_data, const int32_t* code_page_table, int code_num_pages,
                               int code_last_page_len,
                               int num_heads, int num_q_heads, int head_dim, int page_size, float scale,
                               const float* thresholds3_host, int dtype, adamas_stream_t stream);

/* In-place rotary position embedding (Llama rotate-half form, linear position scaling) of
 * q [seq_len, num_q_heads, D] and k [seq_len, num_kv_heads, D]; token s has position past_kv_len + s.
 * Replaces apply_rope_in_place (adamas/ops/csrc/page.cu:228-269,
 * kernels/include/decode/decode_page.cuh:642-726). */
int adamas_apply_rope_in_place(void* q, void* k, int64_t seq_len, int num_q_heads, int num_kv_heads,
                               int head_dim, int64_t past_kv_len, float rope_scale, float rope_theta,
                               int dtype, adamas_stream_t stream);

/* adamas_append_decode_fused with the rotary embedding in front: q and k [1,H,D] arrive un-rotated,
 * are rotated in place for the position of the token being appended, and are then transformed, coded
 * and stored.  One launch for apply_rope_in_place + torch.cat + hadamard_transform + append_kvh
 * (adamas/models/Adamas.py:113,145-161).  rope_inv_freq (optional, device, 64 floats) and rope_mscale:
 * a frequency table instead of (rope_scale, rope_theta), as in adamas_decode_step_dev. */
int adamas_append_decode_rope_fused(void* q, void* k, const void* v, void* q_code_out, void* kv_data,
                                    const int32_t* kv_page_table, int kv_num_pages, int kv_last_page_len,
                                    void* code_data, const int32_t* code_page_table, int code_num_pages,
                                    int code_last_page_len, int num_heads, int num_q_heads, int head_dim,
                                    int page_size, float scale, const float* thresholds3_host, float rope_scale,
                                    float rope_theta, const float* rope_inv_freq, float rope_mscale, int dtype,
                                    adamas_stream_t stream);

/* Prefill append of n_tokens tokens ending at the current sequence end.  k, v, h [n_tokens,H,D];
 * h holds transformed keys.  If h is NULL the transform of k is computed inside (scale used).
 * Replaces append_kv_cache_prefill (adamas/ops/csrc/page.cu:111-226,
 * kernels/include/decode/decode_page.cuh:486-548,607-640) and, with h == NULL, also the
 * hadamard_transform call of adamas/models/Adamas.py:120. */
int adamas_append_prefill(const void* k, const void* v, const void* h, int64_t n_tokens,
                          void* kv_data, const int32_t* kv_page_table, int kv_num_pages,
                          int kv_last_page_len,
                          void* code_data, const int32_t* code_page_table, int code_num_pages,
                          int code_last_page_len,
                          int num_heads, int head_dim, int page_size, float scale,
                          const float* thresholds3_host, int dtype, adamas_stream_t stream);

/* ---- stage 2: distance estimate ----------------------------------------------------------- */

/* out[h * out_stride + t] = distance(q_code[h], code of token t, head h) for t < n_tokens, where
 * n_tokens = (code_num_pages-1)*page_size + code_last_page_len - exclude_last; exclude_last = 1 leaves
 * the newest token out, as the reference does; 0 is for a sequence shard that does not hold it.
 * q_code [H, D/8]; out_format ADAMAS_VAL_F16 (reference) or ADAMAS_VAL_U16.
 * hist (optional, may be NULL): histogram scratch (see ADAMAS_HIST_WORDS_PER_HEAD) that additionally
 * receives the counts a following adamas_select_attend(..., hist_ready = 1) needs; hist_slices is then
 * the value adamas_select_attend_slices gives for that call.
 * Replaces estimate_attn_score (adamas/ops/csrc/estimate.cu:6-84,
 * kernels/include/decode/decode_attn.cuh:287-443,1144-1211). */
int adamas_estimate(const void* q_code, const void* code_data, const int32_t* code_page_table,
                    int code_num_pages, int code_last_page_len, int page_size, int num_heads,
                    int num_q_heads, int head_dim, void* out, int64_t out_stride, int out_format, int metric,
                    int exclude_last, uint32_t* hist, int hist_slices, adamas_stream_t stream);

/* ---- stage 3: top-k ------------------------------------------------------------------------ */

/* For each of num_rows rows select the k smallest of n values; equal values are taken in order of
 * position (lower position first); results are written in ascending position order:
 *   out_values[row*out_stride + j] = value at the j-th selected position p_j,
 *   out_idx[row*out_stride + j]    = in_idx ? in_idx[row*in_idx_stride + p_j/idx_page_size]*idx_page_size
 *                                              + p_j % idx_page_size
 *                                           : p_j.
 * in_idx_stride may be 0 (one index row shared by all rows).  out_values may be NULL.
 * Requires 1 <= k <= n.
 * Replaces topk_filtering (adamas/ops/csrc/topk.cu:7-46, kernels/include/topk/decode_select_k.cuh:25-62,
 * raft radix_topk_one_block_kernel); the reference leaves the tie order undefined. */
int adamas_topk(const void* values, int value_format, int64_t value_stride, int n,
                const int32_t* in_idx, int64_t in_idx_stride, int idx_page_size,
                int num_rows, int k, void* out_values, int32_t* out_idx, int64_t out_stride,
                adamas_stream_t stream);

/* ---- stage 4: sparse paged decode attention ------------------------------------------------ */

typedef struct adamas_decode_handler adamas_decode_handler_t;

/* Handler lifecycle: replaces flashinfer::BatchDecodeHandler and the class
 * BatchDecodeWithPagedKVCachePyTorchWrapper (adamas/ops/csrc/bsk_ops.h:95-124,
 * adamas/ops/csrc/approx_attn.cu:27-151, kernels/include/decode/decode_handler.cuh:39-244). */
int adamas_decode_handler_create(adamas_decode_handler_t** handler);
int adamas_decode_handler_destroy(adamas_decode_handler_t* handler);

/* Plans the split of max_tokens attended tokens per head over thread blocks and makes sure the
 * handler's device scratch (partial outputs) is large enough (allocates on first use or growth).
 * Replaces BeginForward (kernels/include/decode/decode_handler.cuh:73-121). */
int adamas_decode_begin_forward(adamas_decode_handler_t* handler, int64_t max_tokens, int batch,
                                int num_heads, int num_q_heads, int head_dim, int page_size, int dtype,
                                adamas_stream_t stream);
/* Replaces EndForward (decode_handler.cuh:123-136).  Scratch is kept for reuse until destroy. */
int adamas_decode_end_forward(adamas_decode_handler_t* handler);

/* o[h,:] = softmax(sm_scale * q[h,:] . K_sel^T) V_sel over, for head h, the tokens covered by
 * indices[h*idx_stride + i], i < n_idx, followed by the tail.  Each index covers idx_unit
 * consecutive token slots starting at index*idx_unit (idx_unit = 1: physical token slots
 * page*page_size+entry, a negative entry is a hole that is skipped; idx_unit = page_size: whole
 * pages, the reference's meaning).  A head whose list and tail are empty gets zeros and lse = -inf.
 * The tail is the
 * last tail_len filled entries of page last_page_idx, i.e. entries
 * [last_page_len - tail_len, last_page_len).  q, o [H, D]; lse (optional, may be NULL) [H] receives
 * log2(sum exp2(sm_scale*log2(e)*logit)) style base-2 log-sum-exp of the scaled logits.
 * Replaces BatchDecodeWithPagedKVCachePyTorchWrapper::Forward (adamas/ops/csrc/approx_attn.cu:68-151,
 * kernels/include/decode/decode_attn.cuh:469-702,952-1127). */
int adamas_decode_forward(adamas_decode_handler_t* handler, const void* q, void* o, float* lse,
                          const void* kv_data, const int32_t* indices, int64_t idx_stride,
                          int n_idx, int idx_unit, int last_page_idx, int last_page_len,
                          int tail_len, float sm_scale, adamas_stream_t stream);

/* Same as adamas_decode_forward with the output kept in fp32 (o_f32 [H, D]) and lse mandatory: the
 * partial result of one sequence shard, to be combined with adamas_merge_states without an
 * intermediate rounding.  Replaces the (o, lse) partial written by the reference's split-KV kernel
 * (kernels/include/decode/decode_attn.cuh:672-700). */
int adamas_decode_forward_partial(adamas_decode_handler_t* handler, const void* q, float* o_f32,
                                  float* lse, const void* kv_data, const int32_t* indices,
                                  int64_t idx_stride, int n_idx, int idx_unit, int last_page_idx,
                                  int last_page_len, int tail_len, float sm_scale,
                                  adamas_stream_t stream);

/* The same attention as adamas_decode_forward for callers that must not allocate device memory: code
 * that runs while the process is not allowed to call cudaMalloc or cudaFree (a serving process whose
 * memory manager has already claimed the whole device, a thread that cannot afford the device-wide
 * synchronisation those calls imply).
 * It needs no handler and no begin_forward: the split-KV scratch is a fixed array inside the library
 * (about 1.1 MB of device memory, held by every GPU that loads the library until the process exits).
 * Limits: num_heads <= 256 and num_heads * splits <= 2048 (head, split) units, where splits is the
 * number of thread blocks the planner gives each head; larger requests are rejected with
 * ADAMAS_ERR_INVALID and a message, and should use the handler-based call.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress) and sets
 * kernel attributes; make that first call outside any stream capture.  All calls on a device share
 * the one array: two calls whose kernels may overlap on the GPU (different streams, no dependency)
 * race on it; calls on one stream are safe.  Arguments as for adamas_decode_forward, plus the cache
 * geometry that the handler otherwise carries.
 * This entry point has no counterpart in the reference. */
int adamas_decode_forward_static(const void* q, void* o, float* lse, const void* kv_data,
                                 const int32_t* indices, int64_t idx_stride, int n_idx, int idx_unit,
                                 int num_heads, int head_dim, int page_size, int dtype,
                                 int last_page_idx, int last_page_len, int tail_len, float sm_scale,
                                 adamas_stream_t stream);

/* Stages 3 and 4 in one launch: per head, the k smallest of n distances (ADAMAS_VAL_U16, rows on
 * 16-byte boundaries; values of 511 and more count as equal; ties to the lower position) are selected
 * and attended together with the newest token (entry last_page_len-1 of page last_page_idx;
 * last_page_len = 0: there is no newest token, as on a sequence shard that does not hold it).  Token t
 * of the row is looked up as kv_page_table[t / page_size] * page_size + t % page_size.
 * o [H, D] in dtype and / or o_f32 [H, D] fp32 (the partial result of a sequence shard; needs lse).
 * out_idx (optional, [H, out_stride]) receives the winners' physical token slots in ascending position
 * order, exactly what adamas_topk would write.
 * hist: histogram scratch (see ADAMAS_HIST_WORDS_PER_HEAD), all zero on entry unless hist_ready, all
 * zero on exit.  hist_ready = 0: the call counts the distances itself first (one more launch);
 * hist_ready = 1: an adamas_estimate / adamas_append_estimate call with hist_slices =
 * adamas_select_attend_slices(n, k, num_heads) has left the counts there.
 * ext_cut (optional, device, [H][2] int32, 8-byte aligned): the cut distance and the number of
 * cut-valued elements THIS call takes, per head, decided elsewhere (the global cut of a sequence split
 * over several GPUs); k is then only an upper bound for the winners of this call.
 * Replaces the topk_filtering + BatchDecodeWithPagedKVCachePyTorchWrapper::Forward pair
 * (adamas/models/Adamas.py:185-200) for n up to 262144 (32768 x the adamas_set_max_cluster bound). */
int adamas_select_attend(const void* dist, int64_t dist_stride, int n, int k, const void* q, void* o,
                         float* o_f32, float* lse, const void* kv_data, const int32_t* kv_page_table,
                         int page_size, int num_heads, int num_q_heads, int head_dim, int dtype,
                         int last_page_idx, int last_page_len, uint32_t* hist, int hist_ready,
                         const int32_t* ext_cut, int32_t* out_idx, int64_t out_stride, float sm_scale,
                         adamas_stream_t stream);

/* Number of slices (thread blocks per head) adamas_select_attend uses for rows of n distances, k
 * winners and num_heads heads on the current device: the hist_slices an estimate call must be given
 * when it prepares the histogram table for that call.  No counterpart in the reference. */
int adamas_select_attend_slices(int n, int k, int num_heads, int* slices);

/* ---- one sequence split over several GPUs by token range ("sequence shards") -------------------
 * Shard g holds a contiguous token range of every head (its own KV and code caches).  Per layer-step
 * every shard runs adamas_estimate with hist on its range, adamas_hist_rowsum, one all-gather of the
 * [H][512] counts, adamas_global_cut, adamas_select_attend with that ext_cut and an fp32 partial
 * output, one all-gather of the partials (o, lse) and adamas_merge_states: two collectives, and no
 * candidate list ever crosses the link.  The reference is single-GPU; the scheme follows what its
 * split-KV decode does inside one GPU (kernels/include/decode/decode_attn.cuh:1050-1059). */

/* out[h][bin] = sum over the first `slices` histogram rows of head h in a histogram scratch table that
 * an adamas_estimate call has filled: the shard's 512-bin histogram per head, ready to be exchanged. */
/* Counts rows of integer distances (ADAMAS_VAL_U16, as adamas_estimate writes them) into the histogram
 * scratch, `slices` per-slice histograms per row, the layout adamas_select_attend(..., hist_ready = 1)
 * reads: what adamas_estimate does on the side when it is given `hist`, as a launch of its own that counts
 * in shared memory.  Cheaper than counting inside the estimate from about 3 M distances per call. */
int adamas_dist_histograms(const void* dist, int64_t dist_stride, int n, int num_heads, int slices,
                           uint32_t* hist, adamas_stream_t stream);

int adamas_hist_rowsum(const uint32_t* hist, int num_heads, int slices, uint32_t* out, adamas_stream_t stream);

/* all_hists [num_shards][H][512]: the shards' histograms in shard order (ascending token ranges).
 * Writes ext_cut [H][2] for shard `shard`: the cut distance of the k smallest distances of the whole
 * sequence and how many cut-valued elements this shard takes (lower shards are served first: the
 * lower position wins a tie).  If the sequence holds fewer than k distances: (512, 0), every element
 * wins. */
int adamas_global_cut(const uint32_t* all_hists, int num_shards, int shard, int num_heads, int k, int32_t* ext_cut,
                      adamas_stream_t stream);

/* Stages 1 and 2 of a decode step in one launch, for 16, 32 or 64 heads: the append of
 * adamas_append_decode_fused (new token's K, V and code into the caches, query code to q_code; q and k
 * already rotated) and the estimate of adamas_estimate with ADAMAS_VAL_U16 output, the L1 metric and
 * exclude_last = 1 (dist [H, dist_stride], rows on 16-byte boundaries, dist_stride >= context - 1).
 * Every thread block derives the query code from q by itself, so the scan does not wait for an append
 * launch.  hist / hist_slices as for adamas_estimate.  Replaces hadamard_transform + append_kvh +
 * decode_estimate of adamas/models/Adamas.py:145-180. */
int adamas_append_estimate(const void* q, const void* k, const void* v, void* q_code, void* kv_data,
                           const int32_t* kv_page_table, int kv_num_pages, int kv_last_page_len,
                           void* code_data, const int32_t* code_page_table, int code_num_pages,
                           int code_last_page_len, int num_heads, int head_dim, int page_size, int dtype,
                           void* dist, int64_t dist_stride, float hadamard_scale,
                           const float* thresholds3_host, uint32_t* hist, int hist_slices,
                           adamas_stream_t stream);

/* One layer's whole decode step in one call: two launches (the estimate with the append inside, then
 * select+attend) for 32 or 64 heads and rotated inputs, three (fused append, estimate,
 * select+attend) otherwise:
 * what adamas/models/Adamas.py:145-200 does with seven launches.  q, k, v, o [1,H,D]; q_code
 * [1,H,D/8] scratch/output; dist_scratch [H, dist_stride] 16-bit, rows on 16-byte boundaries,
 * dist_stride >= context - 1; hist_scratch: see ADAMAS_HIST_WORDS_PER_HEAD.  Requires context > budget
 * (otherwise every page is attended: use
 * adamas_decode_forward).  kv_last_page_idx is the physical number of the last KV page.  With
 * rope_scale > 0, q and k arrive un-rotated and the append launch rotates them in place first
 * (apply_rope_in_place, adamas/models/Adamas.py:113); rope_scale <= 0: q and k are already rotated.
 * rope_inv_freq (optional, device, 64 floats) and rope_mscale: a frequency table instead of
 * (rope_scale, rope_theta), see adamas_decode_step_dev. */
int adamas_decode_step(void* q, void* k, const void* v, void* o, float* lse, void* q_code,
                       void* kv_data, const int32_t* kv_page_table, int kv_num_pages,
                       int kv_last_page_len, int kv_last_page_idx, void* code_data,
                       const int32_t* code_page_table, int code_num_pages, int code_last_page_len,
                       int num_heads, int num_q_heads, int head_dim, int page_size, int dtype, int budget,
                       void* dist_scratch, int64_t dist_stride, uint32_t* hist_scratch, int32_t* out_idx,
                       int64_t out_stride, float hadamard_scale, const float* thresholds3_host,
                       float rope_scale, float rope_theta, const float* rope_inv_freq, float rope_mscale,
                       float sm_scale, adamas_stream_t stream);

/* ---- decode steps whose sequence length lives on the device ----------------------------------
 * The reference rebuilds its index tensors on the host and re-plans the decode every step
 * (adamas/utils/controller.py:82-131, kernels/include/decode/decode_handler.cuh:73-121), so no two
 * steps are the same sequence of launches.  Here a step can take the sequence length from device
 * memory: *seq_len_dev = tokens in the caches, the one being appended included (int32).  The
 * launches are then shaped by max_seq_len only, every kernel derives page numbers, slots, positions
 * and row lengths from the device value, and ONE captured CUDA graph of the step serves every token:
 * replay it, and add 1 to the length between replays (adamas_seq_len_advance, itself capturable).
 * Rules: *seq_len_dev <= max_seq_len; the page tables hold an entry for every page of the current
 * length before the step runs; the value must not be written by the kernel that directly precedes
 * a step in the stream (parts of a step start early and read it before that kernel has finished):
 * advance it at the END of a token's work, not in front of the next step. */

/* adamas_decode_step with the length on the device.  Needs *seq_len_dev > budget.
 * rope_inv_freq (optional, device, 64 floats): per-pair rotation frequencies with any position
 * scaling folded in; the angle of pair j at position t is t * rope_inv_freq[j] and the rotated values
 * are multiplied by rope_mscale (YaRN-style scaling; rope_scale / rope_theta are then unused). */
int adamas_decode_step_dev(void* q, void* k, const void* v, void* o, float* lse, void* q_code, void* kv_data,
                           const int32_t* kv_page_table, void* code_data, const int32_t* code_page_table,
                           const int32_t* seq_len_dev, int max_seq_len, int num_heads, int num_q_heads,
                           int head_dim, int page_size, int dtype, int budget, void* dist_scratch, int64_t dist_stride,
                           uint32_t* hist_scratch, int32_t* out_idx, int64_t out_stride, float hadamard_scale,
                           const float* thresholds3_host, float rope_scale, float rope_theta,
                           const float* rope_inv_freq, float rope_mscale, float sm_scale,
                           adamas_stream_t stream);

/* The dense counterpart (the reference's first layers, adamas/models/llama.py:428-439: every page is
 * "selected"): fused append (with the rotary embedding when rope_scale > 0 or rope_inv_freq is given)
 * and attention over all *seq_len_dev tokens.  The handler must have been planned with
 * adamas_decode_begin_forward(handler, max_seq_len, ...). */
int adamas_dense_step_dev(adamas_decode_handler_t* handler, void* q, void* k, const void* v, void* o, float* lse,
                          void* q_code, void* kv_data, const int32_t* kv_page_table, void* code_data,
                          const int32_t* code_page_table, const int32_t* seq_len_dev, int max_seq_len,
                          int num_heads, int num_q_heads, int head_dim, int page_size, int dtype,
                          float hadamard_scale, const float* thresholds3_host, float rope_scale, float rope_theta,
                          const float* rope_inv_freq, float rope_mscale, float sm_scale,
                          adamas_stream_t stream);

/* seq_len_dev[i] += delta for i < count (count = 1 for a single sequence, the batch size for a batched
 * step), as one tiny launch that is ordered after everything before it in the stream and before
 * everything after it. */
int adamas_seq_len_advance(int32_t* seq_len_dev, int count, int delta, adamas_stream_t stream);

/* ---- several sequences in one launch ------------------------------------------------------------
 * The reference decodes one sequence per call (adamas/models/Adamas.py:83 asserts batch size 1, and an
 * InferenceController holds one sequence); a server loops over its sequences.
 * Here `batch` sequences of one cache geometry go through the SAME two or three launches of a step:
 * every kernel's grid gets a sequence coordinate.  Each sequence keeps its own caches and page
 * tables, described by one adamas_seq_desc_t in a device array; everything else is one contiguous
 * array over (sequence, head) rows: q, o [batch, Hq, D]; k, v [batch, H, D]; q_code [batch, Hq, D/8];
 * dist_scratch [batch * Hq, dist_stride]; hist_scratch batch * Hq * ADAMAS_HIST_WORDS_PER_HEAD words;
 * out_idx [batch * Hq, out_stride]; lse [batch * Hq]; seq_lens_dev int32 [batch] (advance all of them
 * with adamas_seq_len_advance(seq_lens_dev, batch, 1, ...)).  The sequences may have different
 * lengths; every one must be longer than the budget for the sparse step.  The descriptor array must be
 * complete before the first step is launched and must not change while steps are in flight. */
typedef struct adamas_seq_desc {
  void* kv_data;                    /* this layer's KV cache of the sequence [pages, 2, page_size, H, D] */
  void* code_data;                  /* this layer's code cache [pages, 1, page_size, H, D/8] */
  const int32_t* kv_page_table;     /* device, an entry for every page of the current length */
  const int32_t* code_page_table;
} adamas_seq_desc_t;

/* adamas_decode_step_dev for `batch` sequences. */
int adamas_decode_step_batch_dev(void* q, void* k, const void* v, void* o, float* lse, void* q_code,
                                 const adamas_seq_desc_t* seqs_dev, const int32_t* seq_lens_dev, int batch,
                                 int max_seq_len, int num_heads, int num_q_heads, int head_dim, int page_size,
                                 int dtype, int budget, void* dist_scratch, int64_t dist_stride,
                                 uint32_t* hist_scratch, int32_t* out_idx, int64_t out_stride, float hadamard_scale,
                                 const float* thresholds3_host, float rope_scale, float rope_theta,
                                 const float* rope_inv_freq, float rope_mscale, float sm_scale,
                                 adamas_stream_t stream);

/* adamas_dense_step_dev for `batch` sequences; the handler must have been planned with
 * adamas_decode_begin_forward(handler, max_seq_len, batch, ...). */
int adamas_dense_step_batch_dev(adamas_decode_handler_t* handler, void* q, void* k, const void* v, void* o,
                                float* lse, void* q_code, const adamas_seq_desc_t* seqs_dev,
                                const int32_t* seq_lens_dev, int batch, int max_seq_len, int num_heads,
                                int num_q_heads, int head_dim, int page_size, int dtype, float hadamard_scale,
                                const float* thresholds3_host, float rope_scale, float rope_theta,
                                const float* rope_inv_freq, float rope_mscale, float sm_scale,
                                adamas_stream_t stream);

/* adamas_apply_rope_in_place with a table of rotation frequencies (device, 64 floats) and a factor on
 * the rotated values instead of (rope_scale, rope_theta): the prefill side of YaRN-scaled models.  The
 * reference's kernel knows linear scaling only (kernels/include/decode/decode_page.cuh:650-659). */
int adamas_apply_rope_table_in_place(void* q, void* k, int64_t seq_len, int num_q_heads, int num_kv_heads,
                                     int head_dim, int64_t past_kv_len, const float* inv_freq_dev, float mscale,
                                     int dtype, adamas_stream_t stream);

/* Merge P partial results over disjoint token sets: o_parts [P, H, D] fp32 (each already
 * normalised), lse_parts [P, H] base-2; writes o [H, D] in dtype and, optionally, lse [H].
 * Replaces VariableLengthMergeStates (called at kernels/include/decode/decode_attn.cuh:1050-1059);
 * also the merge step of sequence-sharded decoding. */
int adamas_merge_states(const float* o_parts, const float* lse_parts, int num_parts, int num_heads,
                        int head_dim, void* o, float* lse, int dtype, adamas_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* ADAMAS_B200_H_ */
