/*
 * hipattn.h -- C ABI of libhipattn_sm100.so: HiP / InfiniteHiP attention for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain pointers and sizes (device pointers unless stated otherwise) and a
 * CUDA stream given as an opaque pointer (cudaStream_t).  No entry point allocates, frees or
 * synchronises; the caller owns all buffers.  Return value: HIPATTN_OK or an HIPATTN_ERR_* code;
 * hipattn_error_string() gives a description of the last error on the calling thread.
 *
 * The functions replace, one to one, the device work the reference operator
 * `hip_attention_12` (src/hip_attn/v1_2/attention_extend.py:1918) performs through Triton kernels
 * and torch tensor ops.  The citation above each declaration names the reference code it stands for
 * (paths relative to the DeepAuto-AI/hip-attention checkout).
 */
#ifndef HIPATTN_H_
#define HIPATTN_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HIPATTN_OK 0
#define HIPATTN_ERR_INVALID 1     /* bad argument (null pointer, size out of range, misaligned row) */
#define HIPATTN_ERR_UNSUPPORTED 2 /* valid request this build has no kernel for (dtype / head dim)  */
#define HIPATTN_ERR_CUDA 3        /* a CUDA runtime call failed                                     */

#define HIPATTN_F32 0
#define HIPATTN_F16 1
#define HIPATTN_BF16 2

/* Bits of the device status word written by the kernels (0 = clean). */
#define HIPATTN_STATUS_PAGE_RANGE 1u  /* a block-table entry pointed outside the page pool; clamped */
#define HIPATTN_STATUS_TOKEN_RANGE 2u /* a token index fell outside [0, T); clamped                 */
#define HIPATTN_STATUS_CHUNK_SIZE 8u  /* a chunk was longer than the chunk size the scan was told; its tail was ignored */
#define HIPATTN_STATUS_TIMEOUT 4u     /* a bounded on-chip wait ran out; the launch's output is invalid */

#define HIPATTN_SCORE_INIT (-32000.0f) /* attention_extend.py:2040-2045 */
#define HIPATTN_INDEX_PAD INT64_MAX    /* attention_extend.py:2913 */
#define HIPATTN_MAX_CHUNKS 16384       /* chunks per (batch, query block) the selection kernels sort on chip */

/*
 * Where the rows of K (or V) live: a dense tensor [B, T, HKV, D] or a page pool
 * [n_pages, P, HKV, D] addressed through block_table[b, t / P] (src/hip_attn/v1_2/uvm_gpu_cache.py:865-890,
 * 1034-1042).  Strides are in elements; the last dimension must be contiguous and every row must
 * start on a 16-byte boundary (8 bytes for an fp8 cache).  `cache != NULL` selects paging.
 */
typedef struct hipattn_tokens {
  const void* dense;
  int64_t stride_b, stride_t, stride_h;
  const void* cache;
  int64_t stride_page, stride_off, stride_ch;
  const void* block_table;   /* [B, table_width], int32 or int64 */
  int64_t table_stride_b;
  const void* cache_seq_lens; /* [B], int32 or int64 */
  int64_t n_pages;
  int32_t table_width;
  int32_t table_is_i64;
  int32_t seq_lens_is_i64;
  int32_t page_size;
  int32_t fp8_e5m2;          /* 1: the rows hold 1-byte e5m2 values (an fp8 KV cache, uvm_gpu_cache.py:1043-1046,
                                paged_hip.py:409-418); strides are then in bytes and every value is used as the 16-bit
                                number it converts to exactly.  Needs a 16-bit q. */
  int32_t reserved_;
} hipattn_tokens_t;

#define HIPATTN_ROPE_NONE 0
#define HIPATTN_ROPE_RELATIVE 1
#define HIPATTN_ROPE_STREAMING 2

#define HIPATTN_SCAN_AUTO 0   /* tensor-core scores with exact fallback where built, else strict */
#define HIPATTN_SCAN_STRICT 1 /* sequential fp32 dot products only */
#define HIPATTN_SCAN_CHECK 2  /* as AUTO, but every key is also scored strictly and compared (slow) */

/*
 * One scan stage of the mask estimator.
 * Replaces chunk_controllable_sampling_mask_cuda (attention_extend.py:413-1249) with the dense /
 * paged branches of load_tokens (uvm_gpu_cache.py:843-912, 1034-1046) and the head max-reduce that
 * follows it (attention_extend.py:2566-2570).
 *
 * The chunk list is shared by all heads of a (batch, query block): left/right are [B, BDST, n].
 * score_max [B, BDST, n] receives the maximum over heads of the per-head chunk score in an
 * order-preserving signed-integer encoding (see hipattn_encode_score); it must hold
 * encode(HIPATTN_SCORE_INIT) on entry (hipattn_init_chunks / hipattn_select_stage write that).
 * left_out / right_out / score_out are optional per-head results [B, BDST, H, n].
 */
typedef struct hipattn_scan_params {
  const void* q;             /* [B, TQ, H, D] */
  int64_t q_stride_b, q_stride_t, q_stride_h;
  const int64_t* pos;        /* [B, TQ] absolute positions */
  int64_t pos_stride_b, pos_stride_t;
  hipattn_tokens_t k;
  const int32_t* left;
  const int32_t* right;
  int32_t* score_max;
  int32_t* left_out;
  int32_t* right_out;
  float* score_out;
  uint32_t* status;          /* one word, OR-ed with HIPATTN_STATUS_* */
  const float* key_abs;      /* optional [B, HKV, T]: sum_d |round(k * k_scale)| per key row (hipattn_key_abs_sum);
                                lets the tensor-core path skip computing it per round */
  const void* k_scaled;      /* optional dense [B, HKV, T, D] copy of the keys, element type, already multiplied by k_scale
                                and rounded (hipattn_scan_prepare_keys); with key_abs it enables the tcgen05 scan */
  uint64_t* stats;           /* optional, 4 words: keys scored, keys re-scored strictly, wrong shortcuts
                                (check mode), largest deviation / allowed radius as float bits (check mode) */
  int32_t dtype, D, B, TQ, H, HKV, T;
  int32_t block_size_q;      /* stage_block_size_q */
  int32_t stride_q;          /* stage_block_stride_q */
  int32_t n_chunks;
  int32_t block_chunk;       /* group size that fixes the number of halving rounds (BLOCK_CHUNK) */
  int32_t scan_window;       /* max(0, sliding_window - first chunk size), attention_extend.py:1976-1978 */
  float q_scale, k_scale;    /* already rounded to the element type, attention_extend.py:924-940 */
  int32_t mode;              /* HIPATTN_SCAN_AUTO / _STRICT / _CHECK */
  int32_t chunk_size;        /* optional: upper bound of right - left (the stage's chunk size), 0 = unknown.  A small
                                power of two lets the scan score whole chunks once for all heads of a KV head and
                                replay the search on the scores (same results, fewer key rows gathered) */
  /* In-kernel RoPE of the estimator (attention_extend.py:248-407, 630-703): q and k arrive un-rotated and are
   * rotated on the fly, x * cos + rotate_half(x) * sin in the element type.  rope_mode HIPATTN_ROPE_RELATIVE:
   * queries at position 1 + scan_window, left / right candidate keys at 0 / 1; HIPATTN_ROPE_STREAMING: queries
   * at min(position, n_chunks + scan_window), keys at their chunk's index in the list. */
  const void* rope_cos;      /* [rope_rows, D] in the element type of q (only the first D / 2 columns are read) */
  const void* rope_sin;
  int64_t rope_stride;       /* elements between table rows */
  int32_t rope_rows;
  int32_t rope_mode;         /* HIPATTN_ROPE_NONE / _RELATIVE / _STREAMING */
  /* Access statistics (require_cache_statistics, uvm_gpu_cache.py:846-909): optional int32 [B, HKV, access_n] that
   * receives 1 at every key position (dense K) or page (paged K: the block-table entry, page 0 beyond the sequence)
   * whose row a round of the scan asked for.  The caller zeroes it. */
  int32_t* access_counter;
  int64_t access_stride_b, access_stride_h;
  int32_t access_n;
  int32_t k_scaled_sides;    /* 0 / 1: one prepared copy.  2 (rope_mode RELATIVE only): k_scaled and key_abs hold two
                                consecutive copies, the keys rotated to table position 0 (left candidates) and 1 (right
                                candidates), written by hipattn_scan_prepare_keys_rope: the tensor-core scan then runs
                                with in-kernel RoPE.  1 with rope_mode STREAMING (head dim 128): k_scaled holds the keys
                                as they are (hipattn_scan_prepare_keys with k_scale = 1); the tensor-core scan rotates
                                every key it fetches to its chunk's index and applies k_scale itself */
} hipattn_scan_params_t;

int hipattn_scan_stage(const hipattn_scan_params_t* p, void* stream);

/*
 * Per key row, sum over the head dimension of |round_to_dtype(k * k_scale)| as fp32, out [B, HKV, T].
 * No counterpart in the reference: it is the magnitude from which the tensor-core scan derives the
 * error radius of its approximate dot products, computed once per call instead of once per round.
 */
int hipattn_key_abs_sum(const hipattn_tokens_t* k, int32_t dtype, int32_t D, int32_t B, int32_t T, int32_t HKV,
                        float k_scale, float* out, uint32_t* status, void* stream);

/*
 * As hipattn_key_abs_sum, and also writes the scaled keys round_to_dtype(k * k_scale) as a dense
 * head-major [B, HKV, T, D] array of the element type (either output may be null).  The scan then gathers from
 * this copy: no page-table lookups and no arithmetic between global and shared memory.  No counterpart
 * in the reference, which rescales every gathered key inside the scan (attention_extend.py:924-940).
 */
int hipattn_scan_prepare_keys(const hipattn_tokens_t* k, int32_t dtype, int32_t D, int32_t B, int32_t T, int32_t HKV,
                              float k_scale, float* key_abs, void* k_scaled, uint32_t* status, void* stream);

/*
 * As hipattn_scan_prepare_keys, for the scan's in-kernel RoPE with backend "relative": every key is first rotated to
 * the fixed table position `position` (x * cos + rotate_half(x) * sin in the element type, attention_extend.py:290-407),
 * then scaled.  Two calls (position 0 into the first copy, position 1 into the second, each copy [B, HKV, T, D] resp.
 * [B, HKV, T]) give what hipattn_scan_stage expects with k_scaled_sides = 2; position = -1 writes both copies in one
 * pass (k_scaled [2, B, HKV, T, D], key_abs [2, B, HKV, T]), reading every key once.
 */
int hipattn_scan_prepare_keys_rope(const hipattn_tokens_t* k, int32_t dtype, int32_t D, int32_t B, int32_t T, int32_t HKV,
                                   float k_scale, const void* rope_cos, const void* rope_sin, int64_t rope_stride,
                                   int32_t rope_rows, int32_t position, float* key_abs, void* k_scaled, uint32_t* status,
                                   void* stream);

/*
 * Initial chunk list of stage 0 (attention_extend.py:2027-2046): left[c] = sink + c * chunk,
 * right = min(left + chunk, T - scan_window), score_max = encode(HIPATTN_SCORE_INIT).
 * Arrays are [rows, n] with rows = B * BDST.
 */
int hipattn_init_chunks(int32_t* left, int32_t* right, int32_t* score_max, int64_t rows, int32_t n,
                        int32_t sink, int32_t chunk, int32_t T, int32_t scan_window, void* stream);

/*
 * Selection between two stages, per (batch, query block) row:
 * top-k by (score descending, chunk position ascending) (attention_extend.py:2710-2721), then the
 * slice / realign / sort-by-left / split transform that builds the next stage's chunk list
 * (attention_extend.py:2072-2165).  Writes next_left / next_right [rows, k_keep * (c_prev / c_next)]
 * and next_score_max = encode(HIPATTN_SCORE_INIT).  n <= HIPATTN_MAX_CHUNKS.
 */
int hipattn_select_stage(const int32_t* score_max, const int32_t* left, int64_t rows, int32_t n,
                         int32_t k_keep, int32_t sink, int32_t c_prev, int32_t c_next,
                         int32_t* next_left, int32_t* next_right, int32_t* next_score_max, void* stream);

/*
 * Selection after the last stage and conversion to the block-sparse index format
 * (attention_extend.py:2722-2728, 2772-2776, 2906-2925): order all chunks by (score descending,
 * position ascending), keep the first K = second_stage_k / c_last, align, then per head sort,
 * replace duplicates by HIPATTN_INDEX_PAD, sort again and count the entries below
 * pos[b, d * block_size_q] + block_size_q.
 * left_heads: narrowed per-head left bounds [rows, H, n] with head stride `left_head_stride`
 * (pass the shared [rows, n] list with stride 0 when all heads agree).
 * indices [B * H, BDST, K] int64; ks [B * H, BDST] int64; ks_start_end [B * H, BDST, 2] int32.
 */
int hipattn_finalize_indices(const int32_t* score_max, const int32_t* left_heads, int64_t left_row_stride,
                             int64_t left_head_stride, const int64_t* pos, int64_t pos_stride_b,
                             int64_t pos_stride_t, int32_t B, int32_t BDST, int32_t H, int32_t n, int32_t K,
                             int32_t c_last, int32_t block_size_q, int64_t* indices, int64_t* ks,
                             int32_t* ks_start_end, void* stream);

/*
 * Block-sparse attention over {selected blocks, sink, sliding window}.
 * Replaces block_sparse_attention_cuda (attention_extend_bsa.py:621-1638) for prefill and
 * _fwd_kernel_stage1 (attention_decode_bsa.py:23-1044) for decode; masking rules of
 * block_sparse_attention_cuda_step (attention_extend_bsa.py:511-565).
 *
 * n_splits == 1: writes out [B, TQ, H, D] in the element type.
 * n_splits  > 1: (decode, TQ == 1) the key set is cut into n_splits ranges; split s writes the
 *   normalised partial output part_o [B, H, n_splits, D] fp32 and its base-2 log-sum-exp part_lse
 *   [B, H, n_splits] (-inf for an empty range), to be combined by hipattn_merge_partials.
 * lse_out (optional) [B, TQ, H] fp32 receives the base-2 log-sum-exp of every row (n_splits == 1).
 */
typedef struct hipattn_bsa_params {
  const void* q;
  int64_t q_stride_b, q_stride_t, q_stride_h;
  void* out;
  int64_t o_stride_b, o_stride_t, o_stride_h;
  const int64_t* pos;
  int64_t pos_stride_b, pos_stride_t;
  hipattn_tokens_t k, v;
  const int64_t* indices;    /* [B * H, BDST, K] */
  int64_t idx_stride_n, idx_stride_d;
  const int64_t* ks;         /* [B * H, BDST] */
  int64_t ks_stride_n, ks_stride_d;
  float* part_o;
  float* part_lse;
  float* lse_out;
  uint32_t* status;
  int32_t dtype, D, B, TQ, H, HKV, T;
  int32_t block_size_q;      /* query rows per attention block (scope of the block's largest position) */
  int32_t index_block_q;     /* query rows per row of indices / ks (a multiple of block_size_q) */
  int32_t block_size_k;      /* tokens per selected block (last stage chunk size) */
  int32_t K;
  int32_t sink, window;      /* attention window = max(sliding_window, first chunk size) */
  int32_t n_splits;
  int32_t heads_share_mask;  /* 1: indices / ks are identical for the heads of a KV group */
  float logit_softcap;       /* 0 = off; attention_extend_bsa.py:389-390 */
  /* In-kernel RoPE of the attention, backend "streaming" (attention_extend_bsa.py:126-392, 797-856), when rope_cos
   * is given: queries are rotated to their own position, window keys to theirs, sink and selected keys to
   * max(0, rank_in_list + pmin - window - sink - ks * block_size_k + 1) with pmin the block's smallest query position. */
  int32_t rope_rows;
  const void* rope_cos;      /* [rope_rows, D] in the element type of q */
  const void* rope_sin;
  int64_t rope_stride;
} hipattn_bsa_params_t;

int hipattn_bsa_attention(const hipattn_bsa_params_t* p, void* stream);

/*
 * Access statistics of the attention (the `sa` counter of require_cache_statistics): writes 1 into counter
 * [B, HKV, n] (int32, zeroed by the caller, strides in elements) at every key position / page the reference's
 * attention kernels load for the given mask: the sink tokens below the block's last position, the tokens of the
 * selected blocks inside [sink, last position], and the window from last position + 1 - window - block rows up to
 * the last position (attention_extend_bsa.py:858-891, 1133-1137, 1370-1383; `block rows` = p->block_size_q for the
 * prefill kernel, 1 for the decode kernel: pass it as window_block_rows).  Reads p->pos, indices, ks, k (for the page
 * table) and the mask geometry; no counterpart kernel in the reference, which marks inside load_tokens.
 */
int hipattn_mark_attention_access(const hipattn_bsa_params_t* p, int32_t* counter, int64_t stride_b, int64_t stride_h,
                                  int32_t n, int32_t window_block_rows, void* stream);

/*
 * Log-sum-exp merge of partial outputs (attention_decode_bsa.py:1149-1225).
 * part_o [rows, n_parts, D] fp32 normalised, part_lse [rows, n_parts] base-2; writes out [rows, D]
 * in `dtype` (row stride out_stride elements) and, optionally, merged lse [rows].
 */
int hipattn_merge_partials(const float* part_o, const float* part_lse, int64_t rows, int32_t n_parts,
                           int32_t D, int32_t dtype, void* out, int64_t out_stride, float* lse_out,
                           void* stream);

/*
 * Decode attention (TQ == 1) with key splits for callers that cannot allocate device memory.
 * No counterpart in the reference, which allocates its split buffer with torch on every call
 * (attention_decode_bsa.py:1082-1086).
 *
 * Same parameters as hipattn_bsa_attention, except that part_o / part_lse are ignored: the partial
 * results of the p->n_splits key ranges go to an array that is part of the library image, and the
 * merged result is written to p->out (contiguous [B, 1, H, D]) and, if given, p->lse_out [B, 1, H].
 * The call performs no cudaMalloc / cudaFree and calls no allocating routine.
 *
 * Limit: B * H * n_splits * (D + 1) * 4 bytes <= HIPATTN_NOALLOC_SCRATCH_BYTES, otherwise
 * HIPATTN_ERR_UNSUPPORTED.  That many bytes are resident on every GPU that loads the library until
 * the process exits.  The first call on a device looks up the array's device address (one
 * cudaGetSymbolAddress, with that device current); make that first call before starting any stream
 * capture.  All calls on a device share the array: calls that may overlap on the GPU race with each
 * other and must be ordered by the caller (same stream, or events).
 */
#define HIPATTN_NOALLOC_SCRATCH_BYTES (16 * 1024 * 1024)
int hipattn_bsa_decode_noalloc(const hipattn_bsa_params_t* p, void* stream);

/* Order-preserving image of an fp32 score: a < b  <=>  encode(a) < encode(b) as signed integers
 * (host helpers; across GPUs the head max is an int32 MAX all-reduce of score_max). */
int32_t hipattn_encode_score(float score);
float hipattn_decode_score(int32_t code);

/* Element-wise helpers used by the host wrapper to hand results back in the reference's types. */
int hipattn_decode_scores(const int32_t* codes, float* scores, int64_t count, void* stream);
int hipattn_widen_i32(const int32_t* src, int64_t* dst, int64_t count, void* stream);

/*
 * Failure-handling probe (no counterpart in the reference, whose kernels never report errors): one
 * CTA waits, with the bounded wait of the tcgen05 attention kernel, on a barrier nothing signals; after
 * about 20 ms it sets HIPATTN_STATUS_TIMEOUT in *status and exits normally.  The context stays usable.
 */
int hipattn_debug_bounded_wait(uint32_t* status, void* stream);

/* Number of kernels this library has launched in this process so far (host-side counter; every launch
 * site increments it).  No counterpart in the reference.  Benchmarks report the difference across
 * their timed region. */
uint64_t hipattn_launch_count(void);

const char* hipattn_error_string(void);
int hipattn_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* HIPATTN_H_ */
