/* kestrel_b200 -- C ABI of the B200 (sm_100a) paged-KV hot path.
 *
 * These entry points are what Kestrel's Python layer binds for this path in
 * place of the `kestrel_kernels` wheel (reference tree: m87-labs/kestrel
 * v0.5.0; citations are paths inside that tree).
 *
 * Conventions
 *   - every function returns 0 on success or a negative KB200_ERR_* code and
 *     never aborts, throws, synchronises the device or allocates device memory
 *     (scratch memory is passed in by the caller);
 *   - kb200_last_error() returns the message of the last failure on the calling
 *     thread;
 *   - all pointers named *device* pointers must be valid on GPU `device`; the
 *     work is enqueued on `stream` (a cudaStream_t, may be NULL for the legacy
 *     default stream) and the caller keeps the buffers alive until it ran;
 *   - strides are in ELEMENTS of the tensor's dtype unless the name says bytes;
 *   - a "cache view" is the reference's permuted pool view
 *     k_cache.permute(0, 2, 1, 3) = [n_pages, page_size, n_kv_heads, head_dim]
 *     (kestrel/kv_cache.py:205-206, kestrel/ops/attention.py:71-72) over the
 *     physical pool [n_pages, n_kv_heads, page_size, head_dim]
 *     (kestrel/kv_cache.py:97).
 */
#ifndef KESTREL_B200_H_
#define KESTREL_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KB200_ABI_VERSION 4

#if defined(__GNUC__)
#define KB200_API __attribute__((visibility("default")))
#else
#define KB200_API
#endif

enum {
  KB200_OK = 0,
  KB200_ERR_INVALID = -1,     /* bad argument (shape, dtype, alignment, null pointer) */
  KB200_ERR_CUDA = -2,        /* a CUDA runtime / driver call failed */
  KB200_ERR_UNSUPPORTED = -3, /* valid request this build does not implement */
  KB200_ERR_WORKSPACE = -4    /* workspace missing or too small */
};

enum {
  KB200_DTYPE_F32 = 0,
  KB200_DTYPE_F16 = 1,
  KB200_DTYPE_BF16 = 2,
  KB200_DTYPE_E4M3 = 3 /* FP8 e4m3fn codes, one byte per element */
};

/* Bits of device status word 0 (kb200_device_status). */
enum {
  KB200_STATUS_BAD_SLOT = 1,    /* append: slot >= n_pages * page_size (row skipped) */
  KB200_STATUS_BAD_PAGE = 2,    /* a page index outside [0, n_pages) (access skipped / zero filled) */
  KB200_STATUS_BAD_ROW = 4,     /* a page-table row index outside the table (row skipped) */
  KB200_STATUS_WAIT_TIMEOUT = 8, /* a bounded wait on a shared-memory barrier ran out */
  KB200_STATUS_BAD_POSITION = 16, /* rotary: a position outside the cos/sin table (clamped) */
  KB200_STATUS_BAD_PREFIX = 32   /* attention: shared_prefix_pages covers keys a query row may not see */
};

KB200_API int kb200_abi_version(void);
KB200_API const char* kb200_last_error(void);

/* Reads (and with `clear` != 0 resets) the four diagnostic words kernels write
 * instead of trapping.  Synchronises `device`.  Diagnostic aid, no reference
 * counterpart. */
KB200_API int kb200_device_status(int device, int32_t out[4], int clear);

/* ---------------------------------------------------------------------------
 * Append: scatter new K/V token rows into pool pages by slot, optionally
 * quantising to FP8 e4m3 (code = satfinite(rn(x / scale))).
 * Replaces kestrel_kernels' cache.reshape_and_cache_flash as called from
 * PagedKVCache.update (kestrel/kv_cache.py:222-231; torch restatement of the
 * unquantised case at :216-220).
 *
 *   key, value        device, rows [num_tokens, n_kv_heads, head_dim] of `in_dtype`,
 *                     head stride == head_dim, element stride 1, token stride given
 *                     (rows may be slices of a fused QKV buffer, kv_cache.py:24-48)
 *   key_cache, value_cache   device, cache views of `cache_dtype`
 *   slot_mapping      device int64 [num_tokens]; slot = page * page_size + offset
 *                     (kv_cache.py:549-550); negative slots are skipped
 *   k_scale, v_scale  device fp32, `n_scales` entries each: 1 (per layer, as the
 *                     reference passes k_scale_tensor / v_scale_tensor) or
 *                     n_kv_heads (per KV head); ignored unless cache_dtype is E4M3
 * Allowed dtype pairs: in == cache (bit copy; F32/F16/BF16) or
 * in in {F32,F16,BF16} with cache == E4M3.
 */
KB200_API int kb200_reshape_and_cache_flash(
    const void* key, const void* value, int64_t key_token_stride, int64_t value_token_stride,
    void* key_cache, void* value_cache, int64_t cache_page_stride, int64_t cache_token_stride,
    int64_t cache_head_stride, const int64_t* slot_mapping, int64_t num_tokens, int64_t n_pages,
    int32_t page_size, int32_t n_kv_heads, int32_t head_dim, int32_t in_dtype, int32_t cache_dtype,
    const float* k_scale, const float* v_scale, int32_t n_scales, int32_t device, void* stream);

/* ---------------------------------------------------------------------------
 * Slot mapping: out[i] = page_table[batch(i), pos[i] / P] * P + pos[i] % P.
 * One fused launch for PageTable.build_slot_mapping (kestrel/kv_cache.py:524-551).
 *
 *   page_table   device int32 [pt_rows, pt_cols], row stride given
 *   batch_idx    device int32 or int64; `batch_per_row` != 0: one entry per row of
 *                `row_len` positions (the 1-D batch_idx case), else one per position
 *   positions    device int32 or int64, contiguous [n]
 *   out_slots    device int64 [n]
 * Entries whose row/page lookup is out of range write -1 and set a status bit.
 */
KB200_API int kb200_build_slot_mapping(
    const int32_t* page_table, int64_t pt_row_stride, int64_t pt_rows, int64_t pt_cols,
    const void* batch_idx, int32_t batch_idx_is_i64, int32_t batch_per_row, int64_t row_len,
    const void* positions, int32_t positions_is_i64, int64_t* out_slots, int64_t n,
    int32_t page_size, int32_t device, void* stream);

/* ---------------------------------------------------------------------------
 * Decode metadata: out_seqused_k[r] = input_pos[r] + 1 and the first
 * ceil(out_seqused_k[r] / P) entries of page-table row batch_idx[r] copied to
 * out_page_table[r]; the tail of each output row is left untouched.
 * Replaces cache.build_paged_kv_metadata as called from
 * PageTable.populate_paged_kv_metadata (kestrel/kv_cache.py:515-522; semantics
 * pinned by tests/test_page_table.py:48-79).
 */
KB200_API int kb200_build_paged_kv_metadata(
    const int32_t* page_table, int64_t pt_row_stride, int64_t pt_rows, int64_t pt_cols,
    const void* batch_idx, int32_t batch_idx_is_i64, const int32_t* input_pos,
    int32_t* out_page_table, int64_t out_row_stride, int64_t out_cols, int32_t* out_seqused_k,
    int64_t batch, int32_t page_size, int32_t device, void* stream);

/* ---------------------------------------------------------------------------
 * Per-step decode metadata in one launch: kb200_build_paged_kv_metadata followed
 * by kb200_build_slot_mapping for the `n_new` tokens each active row appends this
 * step (positions input_pos[r] - n_new + 1 .. input_pos[r]).  Fuses the two calls
 * the reference makes at the top of every decode step
 * (kestrel/models/moondream/runtime.py:2554-2564).
 *
 *   out_slots      device int64 [batch, n_new]
 *   out_positions  device int64 [batch, n_new] or NULL (the position_ids the
 *                  reference derives with input_pos.to(long).view(-1, 1))
 * Other arguments as kb200_build_paged_kv_metadata.
 */
KB200_API int kb200_build_decode_step_metadata(
    const int32_t* page_table, int64_t pt_row_stride, int64_t pt_rows, int64_t pt_cols,
    const void* batch_idx, int32_t batch_idx_is_i64, const int32_t* input_pos,
    int32_t* out_page_table, int64_t out_row_stride, int64_t out_cols, int32_t* out_seqused_k,
    int64_t* out_slots, int64_t* out_positions, int64_t batch, int32_t n_new, int32_t page_size,
    int32_t device, void* stream);

/* ---------------------------------------------------------------------------
 * Rotary embedding, optionally fused with the append that follows it.
 * Replaces rotary.rotary_embedding(position_ids, q, k, head_dim, cos_sin_cache)
 * (kestrel/models/moondream/text.py:125) and, when key_cache is non-NULL, also
 * the PagedKVCache.update that comes right after it on the same K
 * (kestrel/models/moondream/text.py:132 -> kestrel/kv_cache.py:222-231) in one
 * launch: Q is rotated in place, K is rotated (written back when `write_k` != 0)
 * and rotated K plus V are scattered into the pool pages by slot, quantised to
 * e4m3 when cache_dtype is E4M3.
 *
 *   q, k, v        device rows [num_tokens, heads, head_dim] of `in_dtype`
 *                  (F32/F16/BF16), head stride == head_dim, token strides given;
 *                  q may be NULL with n_q_heads == 0
 *   positions      device int32/int64 [num_tokens]
 *   cos_sin_cache  device fp32 [max_pos, rot_dim]: cos of rot_dim/2 frequencies, then
 *                  sin (kestrel/models/moondream/rope.py:6-32); rot_dim <= head_dim,
 *                  NeoX pairing (i, i + rot_dim/2), elements past rot_dim pass through
 *   key_cache ...  as kb200_reshape_and_cache_flash; key_cache == NULL: rotate only
 * Rounding: y1 = x1*cos - x2*sin, y2 = x2*cos + x1*sin in fp32 with separately
 * rounded products, rounded once to `in_dtype`; the pool receives the bytes an
 * append of the rotated row would write.  Positions outside [0, max_pos) are
 * clamped and flagged in the device status.
 */
KB200_API int kb200_rope_append(
    void* q, void* k, const void* v, int64_t q_token_stride, int64_t k_token_stride,
    int64_t v_token_stride, int64_t num_tokens, int32_t n_q_heads, int32_t n_kv_heads,
    int32_t head_dim, int32_t rot_dim, const void* positions, int32_t positions_is_i64,
    const float* cos_sin_cache, int64_t max_pos, int64_t cos_sin_row_stride, void* key_cache,
    void* value_cache, int64_t cache_page_stride, int64_t cache_token_stride,
    int64_t cache_head_stride, const int64_t* slot_mapping, int64_t n_pages, int32_t page_size,
    int32_t in_dtype, int32_t cache_dtype, const float* k_scale, const float* v_scale,
    int32_t n_scales, int32_t write_k, int32_t device, void* stream);

/* ---------------------------------------------------------------------------
 * Copy-on-write page copy: for every pool in `caches` (HOST array of `n_caches`
 * device base pointers: the K and V pools of every layer) copy physical page
 * src_pages[i] onto dst_pages[i].  The reference has no counterpart (it forbids
 * prefix caching with page_size > 1, kestrel/kv_cache.py:331-335); this is what a
 * shared, partially filled prefix page needs before a request appends to it.
 *
 *   page_bytes         bytes of one page of one pool (n_kv_heads*page_size*head_dim*elt), multiple of 16
 *   page_stride_bytes  distance between consecutive pages of a pool, multiple of 16
 *   src_pages, dst_pages   device int32 [n_pairs]; dst entries must be distinct and
 *                      disjoint from src entries (pairs are copied concurrently)
 */
KB200_API int kb200_copy_pages(
    void* const* caches, int32_t n_caches, int64_t page_bytes, int64_t page_stride_bytes,
    int64_t n_pages, const int32_t* src_pages, const int32_t* dst_pages, int64_t n_pairs,
    int32_t device, void* stream);

/* ---------------------------------------------------------------------------
 * Paged split-KV decode attention (FlashAttention-forward semantics, paged KV).
 * Replaces attention.flash_attn_fwd for the paged call shapes of
 * kestrel/ops/attention.py:69-86 and kestrel/models/moondream/text.py:158-185:
 * q [B, Sq, H_q, D] (or packed rows with cu_seqlens_q), K/V gathered through
 * `page_table`, `seqused_k` keys per sequence INCLUDING the tokens appended this
 * step, GQA (q head h reads KV head h / (H_q / H_kv)), bottom-right aligned
 * causal mask, optional sliding window, fp32 softmax, FP8 KV dequantised as
 * code * scale.  Output has q's dtype and layout.
 */
typedef struct kb200_attn_args {
  uint32_t struct_bytes; /* sizeof(kb200_attn_args), for ABI checking */
  int32_t device;
  void* stream;

  const void* q; /* device, F16/BF16 */
  void* out;     /* device, same dtype as q */
  float* lse;    /* device fp32 [B, H_q, Sq] (natural log) or NULL; packed: [H_q, total_q] */
  int64_t q_batch_stride, q_row_stride, q_head_stride;
  int64_t o_batch_stride, o_row_stride, o_head_stride;

  const void* k_cache; /* device cache views, F16/BF16 (== q dtype) or E4M3 */
  const void* v_cache;
  int64_t kv_page_stride, kv_token_stride, kv_head_stride;
  int64_t n_pages;

  const int32_t* page_table; /* device int32 [B, >= ceil(seqused_k/P)], row stride given */
  int64_t pt_row_stride;
  const int32_t* seqused_k;    /* device int32 [B] */
  const int32_t* seqused_q;    /* device int32 [B] or NULL (all Sq rows valid) */
  const int32_t* cu_seqlens_q; /* device int32 [B+1] or NULL; when set q/out are packed
                                  [total_q, H_q, D] and q_batch_stride is ignored */

  int64_t batch;
  int64_t total_q;  /* B * Sq, or the packed row count */
  int32_t seqlen_q; /* Sq (padded layout); upper bound of rows per sequence when packed */
  int32_t n_q_heads, n_kv_heads, head_dim, page_size;
  int32_t q_dtype, kv_dtype;

  float softmax_scale;
  int32_t causal;      /* != 0: keys <= L - Sq_b + j for query row j */
  int32_t window_left; /* >= 0: also keys >= L - Sq_b + j - window_left (implies causal); < 0: off */

  float k_scale, v_scale;       /* dequantisation scales (python floats in the reference, */
  const float* k_scale_per_head; /* kv_cache.py:168-169); the device vectors [H_kv], when   */
  const float* v_scale_per_head; /* non-NULL, take precedence                               */

  void* workspace; /* device scratch, >= kb200_attn_workspace_bytes(...), 256-byte aligned */
  uint64_t workspace_bytes;

  /* Block-bidirectional (prefix-LM) mask, the mask_mod / aux_tensors call of
   * kestrel/models/moondream/text.py:139-172: query row j of a sequence also sees the keys of
   * its own sequence's rows up to q_visible_until[j] (>= j), on top of the causal part.  Device
   * int32, NULL for plain causal; indexed [b * q_visible_batch_stride + j] (padded layout) or
   * by packed row.  kb200_block_visibility builds it from the per-token block ids.  Needs
   * causal != 0 and no window. */
  const int32_t* q_visible_until;
  int64_t q_visible_batch_stride;

  /* Shared cached prefix (extension; the reference has no counterpart).  A promise by the caller:
   * the first shared_prefix_pages entries of every page-table row of this call are the same
   * physical pages (requests attached to one radix-cache prefix, kestrel/models/moondream/
   * runtime.py:1572-1623), all of them full, and every query row sees all of their keys
   * (seqused_k[b] - seqlen_q >= shared_prefix_pages * page_size under the causal mask).  The
   * call then reads those pages once for the whole batch: one pass of all query rows over the
   * prefix keys on the tensor-memory kernel, one pass per sequence over the remaining keys, and
   * a combine by the two log-sum-exps.  Same result as 0 up to rounding of the partial outputs
   * to q's dtype.  Ignored (plain path) with cu_seqlens_q, seqused_q, a window, a block mask,
   * fewer than 64 packed query rows in the batch, or q rows that are not evenly spaced across
   * the batch.  A sequence that breaks the promise sets KB200_STATUS_BAD_PREFIX. */
  int32_t shared_prefix_pages;
  int32_t reserved0;
} kb200_attn_args;

/* Scratch bytes kb200_paged_attention needs for the given problem bounds. */
KB200_API uint64_t kb200_attn_workspace_bytes(int64_t batch, int64_t total_q, int32_t n_q_heads,
                                    int32_t n_kv_heads, int32_t head_dim, int32_t device);

/* Scratch bytes the call described by `args` needs (workspace fields ignored): at most the bound
 * above, and much less for prefill-shaped calls (many query rows per sequence), which keep no
 * split-KV partials.  0 on invalid arguments. */
KB200_API uint64_t kb200_attn_workspace_bytes_for(const kb200_attn_args* args);

KB200_API int kb200_paged_attention(const kb200_attn_args* args);

/* ---------------------------------------------------------------------------
 * Visibility rows of the block-bidirectional mask.  `block_ids` int32 [batch, seqlen] holds,
 * per prompt position, an image-block id >= 0 or -1 for text
 * (kestrel/models/moondream/runtime.py:1671-1743); out[b, j] = last position of the run of
 * equal non-negative ids that contains j, or j itself for text.  A block is a contiguous run
 * (one per image occurrence, as the reference builds them).  Replaces the mask_mod callable
 * `attention.block_bidirectional_mask` + aux_tensors = [block_sequence_ids].
 */
KB200_API int kb200_block_visibility(const int32_t* block_ids, int64_t ids_row_stride, int64_t batch,
                                     int64_t seqlen, int32_t* out, int64_t out_row_stride, int32_t device,
                                     void* stream);

/* ---------------------------------------------------------------------------
 * Sampling hand-off: one token per row from the logits of a decode step.
 * Replaces kestrel_kernels' sampling.sample_step_from_logits(logits, temperatures,
 * top_ps, out=, generator=, logprobs_out=) as called right after the decoder stack
 * (kestrel/scheduler/scheduler.py:2986-2991, kestrel/scheduler/spatial.py:105-123).
 *
 *   logits        device [batch, vocab] of `logits_dtype` (F32/F16/BF16), row stride given
 *   temperatures  device fp32 [batch]; <= 1e-6 (kestrel/scheduler/scheduler.py:55) means
 *                 greedy: the first arg-max of the row, log-probability 0
 *   top_ps        device fp32 [batch]; the nucleus is {i : p_i >= tau} with tau the largest
 *                 probability whose tokens-at-or-above hold at least top_p of the mass
 *                 (>= 1: the whole vocabulary)
 *   uniforms      device fp32 [batch] in [0, 1): the row's random number (the Python
 *                 wrapper draws them from the caller's torch generator); the token is
 *                 the first one, in vocabulary order, whose running nucleus mass exceeds
 *                 u * nucleus_mass
 *   out_ids       device int64 [batch]
 *   logprobs      device fp32 [batch] or NULL: logits[id] / T - logsumexp(logits / T) over the
 *                 whole vocabulary (kestrel/scheduler/scheduler.py:3020-3042)
 * Deterministic: all masses are summed in 64-bit fixed point.  vocab <= 2^20.
 */
KB200_API int kb200_sample_step_from_logits(
    const void* logits, int32_t logits_dtype, int64_t batch, int64_t vocab, int64_t row_stride,
    const float* temperatures, const float* top_ps, const float* uniforms, int64_t* out_ids,
    float* logprobs, int32_t device, void* stream);

/* ---------------------------------------------------------------------------
 * kb200_paged_attention without a caller-provided scratch buffer.  This entry
 * point has no counterpart in the reference.
 *
 * Who needs it: hosts that may not (or cannot) create device allocations once
 * they are running -- an engine whose HBM is handed out completely at start-up
 * (Kestrel gives everything left after the weights to the KV pool), a plain C
 * or embedded host with no device allocator at hand, code that runs between
 * the begin and end of a stream capture.  kb200_paged_attention makes such a
 * caller find kb200_attn_workspace_bytes() of device memory first; this
 * variant brings its own.
 *
 * How: the scratch (per-sequence plan arrays and the split-KV partials) lives
 * in a fixed array inside the library's device image,
 * KB200_STATIC_SCRATCH_BYTES (32 MiB) per GPU that loads the library, held
 * until the process exits.  `args->workspace` and `args->workspace_bytes` are
 * ignored; every other field means what it means for kb200_paged_attention and
 * the results are the same.  The call allocates and frees nothing, on the host
 * API or through any library.
 *
 * Limits and rules:
 *   - the problem must fit: kb200_attn_workspace_bytes_for(args) <=
 *     KB200_STATIC_SCRATCH_BYTES (decode batches of up to 187 sequences at
 *     32 query / 8 KV heads, head_dim 128), otherwise KB200_ERR_WORKSPACE with a message saying how
 *     much was needed;
 *   - the first call on each device looks up the array's device address (one
 *     cudaGetSymbolAddress, no allocation): make that first call outside any
 *     stream capture;
 *   - all calls on one GPU share the one array, whatever their stream.  Nothing in
 *     it has to be zero on entry and nothing is carried from call to call (each
 *     call rewrites what it reads), but two calls that overlap in time on the
 *     same GPU would overwrite each other's partial results: run them one after
 *     another (same stream, or ordered by events).
 */
#define KB200_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)
KB200_API int kb200_paged_attention_static(const kb200_attn_args* args);

#ifdef __cplusplus
}
#endif
#endif /* KESTREL_B200_H_ */
