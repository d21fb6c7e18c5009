// C ABI of the paged-KV library (see include/kestrel_b200.h for the contract).
// One translation unit: the kernels live in the .cuh files next to this one.
#include "common.cuh"
#include "cache_ops.cuh"
#include "rope_append.cuh"
#include "paged_attention.cuh"
#include "paged_prefill.cuh"
#include "sampling.cuh"

using namespace kb200;

#define KB200_ENTER(dev)                                                          \
  DeviceGuard _guard(dev);                                                        \
  if (!_guard.ok) return fail(KB200_ERR_CUDA, "cannot switch to CUDA device %d", (int)(dev))

extern "C" {

int kb200_abi_version(void) { return KB200_ABI_VERSION; }

const char* kb200_last_error(void) { return err_buf(); }

int kb200_device_status(int device, int32_t out[4], int clear) {
  KB200_ENTER(device);
  KB200_REQUIRE(out != nullptr, "out is null");
  KB200_CUDA_OK(cudaDeviceSynchronize());
  int host[4] = {0, 0, 0, 0};
  KB200_CUDA_OK(cudaMemcpyFromSymbol(host, g_status, sizeof(host)));
  for (int i = 0; i < 4; ++i) out[i] = host[i];
  if (clear) {
    int zero[4] = {0, 0, 0, 0};
    KB200_CUDA_OK(cudaMemcpyToSymbol(g_status, zero, sizeof(zero)));
  }
  return KB200_OK;
}

int kb200_reshape_and_cache_flash(const void* key, const void* value, int64_t key_token_stride,
                                  int64_t value_token_stride, void* key_cache, void* value_cache,
                                  int64_t cache_page_stride, int64_t cache_token_stride,
                                  int64_t cache_head_stride, const int64_t* slot_mapping,
                                  int64_t num_tokens, int64_t n_pages, int32_t page_size,
                                  int32_t n_kv_heads, int32_t head_dim, int32_t in_dtype,
                                  int32_t cache_dtype, const float* k_scale, const float* v_scale,
                                  int32_t n_scales, int32_t device, void* stream) {
  KB200_ENTER(device);
  return launch_append(key, value, key_token_stride, value_token_stride, key_cache, value_cache,
                       cache_page_stride, cache_token_stride, cache_head_stride, slot_mapping, num_tokens,
                       n_pages, page_size, n_kv_heads, head_dim, in_dtype, cache_dtype, k_scale, v_scale,
                       n_scales, static_cast<cudaStream_t>(stream));
}

int kb200_build_slot_mapping(const int32_t* page_table, int64_t pt_row_stride, int64_t pt_rows,
                             int64_t pt_cols, const void* batch_idx, int32_t batch_idx_is_i64,
                             int32_t batch_per_row, int64_t row_len, const void* positions,
                             int32_t positions_is_i64, int64_t* out_slots, int64_t n, int32_t page_size,
                             int32_t device, void* stream) {
  KB200_ENTER(device);
  return launch_slot_mapping(page_table, pt_row_stride, pt_rows, pt_cols, batch_idx, batch_idx_is_i64,
                             batch_per_row, row_len, positions, positions_is_i64, out_slots, n, page_size,
                             static_cast<cudaStream_t>(stream));
}

int kb200_build_paged_kv_metadata(const int32_t* page_table, int64_t pt_row_stride, int64_t pt_rows,
                                  int64_t pt_cols, const void* batch_idx, int32_t batch_idx_is_i64,
                                  const int32_t* input_pos, int32_t* out_page_table, int64_t out_row_stride,
                                  int64_t out_cols, int32_t* out_seqused_k, int64_t batch, int32_t page_size,
                                  int32_t device, void* stream) {
  KB200_ENTER(device);
  return launch_metadata(page_table, pt_row_stride, pt_rows, pt_cols, batch_idx, batch_idx_is_i64, input_pos,
                         out_page_table, out_row_stride, out_cols, out_seqused_k, batch, page_size,
                         static_cast<cudaStream_t>(stream));
}

int kb200_build_decode_step_metadata(const int32_t* page_table, int64_t pt_row_stride, int64_t pt_rows,
                                     int64_t pt_cols, const void* batch_idx, int32_t batch_idx_is_i64,
                                     const int32_t* input_pos, int32_t* out_page_table, int64_t out_row_stride,
                                     int64_t out_cols, int32_t* out_seqused_k, int64_t* out_slots,
                                     int64_t* out_positions, int64_t batch, int32_t n_new, int32_t page_size,
                                     int32_t device, void* stream) {
  KB200_ENTER(device);
  return launch_decode_step_metadata(page_table, pt_row_stride, pt_rows, pt_cols, batch_idx, batch_idx_is_i64,
                                     input_pos, out_page_table, out_row_stride, out_cols, out_seqused_k, out_slots,
                                     out_positions, batch, n_new, page_size, static_cast<cudaStream_t>(stream));
}

int kb200_rope_append(void* q, void* k, const void* v, int64_t q_token_stride, int64_t k_token_stride,
                      int64_t v_token_stride, int64_t num_tokens, int32_t n_q_heads, int32_t n_kv_heads,
                      int32_t head_dim, int32_t rot_dim, const void* positions, int32_t positions_is_i64,
                      const float* cos_sin_cache, int64_t max_pos, int64_t cos_sin_row_stride, void* key_cache,
                      void* value_cache, int64_t cache_page_stride, int64_t cache_token_stride,
                      int64_t cache_head_stride, const int64_t* slot_mapping, int64_t n_pages, int32_t page_size,
                      int32_t in_dtype, int32_t cache_dtype, const float* k_scale, const float* v_scale,
                      int32_t n_scales, int32_t write_k, int32_t device, void* stream) {
  KB200_ENTER(device);
  RopeAppendArgs a;
  a.q = q; a.k = k; a.v = v;
  a.q_token_stride = q_token_stride; a.k_token_stride = k_token_stride; a.v_token_stride = v_token_stride;
  a.num_tokens = num_tokens;
  a.n_q_heads = n_q_heads; a.n_kv_heads = n_kv_heads; a.head_dim = head_dim; a.rot_dim = rot_dim;
  a.positions = positions; a.positions_is_i64 = positions_is_i64;
  a.cos_sin_cache = cos_sin_cache; a.max_pos = max_pos; a.cos_sin_row_stride = cos_sin_row_stride;
  a.key_cache = key_cache; a.value_cache = value_cache;
  a.cache_page_stride = cache_page_stride; a.cache_token_stride = cache_token_stride;
  a.cache_head_stride = cache_head_stride;
  a.slot_mapping = slot_mapping; a.n_pages = n_pages; a.page_size = page_size;
  a.in_dtype = in_dtype; a.cache_dtype = cache_dtype;
  a.k_scale = k_scale; a.v_scale = v_scale; a.n_scales = n_scales; a.write_k = write_k;
  return launch_rope_append(a, static_cast<cudaStream_t>(stream));
}

int kb200_copy_pages(void* const* caches, int32_t n_caches, int64_t page_bytes, int64_t page_stride_bytes,
                     int64_t n_pages, const int32_t* src_pages, const int32_t* dst_pages, int64_t n_pairs,
                     int32_t device, void* stream) {
  KB200_ENTER(device);
  return launch_copy_pages(caches, n_caches, page_bytes, page_stride_bytes, n_pages, src_pages, dst_pages,
                           n_pairs, static_cast<cudaStream_t>(stream));
}

uint64_t kb200_attn_workspace_bytes(int64_t batch, int64_t total_q, int32_t n_q_heads, int32_t n_kv_heads,
                                    int32_t head_dim, int32_t device) {
  if (batch <= 0 || total_q <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0) return 0;
  int sms = 0;
  if (device_sm_count(device, &sms) != KB200_OK) return 0;
  // a call of these dimensions can reach the 32-row kernel (two partial slots per worker) only when a sequence
  // brings more than 16 packed rows on average
  const bool rows32_possible = (int64_t)(n_q_heads / n_kv_heads) * ((total_q + batch - 1) / batch) > kRowsPerSeg;
  uint64_t need = attn_workspace_layout(batch, total_q, n_q_heads, n_kv_heads, head_dim, sms * kAttnMaxWarps, rows32_possible).total;
  // e4m3 pools with pages of one or two tokens read several KV heads as one wide head of 256 (attn_head_pack):
  // fewer segments, wider partials
  for (int pack = 2; pack <= (head_dim == 64 ? 4 : head_dim == 128 ? 2 : 1); pack *= 2)
    if (n_kv_heads % pack == 0)
      need = std::max<uint64_t>(need, attn_workspace_layout(batch, total_q, n_q_heads, n_kv_heads / pack, head_dim * pack,
                                                            sms * kAttnMaxWarps, false).total);
  return need;
}

uint64_t kb200_attn_workspace_bytes_for(const kb200_attn_args* args) {
  if (!args || args->struct_bytes != sizeof(kb200_attn_args)) return 0;
  if (args->batch <= 0 || args->total_q <= 0 || args->n_q_heads <= 0 || args->n_kv_heads <= 0 || args->head_dim <= 0)
    return 0;
  int sms = 0;
  if (device_sm_count(args->device, &sms) != KB200_OK) return 0;
  return attn_workspace_need(args, sms);
}

int kb200_block_visibility(const int32_t* block_ids, int64_t ids_row_stride, int64_t batch, int64_t seqlen,
                           int32_t* out, int64_t out_row_stride, int32_t device, void* stream) {
  KB200_ENTER(device);
  return launch_block_visibility(block_ids, ids_row_stride, batch, seqlen, out, out_row_stride,
                                 static_cast<cudaStream_t>(stream));
}

int kb200_sample_step_from_logits(const void* logits, int32_t logits_dtype, int64_t batch, int64_t vocab,
                                  int64_t row_stride, const float* temperatures, const float* top_ps,
                                  const float* uniforms, int64_t* out_ids, float* logprobs, int32_t device,
                                  void* stream) {
  KB200_ENTER(device);
  return launch_sample_step(logits, logits_dtype, batch, vocab, row_stride, temperatures, top_ps, uniforms, out_ids,
                            logprobs, static_cast<cudaStream_t>(stream));
}

int kb200_paged_attention(const kb200_attn_args* args) {
  if (!args) return fail(KB200_ERR_INVALID, "args is null");
  KB200_ENTER(args->device);
  return launch_paged_attention(args);
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Allocation-free variant: the scratch is a fixed array in the device image.
// In host code `g_static_scratch` is only a handle for the symbol, not an
// address a kernel could use; the device address is looked up once per GPU,
// with that GPU current, and cached.
// ---------------------------------------------------------------------------

static __device__ __align__(256) unsigned char g_static_scratch[KB200_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_mu;
void* g_static_ptr[64] = {nullptr};

// Device address of g_static_scratch on `device` (which must be the current device).
int static_scratch_address(int device, void** out) {
  if (device < 0 || device >= 64) return fail(KB200_ERR_INVALID, "device index %d out of range", device);
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (!g_static_ptr[device]) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || !ptr)
      return fail(KB200_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed on device %d: %s", device,
                  cudaGetErrorString(e));
    g_static_ptr[device] = ptr;
  }
  *out = g_static_ptr[device];
  return KB200_OK;
}
}  // namespace

extern "C" {

int kb200_paged_attention_static(const kb200_attn_args* args) {
  if (!args) return fail(KB200_ERR_INVALID, "args is null");
  if (args->struct_bytes != sizeof(kb200_attn_args))
    return fail(KB200_ERR_INVALID, "kb200_attn_args size mismatch: got %u, built with %zu", args->struct_bytes,
                sizeof(kb200_attn_args));
  KB200_ENTER(args->device);
  if (args->batch > 0 && args->total_q > 0) {
    const uint64_t need = kb200_attn_workspace_bytes_for(args);
    if (need == 0) return fail(KB200_ERR_INVALID, "cannot size the scratch for these arguments");
    if (need > KB200_STATIC_SCRATCH_BYTES)
      return fail(KB200_ERR_WORKSPACE,
                  "problem needs %llu bytes of scratch, the built-in buffer holds %u: use kb200_paged_attention "
                  "with a caller-provided workspace",
                  (unsigned long long)need, (unsigned)KB200_STATIC_SCRATCH_BYTES);
  }
  void* scratch = nullptr;
  if (int rc = static_scratch_address(args->device, &scratch)) return rc;
  kb200_attn_args local = *args;
  local.workspace = scratch;
  local.workspace_bytes = KB200_STATIC_SCRATCH_BYTES;
  return launch_paged_attention(&local);
}

}  // extern "C"
