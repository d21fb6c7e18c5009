// Integer / copy kernels of the paged-KV path: append (with optional FP8
// quantise), slot mapping, decode metadata, copy-on-write page copy.
// All of them are pure HBM traffic; each thread moves 16 bytes per access and
// consecutive threads touch consecutive 16-byte chunks of a row.
#pragma once

#include "common.cuh"

namespace kb200 {

// ---------------------------------------------------------------------------
// Append
// ---------------------------------------------------------------------------
struct AppendParams {
  const char* key;
  const char* value;
  char* key_cache;
  char* value_cache;
  const int64_t* slots;
  const float* k_scale;
  const float* v_scale;
  int64_t key_token_stride_b;    // bytes
  int64_t value_token_stride_b;  // bytes
  int64_t page_stride_b, token_stride_b, head_stride_b;  // bytes, cache view
  int64_t num_tokens;
  int64_t n_slots_total;  // n_pages * page_size
  int32_t page_size, n_kv_heads, head_dim, n_scales;
};

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

// satfinite(rn(x / s)) as an e4m3fn code; the division is IEEE (no reciprocal).
__device__ __forceinline__ uint32_t quant2(float a, float b, float s) {
  float2 f = make_float2(__fdiv_rn(a, s), __fdiv_rn(b, s));
  return (uint32_t)__nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3);
}

// Copy mode: In == cache element, CHUNK bytes per thread (16, or the element
// size when pointers/strides are not 16-byte aligned).
template <int CHUNK>
__global__ void __launch_bounds__(256) append_copy_kernel(const AppendParams p, int row_bytes) {
  pdl_wait();
  pdl_launch_dependents();
  const int chunks_per_row = row_bytes / CHUNK;
  const int64_t per_tensor = p.num_tokens * p.n_kv_heads * chunks_per_row;
  const int64_t total = 2 * per_tensor;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int kv = i >= per_tensor;
    int64_t r = kv ? i - per_tensor : i;
    const int c = (int)(r % chunks_per_row);
    r /= chunks_per_row;
    const int h = (int)(r % p.n_kv_heads);
    const int64_t t = r / p.n_kv_heads;
    const int64_t slot = p.slots[t];
    if (slot < 0) continue;
    if (slot >= p.n_slots_total) {
      if (c == 0 && h == 0 && kv == 0) report(KB200_STATUS_BAD_SLOT, (int)slot, KID_APPEND);
      continue;
    }
    const int64_t page = slot / p.page_size;
    const int off = (int)(slot - page * p.page_size);
    const char* src = (kv ? p.value + t * p.value_token_stride_b : p.key + t * p.key_token_stride_b) +
                      (int64_t)h * row_bytes + (int64_t)c * CHUNK;
    char* dst = (kv ? p.value_cache : p.key_cache) + page * p.page_stride_b +
                off * p.token_stride_b + h * p.head_stride_b + (int64_t)c * CHUNK;
    if constexpr (CHUNK == 16) {
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
    } else if constexpr (CHUNK == 4) {
      *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(src);
    } else if constexpr (CHUNK == 2) {
      *reinterpret_cast<uint16_t*>(dst) = *reinterpret_cast<const uint16_t*>(src);
    } else {
      *dst = *src;
    }
  }
}

// Quantise mode: In in {float, half, bf16} -> e4m3 codes.  EPT elements per
// thread: 16 (one 16-byte store) when aligned, else 2.
template <typename In, int EPT>
__global__ void __launch_bounds__(256) append_quant_kernel(const AppendParams p) {
  pdl_wait();
  pdl_launch_dependents();
  const int chunks_per_row = p.head_dim / EPT;
  const int64_t per_tensor = p.num_tokens * p.n_kv_heads * chunks_per_row;
  const int64_t total = 2 * per_tensor;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int kv = i >= per_tensor;
    int64_t r = kv ? i - per_tensor : i;
    const int c = (int)(r % chunks_per_row);
    r /= chunks_per_row;
    const int h = (int)(r % p.n_kv_heads);
    const int64_t t = r / p.n_kv_heads;
    const int64_t slot = p.slots[t];
    if (slot < 0) continue;
    if (slot >= p.n_slots_total) {
      if (c == 0 && h == 0 && kv == 0) report(KB200_STATUS_BAD_SLOT, (int)slot, KID_APPEND);
      continue;
    }
    const int64_t page = slot / p.page_size;
    const int off = (int)(slot - page * p.page_size);
    const In* src = reinterpret_cast<const In*>(
                        kv ? p.value + t * p.value_token_stride_b : p.key + t * p.key_token_stride_b) +
                    (int64_t)h * p.head_dim + (int64_t)c * EPT;
    char* dst = (kv ? p.value_cache : p.key_cache) + page * p.page_stride_b +
                off * p.token_stride_b + h * p.head_stride_b + (int64_t)c * EPT;
    const float* sp = kv ? p.v_scale : p.k_scale;
    const float s = sp[p.n_scales == 1 ? 0 : h];
    if constexpr (EPT == 16) {
      In x[16];
      constexpr int NV = (int)(16 * sizeof(In) / 16);
      const uint4* s4 = reinterpret_cast<const uint4*>(src);
      uint4* x4 = reinterpret_cast<uint4*>(x);
#pragma unroll
      for (int v = 0; v < NV; ++v) x4[v] = s4[v];
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t lo = quant2(to_float(x[4 * j + 0]), to_float(x[4 * j + 1]), s);
        uint32_t hi = quant2(to_float(x[4 * j + 2]), to_float(x[4 * j + 3]), s);
        w[j] = lo | (hi << 16);
      }
      *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      uint32_t q = quant2(to_float(src[0]), to_float(src[1]), s);
      dst[0] = (char)(q & 0xff);
      dst[1] = (char)(q >> 8);
    }
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

inline int launch_append(const void* key, const void* value, int64_t key_token_stride,
                         int64_t value_token_stride, void* key_cache, void* value_cache,
                         int64_t cache_page_stride, int64_t cache_token_stride,
                         int64_t cache_head_stride, const int64_t* slot_mapping, int64_t num_tokens,
                         int64_t n_pages, int32_t page_size, int32_t n_kv_heads, int32_t head_dim,
                         int32_t in_dtype, int32_t cache_dtype, const float* k_scale,
                         const float* v_scale, int32_t n_scales, cudaStream_t stream) {
  KB200_REQUIRE(num_tokens >= 0, "num_tokens must be non-negative");
  if (num_tokens == 0) return KB200_OK;
  KB200_REQUIRE(key && value && key_cache && value_cache && slot_mapping, "null pointer argument");
  KB200_REQUIRE(page_size > 0 && n_kv_heads > 0 && head_dim > 0 && n_pages > 0,
                "page_size, n_kv_heads, head_dim and n_pages must be positive");
  const int in_sz = dtype_size(in_dtype), c_sz = dtype_size(cache_dtype);
  KB200_REQUIRE(in_sz && c_sz, "unknown dtype");
  const bool quant = cache_dtype == KB200_DTYPE_E4M3;
  if (quant) {
    KB200_REQUIRE(in_dtype != KB200_DTYPE_E4M3, "FP8 input rows are not supported");
    KB200_REQUIRE(k_scale && v_scale, "FP8 append requires k_scale and v_scale");
    KB200_REQUIRE(n_scales == 1 || n_scales == n_kv_heads, "n_scales must be 1 or n_kv_heads");
    KB200_REQUIRE(head_dim % 2 == 0, "FP8 append requires an even head_dim");
  } else {
    KB200_REQUIRE(in_dtype == cache_dtype, "input dtype must equal cache dtype (or cache must be E4M3)");
  }

  AppendParams p;
  p.key = static_cast<const char*>(key);
  p.value = static_cast<const char*>(value);
  p.key_cache = static_cast<char*>(key_cache);
  p.value_cache = static_cast<char*>(value_cache);
  p.slots = slot_mapping;
  p.k_scale = k_scale;
  p.v_scale = v_scale;
  p.key_token_stride_b = key_token_stride * in_sz;
  p.value_token_stride_b = value_token_stride * in_sz;
  p.page_stride_b = cache_page_stride * c_sz;
  p.token_stride_b = cache_token_stride * c_sz;
  p.head_stride_b = cache_head_stride * c_sz;
  p.num_tokens = num_tokens;
  p.n_slots_total = n_pages * page_size;
  p.page_size = page_size;
  p.n_kv_heads = n_kv_heads;
  p.head_dim = head_dim;
  p.n_scales = n_scales;

  const int row_in_bytes = head_dim * in_sz;
  const int row_out_bytes = head_dim * c_sz;
  const bool vec_ok = aligned16(key) && aligned16(value) && aligned16(key_cache) &&
                      aligned16(value_cache) && p.key_token_stride_b % 16 == 0 &&
                      p.value_token_stride_b % 16 == 0 && p.page_stride_b % 16 == 0 &&
                      p.token_stride_b % 16 == 0 && p.head_stride_b % 16 == 0 &&
                      row_out_bytes % 16 == 0 && row_in_bytes % 16 == 0;
  const int threads = 256;
  auto blocks_for = [&](int64_t items) {
    int64_t b = (items + threads - 1) / threads;
    const int64_t cap = 148 * 16;  // grid-stride beyond this
    return (int)(b < 1 ? 1 : (b > cap ? cap : b));
  };
  if (!quant) {
    if (vec_ok) {
      int64_t items = 2 * num_tokens * n_kv_heads * (row_out_bytes / 16);
      KB200_CUDA_OK(launch_kernel(append_copy_kernel<16>, dim3(blocks_for(items)), dim3(threads), 0, stream, p, row_out_bytes));
    } else {
      int64_t items = 2 * num_tokens * n_kv_heads * head_dim;
      if (c_sz == 4)
        KB200_CUDA_OK(launch_kernel(append_copy_kernel<4>, dim3(blocks_for(items)), dim3(threads), 0, stream, p, row_out_bytes));
      else if (c_sz == 2)
        KB200_CUDA_OK(launch_kernel(append_copy_kernel<2>, dim3(blocks_for(items)), dim3(threads), 0, stream, p, row_out_bytes));
      else
        KB200_CUDA_OK(launch_kernel(append_copy_kernel<1>, dim3(blocks_for(items)), dim3(threads), 0, stream, p, row_out_bytes));
    }
  } else {
    if (vec_ok) {
      int64_t items = 2 * num_tokens * n_kv_heads * (head_dim / 16);
      if (in_dtype == KB200_DTYPE_BF16)
        KB200_CUDA_OK(launch_kernel(append_quant_kernel<__nv_bfloat16, 16>, dim3(blocks_for(items)), dim3(threads), 0, stream, p));
      else if (in_dtype == KB200_DTYPE_F16)
        KB200_CUDA_OK(launch_kernel(append_quant_kernel<__half, 16>, dim3(blocks_for(items)), dim3(threads), 0, stream, p));
      else
        KB200_CUDA_OK(launch_kernel(append_quant_kernel<float, 16>, dim3(blocks_for(items)), dim3(threads), 0, stream, p));
    } else {
      int64_t items = 2 * num_tokens * n_kv_heads * (head_dim / 2);
      if (in_dtype == KB200_DTYPE_BF16)
        KB200_CUDA_OK(launch_kernel(append_quant_kernel<__nv_bfloat16, 2>, dim3(blocks_for(items)), dim3(threads), 0, stream, p));
      else if (in_dtype == KB200_DTYPE_F16)
        KB200_CUDA_OK(launch_kernel(append_quant_kernel<__half, 2>, dim3(blocks_for(items)), dim3(threads), 0, stream, p));
      else
        KB200_CUDA_OK(launch_kernel(append_quant_kernel<float, 2>, dim3(blocks_for(items)), dim3(threads), 0, stream, p));
    }
  }
  KB200_CUDA_OK(cudaGetLastError());
  return KB200_OK;
}

// ---------------------------------------------------------------------------
// Slot mapping
// ---------------------------------------------------------------------------
template <typename BI, typename PI>
__global__ void __launch_bounds__(256)
slot_mapping_kernel(const int32_t* __restrict__ page_table, int64_t pt_row_stride, int64_t pt_rows,
                    int64_t pt_cols, const BI* __restrict__ batch_idx, int batch_per_row,
                    int64_t row_len, const PI* __restrict__ positions, int64_t* __restrict__ out,
                    int64_t n, int page_size) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t b = (int64_t)batch_idx[batch_per_row ? i / row_len : i];
    const int64_t pos = (int64_t)positions[i];
    // floor division / non-negative remainder, as torch's `//` and `%`
    int64_t blk = pos / page_size;
    int64_t off = pos - blk * page_size;
    if (off < 0) { off += page_size; blk -= 1; }
    if (b < 0 || b >= pt_rows || blk < 0 || blk >= pt_cols) {
      report(KB200_STATUS_BAD_ROW, (int)b, KID_SLOT_MAPPING);
      out[i] = -1;
      continue;
    }
    const int64_t phys = page_table[b * pt_row_stride + blk];
    out[i] = phys * page_size + off;
  }
}

inline int launch_slot_mapping(const int32_t* page_table, int64_t pt_row_stride, int64_t pt_rows,
                               int64_t pt_cols, const void* batch_idx, int32_t bi64,
                               int32_t batch_per_row, int64_t row_len, const void* positions,
                               int32_t pi64, int64_t* out, int64_t n, int32_t page_size,
                               cudaStream_t stream) {
  if (n == 0) return KB200_OK;
  KB200_REQUIRE(n > 0, "n must be non-negative");
  KB200_REQUIRE(page_table && batch_idx && positions && out, "null pointer argument");
  KB200_REQUIRE(page_size > 0, "page_size must be positive");
  KB200_REQUIRE(!batch_per_row || row_len > 0, "row_len must be positive");
  const int threads = 256;
  int64_t nb = (n + threads - 1) / threads;
  const int blocks = (int)(nb > 148 * 16 ? 148 * 16 : nb);
#define KB200_SM_LAUNCH(BI, PI)                                                             \
  slot_mapping_kernel<BI, PI><<<blocks, threads, 0, stream>>>(                              \
      page_table, pt_row_stride, pt_rows, pt_cols, static_cast<const BI*>(batch_idx),       \
      batch_per_row, row_len, static_cast<const PI*>(positions), out, n, page_size)
  if (bi64 && pi64) KB200_SM_LAUNCH(int64_t, int64_t);
  else if (bi64) KB200_SM_LAUNCH(int64_t, int32_t);
  else if (pi64) KB200_SM_LAUNCH(int32_t, int64_t);
  else KB200_SM_LAUNCH(int32_t, int32_t);
#undef KB200_SM_LAUNCH
  KB200_CUDA_OK(cudaGetLastError());
  return KB200_OK;
}

// ---------------------------------------------------------------------------
// Decode metadata (compact page table + seqused_k)
// ---------------------------------------------------------------------------
template <typename BI>
__global__ void __launch_bounds__(128)
paged_kv_metadata_kernel(const int32_t* __restrict__ page_table, int64_t pt_row_stride,
                         int64_t pt_rows, int64_t pt_cols, const BI* __restrict__ batch_idx,
                         const int32_t* __restrict__ input_pos, int32_t* __restrict__ out_page_table,
                         int64_t out_row_stride, int64_t out_cols, int32_t* __restrict__ out_seqused_k,
                         int page_size) {
  const int64_t r = blockIdx.x;
  const int64_t b = (int64_t)batch_idx[r];
  const int used = input_pos[r] + 1;
  if (threadIdx.x == 0) out_seqused_k[r] = used;
  if (b < 0 || b >= pt_rows) {
    if (threadIdx.x == 0) report(KB200_STATUS_BAD_ROW, (int)b, KID_METADATA);
    return;
  }
  int64_t n = used > 0 ? (used + page_size - 1) / page_size : 0;
  if (n > pt_cols) n = pt_cols;
  if (n > out_cols) n = out_cols;
  const int32_t* src = page_table + b * pt_row_stride;
  int32_t* dst = out_page_table + r * out_row_stride;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
}

inline int launch_metadata(const int32_t* page_table, int64_t pt_row_stride, int64_t pt_rows,
                           int64_t pt_cols, const void* batch_idx, int32_t bi64,
                           const int32_t* input_pos, int32_t* out_page_table, int64_t out_row_stride,
                           int64_t out_cols, int32_t* out_seqused_k, int64_t batch, int32_t page_size,
                           cudaStream_t stream) {
  if (batch == 0) return KB200_OK;
  KB200_REQUIRE(batch > 0, "batch must be non-negative");
  KB200_REQUIRE(page_table && batch_idx && input_pos && out_page_table && out_seqused_k,
                "null pointer argument");
  KB200_REQUIRE(page_size > 0, "page_size must be positive");
  KB200_REQUIRE(batch <= 0x7fffffff, "batch too large");
  if (bi64)
    paged_kv_metadata_kernel<int64_t><<<(int)batch, 128, 0, stream>>>(
        page_table, pt_row_stride, pt_rows, pt_cols, static_cast<const int64_t*>(batch_idx), input_pos,
        out_page_table, out_row_stride, out_cols, out_seqused_k, page_size);
  else
    paged_kv_metadata_kernel<int32_t><<<(int)batch, 128, 0, stream>>>(
        page_table, pt_row_stride, pt_rows, pt_cols, static_cast<const int32_t*>(batch_idx), input_pos,
        out_page_table, out_row_stride, out_cols, out_seqused_k, page_size);
  KB200_CUDA_OK(cudaGetLastError());
  return KB200_OK;
}

// ---------------------------------------------------------------------------
// Copy-on-write page copy
// ---------------------------------------------------------------------------
constexpr int kCopyMaxCaches = 96;  // pointers per launch (passed by value)

struct CopyPagesParams {
  char* caches[kCopyMaxCaches];
  const int32_t* src;
  const int32_t* dst;
  int64_t page_bytes, page_stride_bytes, n_pages;
};

// grid = (pairs, caches); each block streams one page of one pool, 16 B per
// thread per step, four independent loads in flight per thread.
__global__ void __launch_bounds__(256) copy_pages_kernel(const CopyPagesParams p) {
  const int64_t pair = blockIdx.x;
  const int32_t s = p.src[pair], d = p.dst[pair];
  if (s < 0 || s >= p.n_pages || d < 0 || d >= p.n_pages) {
    if (threadIdx.x == 0 && blockIdx.y == 0) report(KB200_STATUS_BAD_PAGE, s < 0 || s >= p.n_pages ? s : d, KID_COPY_PAGES);
    return;
  }
  if (s == d) return;
  char* base = p.caches[blockIdx.y];
  const uint4* src = reinterpret_cast<const uint4*>(base + s * p.page_stride_bytes);
  uint4* dst = reinterpret_cast<uint4*>(base + d * p.page_stride_bytes);
  const int64_t n = p.page_bytes / 16;
  int64_t i = threadIdx.x;
  for (; i + 3 * 256 < n; i += 4 * 256) {
    uint4 a = src[i], b = src[i + 256], c = src[i + 512], e = src[i + 768];
    dst[i] = a; dst[i + 256] = b; dst[i + 512] = c; dst[i + 768] = e;
  }
  for (; i < n; i += 256) dst[i] = src[i];
}

inline int launch_copy_pages(void* const* caches, int32_t n_caches, int64_t page_bytes,
                             int64_t page_stride_bytes, int64_t n_pages, const int32_t* src_pages,
                             const int32_t* dst_pages, int64_t n_pairs, cudaStream_t stream) {
  if (n_pairs == 0 || n_caches == 0) return KB200_OK;
  KB200_REQUIRE(n_pairs > 0 && n_caches > 0, "n_pairs and n_caches must be non-negative");
  KB200_REQUIRE(caches && src_pages && dst_pages, "null pointer argument");
  KB200_REQUIRE(page_bytes > 0 && page_bytes % 16 == 0, "page_bytes must be a positive multiple of 16");
  KB200_REQUIRE(page_stride_bytes >= page_bytes && page_stride_bytes % 16 == 0,
                "page_stride_bytes must be a multiple of 16 and >= page_bytes");
  KB200_REQUIRE(n_pairs <= 0x7fffffff, "too many page pairs");
  for (int32_t c0 = 0; c0 < n_caches; c0 += kCopyMaxCaches) {
    const int nc = n_caches - c0 < kCopyMaxCaches ? n_caches - c0 : kCopyMaxCaches;
    CopyPagesParams p;
    for (int i = 0; i < nc; ++i) {
      KB200_REQUIRE(caches[c0 + i] && aligned16(caches[c0 + i]), "cache pointers must be 16-byte aligned");
      p.caches[i] = static_cast<char*>(caches[c0 + i]);
    }
    p.src = src_pages;
    p.dst = dst_pages;
    p.page_bytes = page_bytes;
    p.page_stride_bytes = page_stride_bytes;
    p.n_pages = n_pages;
    dim3 grid((unsigned)n_pairs, (unsigned)nc);
    copy_pages_kernel<<<grid, 256, 0, stream>>>(p);
    KB200_CUDA_OK(cudaGetLastError());
  }
  return KB200_OK;
}

}  // namespace kb200
