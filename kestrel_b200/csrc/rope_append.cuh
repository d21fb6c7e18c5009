// Rotary embedding fused with the append, and the fused per-step decode metadata.
//
// rope_append_kernel rotates Q in place and, in the same pass, rotates K, writes
// it back (optional) and scatters rotated K plus V into the pool pages by slot
// (optionally quantising to e4m3).  Compared with a rotary launch followed by an
// append launch it saves one launch and one read of K per layer.
//
// Arithmetic (NeoX layout, partial rotary): for i < rot/2, with c = cos[pos][i],
// s = sin[pos][i] in fp32 and x1 = x[i], x2 = x[i + rot/2] widened to fp32:
//     y1 = rn(rn(x1*c) - rn(x2*s))      y2 = rn(rn(x2*c) + rn(x1*s))
// (separately rounded products: no fused multiply-add), then rounded once to the
// row dtype.  The pool receives exactly the bytes an append of the rotated row
// would have written, so fused and unfused paths are bit-identical.
#pragma once

#include "common.cuh"
#include "cache_ops.cuh"

namespace kb200 {

// Exact n / d for 0 <= n < 2^31 and a divisor fixed at launch: one wide multiply and a shift
// (m = floor(2^(31+s) / d) + 1 with s = ceil(log2 d); the error term n * (m d - 2^(31+s)) stays below 2^(31+s)).
struct FastDiv {
  uint32_t d, m, sh;
  __host__ static FastDiv make(uint32_t d_) {
    FastDiv f;
    f.d = d_ ? d_ : 1;
    uint32_t s = 0;
    while ((1ull << s) < f.d) ++s;
    f.sh = 31 + s;
    f.m = (uint32_t)((1ull << f.sh) / f.d + 1);
    return f;
  }
  __device__ __forceinline__ uint32_t div(uint32_t n) const { return (uint32_t)(((uint64_t)n * m) >> sh); }
};

struct RopeAppendParams {
  char* q;            // [T, Hq, D] rows, rotated in place (may be null: no query rotation)
  char* k;            // [T, Hkv, D] rows
  const char* v;      // [T, Hkv, D] rows (null when there is no append)
  const void* positions;
  const float* cos_sin;   // [max_pos, rot_dim]: cos (rot/2) then sin (rot/2)
  char* key_cache;        // null: rotate only
  char* value_cache;
  const int64_t* slots;
  const float* k_scale;
  const float* v_scale;
  int64_t q_token_stride_b, k_token_stride_b, v_token_stride_b;
  int64_t page_stride_b, token_stride_b, head_stride_b;
  int64_t cos_sin_row_stride, max_pos;
  int64_t num_tokens, n_slots_total;
  int32_t n_q_heads, n_kv_heads, head_dim, rot_dim, page_size, n_scales;
  int32_t positions_is_i64, write_k, quant;
  int32_t cs_vec;                 // cos/sin rows can be read 16 bytes at a time
  FastDiv d_token, d_rot, d_pass, d_copy, d_page;   // per_token, rot/pass/copy items per head, page_size
  int64_t token_base;             // first token of this launch (launches are cut below 2^31 items)
};

template <typename In>
__device__ __forceinline__ In from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

template <typename In, int EPT>
struct __align__(16) Vec {
  In e[EPT];
};

template <typename In, int EPT>
__device__ __forceinline__ void load_vec(Vec<In, EPT>& d, const char* src) {
  if constexpr (EPT == 1) {
    d.e[0] = *reinterpret_cast<const In*>(src);
  } else {
    constexpr int NV = (int)(EPT * sizeof(In) / 16);
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(d.e);
#pragma unroll
    for (int i = 0; i < NV; ++i) d4[i] = s4[i];
  }
}
template <typename In, int EPT>
__device__ __forceinline__ void store_vec(char* dst, const Vec<In, EPT>& d) {
  if constexpr (EPT == 1) {
    *reinterpret_cast<In*>(dst) = d.e[0];
  } else {
    constexpr int NV = (int)(EPT * sizeof(In) / 16);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    const uint4* s4 = reinterpret_cast<const uint4*>(d.e);
#pragma unroll
    for (int i = 0; i < NV; ++i) d4[i] = s4[i];
  }
}
// e4m3 codes of EPT values (EPT == 8: one 8-byte store; EPT == 1: one byte)
template <typename In, int EPT>
__device__ __forceinline__ void store_quant(char* dst, const Vec<In, EPT>& d, float scale) {
  if constexpr (EPT == 1) {
    const uint32_t q = quant2(to_float(d.e[0]), 0.f, scale);
    *dst = (char)(q & 0xff);
  } else {
    uint32_t w[EPT / 4];
#pragma unroll
    for (int j = 0; j < EPT / 4; ++j) {
      const uint32_t lo = quant2(to_float(d.e[4 * j + 0]), to_float(d.e[4 * j + 1]), scale);
      const uint32_t hi = quant2(to_float(d.e[4 * j + 2]), to_float(d.e[4 * j + 3]), scale);
      w[j] = lo | (hi << 16);
    }
    *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
  }
}

// One work item = EPT consecutive elements of one (token, head) row:
//   Q heads:  rot/2/EPT rotation items (each touches the chunk and its partner at +rot/2)
//   K heads:  the same rotation items, then (D - rot)/EPT pass-through items (pool only)
//   V heads:  D/EPT copy items (pool only)
template <typename In, int EPT>
__global__ void __launch_bounds__(256) rope_append_kernel(const RopeAppendParams p) {
  pdl_wait();
  pdl_launch_dependents();
  const int half = p.rot_dim / 2;
  const int rot_items = (int)p.d_rot.d;
  const int pass_items = (p.head_dim - p.rot_dim) / EPT;
  const int copy_items = (int)p.d_copy.d;
  const bool append = p.key_cache != nullptr;
  const int q_items = p.q ? p.n_q_heads * rot_items : 0;
  const int per_token = (int)p.d_token.d;
  const uint32_t total = (uint32_t)(p.num_tokens * per_token);   // < 2^31: the host cuts larger calls
  constexpr int ES = (int)sizeof(In);
  for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
    const uint32_t tl = p.d_token.div(idx);
    int r = (int)(idx - tl * per_token);
    const int64_t t = p.token_base + tl;

    // destination in the pool (K and V items only)
    char* pool_row = nullptr;   // start of the (slot, head 0) row in the K or V pool
    int64_t slot = -1;
    const bool is_q = r < q_items;
    if (!is_q && append) {
      slot = p.slots[t];
      if (slot >= p.n_slots_total) {
        if (r == q_items) report(KB200_STATUS_BAD_SLOT, (int)slot, KID_ROPE_APPEND);
        slot = -1;
      }
    }
    // page and offset of the slot (slots of one call fit 31 bits whenever the pool does)
    auto pool_base = [&](char* cache, int h) {
      int64_t page;
      int off;
      if (p.n_slots_total < (1ll << 31)) {
        const uint32_t pg = p.d_page.div((uint32_t)slot);
        page = pg;
        off = (int)((uint32_t)slot - pg * p.d_page.d);
      } else {
        page = slot / p.page_size;
        off = (int)(slot - page * p.page_size);
      }
      return cache + page * p.page_stride_b + off * p.token_stride_b + h * p.head_stride_b;
    };

    if (r < q_items + p.n_kv_heads * rot_items) {
      // ---- rotation item (Q or K)
      int h, c;
      char* row;
      bool is_k = false;
      if (is_q) {
        h = (int)p.d_rot.div((uint32_t)r);
        c = r - h * rot_items;
        row = p.q + t * p.q_token_stride_b + (int64_t)h * p.head_dim * ES;
      } else {
        r -= q_items;
        h = (int)p.d_rot.div((uint32_t)r);
        c = r - h * rot_items;
        row = p.k + t * p.k_token_stride_b + (int64_t)h * p.head_dim * ES;
        is_k = true;
      }
      int64_t pos = p.positions_is_i64 ? reinterpret_cast<const int64_t*>(p.positions)[t]
                                       : (int64_t)reinterpret_cast<const int32_t*>(p.positions)[t];
      if (pos < 0 || pos >= p.max_pos) {
        if (c == 0 && h == 0) report(KB200_STATUS_BAD_POSITION, (int)pos, KID_ROPE_APPEND);
        pos = pos < 0 ? 0 : p.max_pos - 1;
      }
      const float* cs = p.cos_sin + pos * p.cos_sin_row_stride + c * EPT;
      Vec<In, EPT> x1, x2;
      load_vec<In, EPT>(x1, row + (int64_t)c * EPT * ES);
      load_vec<In, EPT>(x2, row + (int64_t)(half + c * EPT) * ES);
      float co[EPT], si[EPT];
      if constexpr (EPT % 4 == 0) {
        if (p.cs_vec) {
#pragma unroll
          for (int i = 0; i < EPT / 4; ++i) {
            *reinterpret_cast<float4*>(&co[4 * i]) = *reinterpret_cast<const float4*>(cs + 4 * i);
            *reinterpret_cast<float4*>(&si[4 * i]) = *reinterpret_cast<const float4*>(cs + half + 4 * i);
          }
        } else {
#pragma unroll
          for (int i = 0; i < EPT; ++i) { co[i] = cs[i]; si[i] = cs[half + i]; }
        }
      } else {
#pragma unroll
        for (int i = 0; i < EPT; ++i) { co[i] = cs[i]; si[i] = cs[half + i]; }
      }
#pragma unroll
      for (int i = 0; i < EPT; ++i) {
        const float a = to_float(x1.e[i]), b = to_float(x2.e[i]);
        const float y1 = __fsub_rn(__fmul_rn(a, co[i]), __fmul_rn(b, si[i]));
        const float y2 = __fadd_rn(__fmul_rn(b, co[i]), __fmul_rn(a, si[i]));
        x1.e[i] = from_float<In>(y1);
        x2.e[i] = from_float<In>(y2);
      }
      if (is_q || p.write_k) {
        store_vec<In, EPT>(row + (int64_t)c * EPT * ES, x1);
        store_vec<In, EPT>(row + (int64_t)(half + c * EPT) * ES, x2);
      }
      if (is_k && slot >= 0) {
        pool_row = pool_base(p.key_cache, h);
        if (p.quant) {
          const float s = p.k_scale[p.n_scales == 1 ? 0 : h];
          store_quant<In, EPT>(pool_row + c * EPT, x1, s);
          store_quant<In, EPT>(pool_row + half + c * EPT, x2, s);
        } else {
          store_vec<In, EPT>(pool_row + (int64_t)c * EPT * ES, x1);
          store_vec<In, EPT>(pool_row + (int64_t)(half + c * EPT) * ES, x2);
        }
      }
      continue;
    }

    // ---- pool-only items: the unrotated tail of K, all of V
    if (slot < 0) continue;
    r -= q_items + p.n_kv_heads * rot_items;
    const bool is_v = r >= p.n_kv_heads * pass_items;
    int h, e0;
    const char* src;
    if (!is_v) {
      h = (int)p.d_pass.div((uint32_t)r);
      e0 = p.rot_dim + (r - h * pass_items) * EPT;
      src = p.k + t * p.k_token_stride_b + ((int64_t)h * p.head_dim + e0) * ES;
    } else {
      r -= p.n_kv_heads * pass_items;
      h = (int)p.d_copy.div((uint32_t)r);
      e0 = (r - h * copy_items) * EPT;
      src = p.v + t * p.v_token_stride_b + ((int64_t)h * p.head_dim + e0) * ES;
    }
    pool_row = pool_base(is_v ? p.value_cache : p.key_cache, h);
    Vec<In, EPT> x;
    load_vec<In, EPT>(x, src);
    if (p.quant) {
      const float* sp = is_v ? p.v_scale : p.k_scale;
      store_quant<In, EPT>(pool_row + e0, x, sp[p.n_scales == 1 ? 0 : h]);
    } else {
      store_vec<In, EPT>(pool_row + (int64_t)e0 * ES, x);
    }
  }
}

struct RopeAppendArgs {
  void* q; void* k; const void* v;
  int64_t q_token_stride, k_token_stride, v_token_stride;  // elements
  int64_t num_tokens;
  int32_t n_q_heads, n_kv_heads, head_dim, rot_dim;
  const void* positions; int32_t positions_is_i64;
  const float* cos_sin_cache; int64_t max_pos, cos_sin_row_stride;
  void* key_cache; void* value_cache;
  int64_t cache_page_stride, cache_token_stride, cache_head_stride;
  const int64_t* slot_mapping;
  int64_t n_pages; int32_t page_size;
  int32_t in_dtype, cache_dtype;
  const float* k_scale; const float* v_scale; int32_t n_scales;
  int32_t write_k;
};

// Blocks of `threads` threads that fit on the current device at once (all SMs).
template <typename K>
inline int resident_blocks(K kernel, int threads) {
  int per_sm = 0, dev = 0, sms = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0) != cudaSuccess || per_sm < 1) per_sm = 4;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
    sms = 148;
  return per_sm * sms;
}

template <typename In>
inline int launch_rope_append_typed(RopeAppendParams p, bool vec, int64_t per_token, cudaStream_t stream) {
  const int threads = 256;
  // the kernel indexes its items with 32 bits: calls above 2^31 items are cut into several launches
  const int64_t max_tokens = ((1ll << 31) - 1) / per_token;
  const int64_t all_tokens = p.num_tokens;
  for (int64_t t0 = 0; t0 < all_tokens; t0 += max_tokens) {
    p.token_base = t0;
    p.num_tokens = all_tokens - t0 < max_tokens ? all_tokens - t0 : max_tokens;
    const int64_t items = p.num_tokens * per_token;
    int64_t b = (items + threads - 1) / threads;
    // grid-stride loop: at most one resident wave, so that no SM is left with a part-filled last wave
    static const int resident8 = resident_blocks(rope_append_kernel<In, 8>, threads);
    static const int resident1 = resident_blocks(rope_append_kernel<In, 1>, threads);
    const int64_t cap = vec ? resident8 : resident1;
    const int blocks = (int)(b < 1 ? 1 : (b > cap ? cap : b));
    if (vec) KB200_CUDA_OK(launch_kernel(rope_append_kernel<In, 8>, dim3(blocks), dim3(threads), 0, stream, p));
    else KB200_CUDA_OK(launch_kernel(rope_append_kernel<In, 1>, dim3(blocks), dim3(threads), 0, stream, p));
  }
  return KB200_OK;
}

inline int launch_rope_append(const RopeAppendArgs& a, cudaStream_t stream) {
  KB200_REQUIRE(a.num_tokens >= 0, "num_tokens must be non-negative");
  if (a.num_tokens == 0) return KB200_OK;
  KB200_REQUIRE(a.k != nullptr && a.positions != nullptr && a.cos_sin_cache != nullptr, "null pointer argument");
  KB200_REQUIRE(a.n_kv_heads > 0 && a.head_dim > 0 && a.n_q_heads >= 0, "head counts and head_dim must be positive");
  KB200_REQUIRE(a.q != nullptr || a.n_q_heads == 0, "q is null but n_q_heads > 0");
  KB200_REQUIRE(a.rot_dim > 0 && a.rot_dim % 2 == 0 && a.rot_dim <= a.head_dim,
                "rot_dim must be even and in (0, head_dim]");
  KB200_REQUIRE(a.max_pos > 0 && a.cos_sin_row_stride >= a.rot_dim, "cos/sin cache geometry is inconsistent");
  const bool append = a.key_cache != nullptr;
  const int in_sz = dtype_size(a.in_dtype);
  KB200_REQUIRE(in_sz && a.in_dtype != KB200_DTYPE_E4M3, "rows must be F32, F16 or BF16");
  int c_sz = in_sz;
  bool quant = false;
  if (append) {
    KB200_REQUIRE(a.v && a.value_cache && a.slot_mapping, "append needs v, value_cache and slot_mapping");
    KB200_REQUIRE(a.page_size > 0 && a.n_pages > 0, "page_size and n_pages must be positive");
    c_sz = dtype_size(a.cache_dtype);
    KB200_REQUIRE(c_sz, "unknown cache dtype");
    quant = a.cache_dtype == KB200_DTYPE_E4M3;
    if (quant) {
      KB200_REQUIRE(a.k_scale && a.v_scale, "FP8 append requires k_scale and v_scale");
      KB200_REQUIRE(a.n_scales == 1 || a.n_scales == a.n_kv_heads, "n_scales must be 1 or n_kv_heads");
    } else {
      KB200_REQUIRE(a.in_dtype == a.cache_dtype, "input dtype must equal cache dtype (or cache must be E4M3)");
    }
  }
  RopeAppendParams p;
  p.q = a.n_q_heads > 0 ? static_cast<char*>(a.q) : nullptr;
  p.k = static_cast<char*>(a.k);
  p.v = static_cast<const char*>(a.v);
  p.positions = a.positions;
  p.cos_sin = a.cos_sin_cache;
  p.key_cache = static_cast<char*>(a.key_cache);
  p.value_cache = static_cast<char*>(a.value_cache);
  p.slots = a.slot_mapping;
  p.k_scale = a.k_scale;
  p.v_scale = a.v_scale;
  p.q_token_stride_b = a.q_token_stride * in_sz;
  p.k_token_stride_b = a.k_token_stride * in_sz;
  p.v_token_stride_b = a.v_token_stride * in_sz;
  p.page_stride_b = a.cache_page_stride * c_sz;
  p.token_stride_b = a.cache_token_stride * c_sz;
  p.head_stride_b = a.cache_head_stride * c_sz;
  p.cos_sin_row_stride = a.cos_sin_row_stride;
  p.max_pos = a.max_pos;
  p.num_tokens = a.num_tokens;
  p.n_slots_total = append ? a.n_pages * a.page_size : 0;
  p.n_q_heads = a.n_q_heads;
  p.n_kv_heads = a.n_kv_heads;
  p.head_dim = a.head_dim;
  p.rot_dim = a.rot_dim;
  p.page_size = append ? a.page_size : 1;
  p.n_scales = a.n_scales;
  p.positions_is_i64 = a.positions_is_i64;
  p.write_k = a.write_k || !append;
  p.quant = quant;

  // 8 elements per thread when every access is 16-byte aligned (8 bytes for e4m3 stores)
  const int half = a.rot_dim / 2;
  bool vec = in_sz == 2 && half % 8 == 0 && (a.head_dim - a.rot_dim) % 8 == 0 && a.head_dim % 8 == 0 &&
             aligned16(a.k) && (p.q == nullptr || aligned16(a.q)) && p.k_token_stride_b % 16 == 0 &&
             (p.q == nullptr || p.q_token_stride_b % 16 == 0);
  if (append)
    vec = vec && aligned16(a.v) && p.v_token_stride_b % 16 == 0 && aligned16(a.key_cache) &&
          aligned16(a.value_cache) && p.page_stride_b % 16 == 0 && p.token_stride_b % 16 == 0 &&
          p.head_stride_b % 16 == 0;
  const int ept = vec ? 8 : 1;
  const int64_t per_token = (int64_t)(p.q ? a.n_q_heads : 0) * (half / ept) +
                            (int64_t)a.n_kv_heads * (half / ept + (append ? (a.head_dim - a.rot_dim) / ept : 0)) +
                            (append ? (int64_t)a.n_kv_heads * (a.head_dim / ept) : 0);
  KB200_REQUIRE(per_token > 0 && per_token < (1ll << 24), "row too large");
  p.d_token = FastDiv::make((uint32_t)per_token);
  p.d_rot = FastDiv::make((uint32_t)(half / ept));
  p.d_pass = FastDiv::make((uint32_t)((a.head_dim - a.rot_dim) / ept));
  p.d_copy = FastDiv::make((uint32_t)(a.head_dim / ept));
  p.d_page = FastDiv::make((uint32_t)p.page_size);
  p.cs_vec = aligned16(a.cos_sin_cache) && a.cos_sin_row_stride % 4 == 0 && half % 4 == 0;
  p.token_base = 0;
  if (a.in_dtype == KB200_DTYPE_BF16) return launch_rope_append_typed<__nv_bfloat16>(p, vec, per_token, stream);
  if (a.in_dtype == KB200_DTYPE_F16) return launch_rope_append_typed<__half>(p, vec, per_token, stream);
  return launch_rope_append_typed<float>(p, false, per_token, stream);
}

// ---------------------------------------------------------------------------
// Per-step decode metadata in one launch: for active row r with the last new
// token at position input_pos[r] and n_new new tokens,
//   out_seqused_k[r]      = input_pos[r] + 1
//   out_page_table[r, :ceil(seqused/P)] = page_table[batch_idx[r], ...]  (tail untouched)
//   out_positions[r, j]   = input_pos[r] - (n_new - 1) + j
//   out_slots[r, j]       = page_table[batch_idx[r], pos // P] * P + pos % P
// i.e. build_paged_kv_metadata followed by build_slot_mapping.
// ---------------------------------------------------------------------------
template <typename BI>
__global__ void __launch_bounds__(128)
decode_step_metadata_kernel(const int32_t* __restrict__ page_table, int64_t pt_row_stride, int64_t pt_rows,
                            int64_t pt_cols, const BI* __restrict__ batch_idx,
                            const int32_t* __restrict__ input_pos, int32_t* __restrict__ out_page_table,
                            int64_t out_row_stride, int64_t out_cols, int32_t* __restrict__ out_seqused_k,
                            int64_t* __restrict__ out_slots, int64_t* __restrict__ out_positions, int n_new,
                            int page_size) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t r = blockIdx.x;
  const int64_t b = (int64_t)batch_idx[r];
  const int last = input_pos[r];
  const int used = last + 1;
  if (threadIdx.x == 0) out_seqused_k[r] = used;
  const bool bad_row = b < 0 || b >= pt_rows;
  if (bad_row && threadIdx.x == 0) report(KB200_STATUS_BAD_ROW, (int)b, KID_METADATA);
  const int32_t* src = page_table + (bad_row ? 0 : b) * pt_row_stride;
  for (int j = threadIdx.x; j < n_new; j += blockDim.x) {
    const int64_t pos = (int64_t)last - (n_new - 1) + j;
    if (out_positions) out_positions[r * n_new + j] = pos;
    int64_t blk = pos / page_size;
    int64_t off = pos - blk * page_size;
    if (off < 0) { off += page_size; blk -= 1; }
    int64_t slot = -1;
    if (!bad_row && blk >= 0 && blk < pt_cols) slot = (int64_t)src[blk] * page_size + off;
    else if (!bad_row) report(KB200_STATUS_BAD_ROW, (int)b, KID_METADATA);
    out_slots[r * n_new + j] = slot;
  }
  if (bad_row) return;
  int64_t n = used > 0 ? (used + page_size - 1) / page_size : 0;
  if (n > pt_cols) n = pt_cols;
  if (n > out_cols) n = out_cols;
  int32_t* dst = out_page_table + r * out_row_stride;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
}

inline int launch_decode_step_metadata(const int32_t* page_table, int64_t pt_row_stride, int64_t pt_rows,
                                       int64_t pt_cols, const void* batch_idx, int32_t bi64,
                                       const int32_t* input_pos, int32_t* out_page_table,
                                       int64_t out_row_stride, int64_t out_cols, int32_t* out_seqused_k,
                                       int64_t* out_slots, int64_t* out_positions, int64_t batch, int32_t n_new,
                                       int32_t page_size, cudaStream_t stream) {
  if (batch == 0) return KB200_OK;
  KB200_REQUIRE(batch > 0 && batch <= 0x7fffffff, "batch out of range");
  KB200_REQUIRE(page_table && batch_idx && input_pos && out_page_table && out_seqused_k && out_slots,
                "null pointer argument");
  KB200_REQUIRE(page_size > 0 && n_new > 0, "page_size and n_new must be positive");
  if (bi64)
    KB200_CUDA_OK(launch_kernel(decode_step_metadata_kernel<int64_t>, dim3((unsigned)batch), dim3(128), 0, stream,
                                page_table, pt_row_stride, pt_rows, pt_cols, static_cast<const int64_t*>(batch_idx),
                                input_pos, out_page_table, out_row_stride, out_cols, out_seqused_k, out_slots,
                                out_positions, (int)n_new, (int)page_size));
  else
    KB200_CUDA_OK(launch_kernel(decode_step_metadata_kernel<int32_t>, dim3((unsigned)batch), dim3(128), 0, stream,
                                page_table, pt_row_stride, pt_rows, pt_cols, static_cast<const int32_t*>(batch_idx),
                                input_pos, out_page_table, out_row_stride, out_cols, out_seqused_k, out_slots,
                                out_positions, (int)n_new, (int)page_size));
  return KB200_OK;
}

// ---------------------------------------------------------------------------
// Block-bidirectional mask: out[b, j] = last position of the run of equal, non-negative block
// ids that contains j (j itself for text, id < 0).  One block of threads per sequence; every
// thread walks forward from its position to the end of its run (runs are image blocks, a few
// hundred positions, and the walk is tiny next to the prefill it serves).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
block_visibility_kernel(const int32_t* __restrict__ ids, int64_t ids_rs, int64_t seqlen, int32_t* __restrict__ out,
                        int64_t out_rs) {
  pdl_wait();
  pdl_launch_dependents();
  const int32_t* row = ids + (int64_t)blockIdx.x * ids_rs;
  int32_t* dst = out + (int64_t)blockIdx.x * out_rs;
  for (int64_t j = threadIdx.x; j < seqlen; j += blockDim.x) {
    const int32_t id = row[j];
    int64_t e = j;
    if (id >= 0)
      while (e + 1 < seqlen && row[e + 1] == id) ++e;
    dst[j] = (int32_t)e;
  }
}

inline int launch_block_visibility(const int32_t* ids, int64_t ids_rs, int64_t batch, int64_t seqlen, int32_t* out,
                                   int64_t out_rs, cudaStream_t stream) {
  if (batch == 0 || seqlen == 0) return KB200_OK;
  KB200_REQUIRE(batch > 0 && seqlen > 0 && batch <= 0x7fffffff && seqlen <= 0x7fffffff, "batch / seqlen out of range");
  KB200_REQUIRE(ids && out, "null pointer argument");
  KB200_CUDA_OK(launch_kernel(block_visibility_kernel, dim3((unsigned)batch), dim3(256), 0, stream, ids, ids_rs, seqlen,
                              out, out_rs));
  return KB200_OK;
}

}  // namespace kb200
