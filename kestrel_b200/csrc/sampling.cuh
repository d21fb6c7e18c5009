// Token sampling from the logits of a decode step: temperature, top-p nucleus, one draw per row.
// The step after the decoder stack (kestrel_kernels.sampling.sample_step_from_logits as called at
// kestrel/scheduler/scheduler.py:2986-2991 and kestrel/scheduler/spatial.py:105-123).
//
// One CTA of 1024 threads per row; the row (vocab x 2 or 4 bytes, at most a few hundred KB) comes
// from HBM once and from L2 on the later passes.  HBM-bound: batch x vocab x sizeof(logit) bytes.
//
//   pass 1  row maximum and its first index            -> greedy rows are done here
//   pass 2  every thread sums exp((x - max) / T) over its contiguous slice of the vocabulary; a block scan
//           gives Z and, with top_p >= 1, already the slice that holds u * Z
//   pass 3  (top_p < 1) threshold tau of the nucleus {p >= tau}: radix select over the bit pattern of p,
//           three rounds of 11 + 11 + 10 bits, each a histogram of probability MASS per digit; then the
//           slice sums again, restricted to the nucleus
//   last    the owner of the slice that holds u * mass walks it to the token
//
// Everything that decides the outcome is summed in 64-bit fixed point (p * 2^40, exact integer adds in any
// order), so the result does not depend on the order in which threads or atomics arrive: the same logits
// and the same uniform give the same token on every run.
#pragma once

#include <type_traits>

#include "common.cuh"

namespace kb200 {

struct SampleParams {
  const char* logits;
  int64_t row_stride;   // elements
  int64_t vocab;
  const float* temps;
  const float* top_ps;
  const float* uniforms;
  int64_t* out_ids;
  float* logprobs;      // or nullptr
  int batch;
  int vec_ok;           // rows are 16-byte aligned and vocab is a multiple of the vector width
};

constexpr int kSampleThreads = 1024;
constexpr float kSamplingEps = 1e-6f;                 // temperatures at or below this are greedy (scheduler.py:55)
constexpr float kFix = 1099511627776.f;               // 2^40

template <typename LT> struct SampleVec;
template <> struct SampleVec<float> { static constexpr int N = 4; };
template <> struct SampleVec<__half> { static constexpr int N = 8; };
template <> struct SampleVec<__nv_bfloat16> { static constexpr int N = 8; };

template <typename LT>
__device__ __forceinline__ float logit_to_float(LT v) {
  if constexpr (std::is_same<LT, float>::value) return v;
  else if constexpr (std::is_same<LT, __half>::value) return __half2float(v);
  else return __bfloat162float(v);
}

// f(index, value) for every element of [lo, hi) that this thread owns when `nthreads` threads share the
// range: vectors of 16 bytes in a thread-strided pattern (coalesced), scalar loads for unaligned rows
template <typename LT, typename F>
__device__ __forceinline__ void for_strided(const LT* row, int64_t lo, int64_t hi, int tid, int nthreads, bool vec_ok, F&& f) {
  constexpr int N = SampleVec<LT>::N;
  if (vec_ok) {
    for (int64_t i = lo + (int64_t)tid * N; i < hi; i += (int64_t)nthreads * N) {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(row + i));
      const LT* e = reinterpret_cast<const LT*>(&raw);
#pragma unroll
      for (int k = 0; k < N; ++k) f(i + k, logit_to_float<LT>(e[k]));
    }
  } else {
    for (int64_t i = lo + tid; i < hi; i += nthreads) f(i, logit_to_float<LT>(__ldg(row + i)));
  }
}

__device__ __forceinline__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* scratch) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  __syncthreads();   // scratch may still be read from the previous use
  if (lane == 0) scratch[wid] = v;
  __syncthreads();
  unsigned long long t = lane < (kSampleThreads >> 5) ? scratch[lane] : 0ull;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) t += __shfl_xor_sync(0xffffffffu, t, d);
  return t;   // the same on every thread
}

// exclusive prefix sum over the threads of the block (thread order), and the block total
__device__ __forceinline__ unsigned long long block_exclusive_scan_u64(unsigned long long v, unsigned long long* scratch,
                                                                       unsigned long long& total) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  unsigned long long inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const unsigned long long u = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += u;
  }
  __syncthreads();
  if (lane == 31) scratch[wid] = inc;
  __syncthreads();
  unsigned long long w = lane < (kSampleThreads >> 5) ? scratch[lane] : 0ull, winc = w;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const unsigned long long u = __shfl_up_sync(0xffffffffu, winc, d);
    if (lane >= d) winc += u;
  }
  total = __shfl_sync(0xffffffffu, winc, 31);
  const unsigned long long warp_off = __shfl_sync(0xffffffffu, winc - w, wid);
  return warp_off + inc - v;
}

template <typename LT>
__global__ void __launch_bounds__(kSampleThreads, 1) sample_kernel(const SampleParams p) {
  // mass per digit as two 32-bit halves: native 32-bit shared-memory atomics, the carry propagated by hand
  __shared__ unsigned int hist_lo[2048];
  __shared__ unsigned int hist_hi[2048];
  __shared__ unsigned long long scratch[32];
  __shared__ float red_v[32];
  __shared__ long long red_i[32];
  __shared__ unsigned long long sel_above;
  __shared__ unsigned int sel_digit;
  __shared__ long long found_id;
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const LT* row = reinterpret_cast<const LT*>(p.logits) + (int64_t)b * p.row_stride;
  const int64_t V = p.vocab;
  const bool vec = p.vec_ok != 0;
  const float temp = fmaxf(p.temps[b], 0.f);
  const float top_p = p.top_ps[b];

  // ---- pass 1: maximum and its first index
  float best = -INFINITY;
  long long best_i = 0x7fffffffffffffffll;
  for_strided<LT>(row, 0, V, tid, kSampleThreads, vec, [&](int64_t i, float x) {
    if (x > best || (x == best && i < best_i)) { best = x; best_i = i; }
  });
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, d);
    const long long oi = __shfl_xor_sync(0xffffffffu, best_i, d);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if (lane == 0) { red_v[wid] = best; red_i[wid] = best_i; }
  __syncthreads();
  best = red_v[lane];
  best_i = red_i[lane];
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, d);
    const long long oi = __shfl_xor_sync(0xffffffffu, best_i, d);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if (best_i >= V) best_i = 0;   // a row of NaNs: out of contract, stay in range
  // greedy: temperature at or below the threshold, or nothing finite to normalise
  if (temp <= kSamplingEps || !(best > -INFINITY) || !(best < INFINITY)) {
    if (tid == 0) {
      p.out_ids[b] = best_i;
      if (p.logprobs) p.logprobs[b] = 0.f;
    }
    return;
  }
  const float c = 1.4426950408889634f / temp;   // exp(x / T) = 2^(x * c)
  auto prob = [&](float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"((x - best) * c)); return y; };
  auto fixed = [&](float pr) { return (unsigned long long)__float2ull_rz(pr * kFix); };

  // ---- pass 2: slice sums over the whole vocabulary, Z
  constexpr int N = SampleVec<LT>::N;
  int64_t chunk = (V + kSampleThreads - 1) / kSampleThreads;
  chunk = (chunk + N - 1) / N * N;
  const int64_t lo = min((int64_t)tid * chunk, V), hi = min(lo + chunk, V);
  unsigned long long local = 0;
  for_strided<LT>(row, lo, hi, 0, 1, vec, [&](int64_t, float x) { local += fixed(prob(x)); });
  unsigned long long Z, pre = block_exclusive_scan_u64(local, scratch, Z);

  // ---- pass 3: nucleus threshold (bit pattern of p), then the slice sums restricted to the nucleus
  unsigned int tau = 0;
  unsigned long long total = Z;
  if (top_p < 1.f) {
    unsigned long long target = (unsigned long long)((double)fmaxf(top_p, 0.f) * (double)Z);
    if (target < 1) target = 1;
    unsigned long long above = 0;   // mass of the elements whose bits exceed every candidate left
    unsigned int prefix = 0;
    int shift = 32;
#pragma unroll 1
    for (int round = 0; round < 3; ++round) {
      const int width = round < 2 ? 11 : 10;
      shift -= width;
      for (int i = tid; i < 2048; i += kSampleThreads) { hist_lo[i] = 0u; hist_hi[i] = 0u; }
      __syncthreads();
      const unsigned int dmask = (1u << width) - 1u;
      const int hi_shift = shift + width;
      for_strided<LT>(row, 0, V, tid, kSampleThreads, vec, [&](int64_t, float x) {
        const float pr = prob(x);
        const unsigned int bits = __float_as_uint(pr);
        if (hi_shift >= 32 || (bits >> hi_shift) == prefix) {
          const unsigned long long q = fixed(pr);
          const unsigned int d = (bits >> shift) & dmask, ql = (unsigned int)q, qh = (unsigned int)(q >> 32);
          if (q) {
            const unsigned int old = atomicAdd(&hist_lo[d], ql);
            const unsigned int carry = (old + ql < old) ? 1u : 0u;
            if (qh + carry) atomicAdd(&hist_hi[d], qh + carry);
          }
        }
      });
      __syncthreads();
      // suffix sums from the top digit down; thread t owns digits 2t and 2t + 1
      const unsigned long long h0 = ((unsigned long long)hist_hi[2 * tid] << 32) + hist_lo[2 * tid];
      const unsigned long long h1 = ((unsigned long long)hist_hi[2 * tid + 1] << 32) + hist_lo[2 * tid + 1];
      unsigned long long tot, excl = block_exclusive_scan_u64(h0 + h1, scratch, tot);
      const unsigned long long s_hi1 = tot - excl - (h0 + h1);     // mass of digits above 2t + 1
      const unsigned long long s1 = s_hi1 + h1, s0 = s1 + h0;      // mass of digits >= 2t + 1, >= 2t
      if (above + s1 >= target && above + s_hi1 < target) { sel_digit = 2 * tid + 1; sel_above = above + s_hi1; }
      else if (above + s0 >= target && above + s1 < target) { sel_digit = 2 * tid; sel_above = above + s1; }
      __syncthreads();
      prefix = (prefix << width) | sel_digit;
      above = sel_above;
      __syncthreads();
    }
    tau = prefix;
    local = 0;
    for_strided<LT>(row, lo, hi, 0, 1, vec, [&](int64_t, float x) {
      const float pr = prob(x);
      if (__float_as_uint(pr) >= tau) local += fixed(pr);
    });
    pre = block_exclusive_scan_u64(local, scratch, total);
  }

  // ---- the slice of the vocabulary that holds u * mass, then the token inside it
  unsigned long long want = (unsigned long long)((double)p.uniforms[b] * (double)total);
  if (total > 0 && want >= total) want = total - 1;
  if (tid == 0) found_id = best_i;   // (only kept if no slice claims the target: an empty nucleus cannot happen)
  __syncthreads();
  if (local > 0 && pre <= want && want < pre + local) {
    unsigned long long cum = pre;
    long long id = -1;
    for_strided<LT>(row, lo, hi, 0, 1, vec, [&](int64_t i, float x) {
      const float pr = prob(x);
      if (id < 0 && __float_as_uint(pr) >= tau) {
        cum += fixed(pr);
        if (cum > want) id = i;
      }
    });
    if (id >= 0) found_id = id;
  }
  __syncthreads();
  if (tid == 0) {
    const long long id = found_id;
    p.out_ids[b] = id;
    if (p.logprobs) {
      const float x = logit_to_float<LT>(row[id]);
      p.logprobs[b] = (x - best) * c * 0.6931471805599453f - logf((float)((double)Z / (double)kFix));
    }
  }
}

inline int launch_sample_step(const void* logits, int logits_dtype, int64_t batch, int64_t vocab, int64_t row_stride,
                              const float* temps, const float* top_ps, const float* uniforms, int64_t* out_ids,
                              float* logprobs, cudaStream_t stream) {
  KB200_REQUIRE(batch >= 0 && vocab > 0, "batch must be non-negative and vocab positive");
  if (batch == 0) return KB200_OK;
  KB200_REQUIRE(batch <= 0x7fffffff, "batch out of range");
  KB200_REQUIRE(vocab <= (1ll << 20), "vocab above 2^20 would overflow the fixed-point mass");
  KB200_REQUIRE(logits && temps && top_ps && uniforms && out_ids, "null pointer argument");
  KB200_REQUIRE(row_stride >= vocab, "row_stride is smaller than the vocabulary");
  const int es = dtype_size(logits_dtype);
  KB200_REQUIRE(es != 0 && logits_dtype != KB200_DTYPE_E4M3, "logits must be F32, F16 or BF16");
  SampleParams p;
  p.logits = static_cast<const char*>(logits);
  p.row_stride = row_stride;
  p.vocab = vocab;
  p.temps = temps;
  p.top_ps = top_ps;
  p.uniforms = uniforms;
  p.out_ids = out_ids;
  p.logprobs = logprobs;
  p.batch = (int)batch;
  const int vecn = 16 / es;
  p.vec_ok = ((reinterpret_cast<uintptr_t>(logits) & 15) == 0 && (row_stride * es) % 16 == 0 && vocab % vecn == 0) ? 1 : 0;
  const dim3 grid((unsigned)batch), block(kSampleThreads);
  if (logits_dtype == KB200_DTYPE_F32) KB200_CUDA_OK(launch_kernel(sample_kernel<float>, grid, block, 0, stream, p));
  else if (logits_dtype == KB200_DTYPE_F16) KB200_CUDA_OK(launch_kernel(sample_kernel<__half>, grid, block, 0, stream, p));
  else KB200_CUDA_OK(launch_kernel(sample_kernel<__nv_bfloat16>, grid, block, 0, stream, p));
  return KB200_OK;
}

}  // namespace kb200
