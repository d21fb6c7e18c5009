// Paged split-KV decode attention for sm_100a.
//
// Work decomposition
//   A *segment* is one (sequence b, KV head h, 16-row query block mb): the rows
//   are the GQA group's query heads times the (few) query positions of the
//   sequence, row r = j * group + g.  A segment's keys are cut into *tiles* of
//   TILE_N tokens.  All tiles of all segments form one flat index space
//   [0, T); worker w (one warp) owns the contiguous range
//   [w*T/W, (w+1)*T/W), so every warp streams the same number of tiles (+-1)
//   whatever the mix of context lengths.  A warp keeps the running
//   (max, sum, O) of its current segment in registers; a segment that lies
//   inside one warp's range is normalised and written straight to `out`, a
//   segment cut by a range boundary leaves one partial per warp in scratch
//   memory and a small merge kernel combines them.
//
// Data movement
//   The pool view [n_pages, P, H_kv, D] is described to the TMA unit once per
//   pool as a 4-D tensor map; a (page, head) tile of K or V is one
//   cp.async.bulk.tensor box of P rows x 128 bytes (a 256-byte row: two boxes,
//   or one box of a 5-D map that splits the row into two 128-byte halves),
//   landing in 128-byte-swizzled shared memory so that ldmatrix is
//   bank-conflict free.  Each warp owns a ring of NS stages (two) and
//   refills a stage as soon as it has read it, so one tile per warp is always
//   in flight behind the one being computed.  Page indices are read one tile
//   ahead of the copy that needs them.  No multicast, no cluster.
//
// Math
//   S = Q K^T and O += P V on mma.sync m16n8k16 (bf16 or f16 operands, fp32
//   accumulate); FP8 e4m3 K/V are widened to f16 in registers (exact) and the
//   per-head scales are folded into the softmax scale and the final
//   normalisation.  Softmax is the usual online form in fp32, base 2.
#pragma once

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <type_traits>
#include <mutex>
#include <unordered_map>
#include <string>

#include "common.cuh"

namespace kb200 {

constexpr int kAttnMaxWarps = 12;
constexpr int kRowsPerSeg = 16;   // query rows per segment, general kernel (also the stride of scratch slots)
constexpr int kDecodeRows = 8;    // query rows per segment, decode kernel
// NW worker warps per CTA, each with a ring of NS stages of kAttnStageBytes(NW) (K tile then V tile).
// Stages are 8 KB (two of them per warp: one being read, one in flight).
// More bytes in flight do not help: 8 warps x 3 stages (128 KB behind the tiles being read) measured
// 3-5 % slower than x 2 (64 KB) once the kernel is HBM-bound; the requests queue up in the memory system and
// the SMs' shares of the bandwidth grow apart.
constexpr int kAttnStageBytes(int) { return 8 * 1024; }

template <int KVB, int HD, int NW, int NS>
struct AttnTile {
  static constexpr int STAGES = NS;
  static constexpr int ROW_BYTES = HD * KVB;                      // bytes of one token row of one head
  static constexpr int RB = ROW_BYTES > 128 ? 128 : ROW_BYTES;    // swizzled row width in smem
  static constexpr int NH = ROW_BYTES / RB;                       // 128-byte halves per row
  static constexpr int STAGE_TARGET = kAttnStageBytes(NW);
  static constexpr int TILE_RAW = STAGE_TARGET / (2 * ROW_BYTES);
  static constexpr int TILE_N = TILE_RAW > 64 ? 64 : TILE_RAW;
  static constexpr int KV_TILE_BYTES = TILE_N * ROW_BYTES;
  static constexpr int STAGE_BYTES = 2 * KV_TILE_BYTES;           // K then V
  static constexpr int PLAN_OFF = (NW * NS * STAGE_BYTES + NW * NS * 8 + 15) & ~15;   // in-kernel plan, after the barriers
  static constexpr int SMEM_BYTES = PLAN_OFF + 1024;                                  // + plan_smem_bytes(batch) at launch
};

struct AttnParams {
  const char* q;
  char* out;
  float* lse;
  int64_t q_bs, q_rs, q_hs, o_bs, o_rs, o_hs;  // element strides
  int64_t lse_bs, lse_hs;
  const int32_t* page_table;
  int64_t pt_rs;
  const int32_t* seqused_k;
  const int32_t* seqused_q;
  const int32_t* cu_seqlens_q;
  const float* ks_vec;
  const float* vs_vec;
  const int32_t* q_vis;   // per query row: last row of its sequence whose key it may see (prefill kernel only)
  int64_t q_vis_bs;
  float ks, vs, softmax_scale;
  // plan (written by attn_plan_kernel)
  long long* tile_cum;  // [B+1]
  int* seg_cum;         // [B+1]
  int* nt;              // [B] tiles per segment
  int* tile0;           // [B] first tile (sliding window)
  int* sq;              // [B] valid query rows
  int* qrow0;           // [B] first packed query row (0 in the padded layout)
  int* klen;            // [B] keys
  int* bound_rec;       // [n_workers][8]: where each worker's range starts (written by the attention kernel for the merge)
  float* part_ml;       // [slots][16][2]  (scaled max in log2 units, sum)
  float* part_o;        // [slots][16][HD] unnormalised
  int64_t n_pages;
  int batch, seqlen_q, hq, hkv, group, page_size, causal, window_left, q_is_bf16, n_workers, tile_n;
  int rows_per_seg;  // query rows per segment: 16 (general kernel), 8 (decode kernel) or 32 (32-row kernel)
  int seg_blocks;    // 16-row partial slots per (segment, worker): 2 for 32-row segments, else 1
  int uniform_nseg;  // segments per sequence when that is the same for all (padded q, no seqused_q), else 0
  // Shared-prefix passes.  k_skip: the first k_skip keys of every sequence are served by another pass
  // (page_table already points past their pages; lengths are taken relative to them).
  // fixed_klen >= 0: every sequence has exactly that many keys, the last one fixed_klen_last
  // (seqused_k is not read).  no_plan: the prefill kernel derives its segments from these and the
  // launch parameters; no plan kernel ran.
  int k_skip, fixed_klen, fixed_klen_last, no_plan;
  // 256-byte rows (16-bit K/V, head_dim 128) with pages at least a tile long: the tensor maps are
  // 5-D (64 elements, token, 128-byte half, head, page) and one box brings both halves of a page
  int merged_halves;
  // plan_in_kernel: every CTA of the attention kernel computes the plan itself into shared memory
  // (no plan launch; CTA 0 also stores it for the merge kernel); else attn_plan_kernel ran first
  int plan_in_kernel;
  long long total_q;     // rows of q (bounds the packed row ranges)
  // gather: the warps fetch their tiles 16 bytes at a time with cp.async, through these plain pointers and
  // byte strides, into the same swizzled layout as the TMA boxes would.  For pools whose (page, head) rows
  // are too short for a box (a box must fill a multiple of 128 bytes of shared memory: page size 1 with
  // 64-byte e4m3 rows, the reference's own FP8 configuration, kestrel/models/moondream/runtime.py:645-663)
  // and for pages of one or two tokens (the reference's default page size is 1, kestrel/config.py:164),
  // where a box per token costs more than it moves.
  int gather;
  // head_pack > 1: `head_pack` KV heads whose rows lie side by side in the pool are read as ONE head of
  // head_pack * real_hd elements (hkv, group and the kernel's head_dim are those of that wide head); a query
  // row is zero outside the real_hd-wide slice of its own KV head and owns only that slice of the output.
  // For pools with tiny pages and rows: page size 1 or 2 with 64- or 128-byte e4m3 rows.
  int head_pack, real_hd;
  const char* k_base;
  const char* v_base;
  long long kv_ps_b, kv_ts_b, kv_hs_b;
};

// Where the attention kernels read the plan from: shared memory (built by the CTA itself) or the
// scratch arrays a plan launch filled.  Generic pointers serve both.
struct PlanView {
  const long long* tile_cum;
  const int* seg_cum;
  const int* nt;
  const int* tile0;
  const int* sq;
  const int* qrow0;
  const int* klen;
};
struct PlanOut {
  long long* tile_cum;
  int* seg_cum;
  int* nt;
  int* tile0;
  int* sq;
  int* qrow0;
  int* klen;
};
constexpr int kPlanSmemMaxBatch = 1024;   // largest batch whose plan the attention kernels keep in shared memory
__host__ __device__ constexpr int plan_smem_bytes(int batch) {
  // tile_cum (B+1) x 8, then seg_cum (B+1) x 4 and five arrays of B ints, then the scan scratch
  return ((((batch + 1) * 8 + (batch + 1) * 4 + 5 * batch * 4 + 7) & ~7) + 448 + 15) & ~15;   // 448 >= sizeof(PlanScan)
}

// ---------------------------------------------------------------------------
// PTX helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Waits for the phase with the given parity; gives up after ~2 s of wall time
// and returns false (the caller records the failure and leaves the kernel).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t start = 0;
  for (uint32_t spins = 0;; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 63) == 63) {
      const uint64_t now = global_timer_ns();
      if (start == 0) start = now;
      else if (now - start > 2000000000ull) return false;
    }
  }
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0,
                                            int c1, int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// the barrier gets one more pending arrival, which completes when this thread's cp.async so far have landed
__device__ __forceinline__ void cp_async_mbar_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_plain(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t& r0, uint32_t& r1, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
template <bool BF16>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (BF16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}
__device__ __forceinline__ void prefetch_l1(const void* ptr) {
  asm volatile("prefetch.global.L1 [%0];" ::"l"(ptr));
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// four e4m3 codes (one 32-bit word) -> two f16x2 words (bytes 0,1 and bytes 2,3); exact
__device__ __forceinline__ void e4m3x4_to_f16x4(uint32_t x, uint32_t& lo, uint32_t& hi) {
  asm("{\n\t.reg .b16 a, b;\n\t"
      "mov.b32 {a, b}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, a;\n\t"
      "cvt.rn.f16x2.e4m3x2 %1, b;\n\t}"
      : "=r"(lo), "=r"(hi)
      : "r"(x));
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}
__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

// ---------------------------------------------------------------------------
// Plan: per-sequence tile/segment counts and their exclusive prefix sums.
// One block of NT threads; sequences are scanned NT at a time with a running carry.
// Runs either as its own one-block launch (large batches) or at the start of every CTA of the
// attention kernels, which then keep the result in shared memory.
// ---------------------------------------------------------------------------
struct PlanScan {
  long long warp_t[32];
  int warp_s[32];
  long long carry_t;
  int carry_s;
  int bad;
};
static_assert(sizeof(PlanScan) <= 448, "plan_smem_bytes reserves 448 bytes for the scan scratch");

template <int NT>
__device__ __forceinline__ void build_plan(const AttnParams& p, const PlanOut& o, PlanScan& sc, bool reporter) {
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  if (tid == 0) { sc.carry_t = 0; sc.carry_s = 0; sc.bad = 0; }
  __syncthreads();
  if (p.cu_seqlens_q) {
    // Packed rows: the row ranges must be non-negative, ascending and inside q.  Anything else would
    // make more segments than the scratch was sized for: such a call computes nothing.
    int bad = 0;
    for (int b = tid; b < p.batch; b += NT) {
      const int r0 = p.cu_seqlens_q[b], r1 = p.cu_seqlens_q[b + 1];
      if (r0 < 0 || r1 < r0 || (long long)r1 > p.total_q) bad = 1;
    }
    if (bad) sc.bad = 1;
    __syncthreads();
    if (sc.bad && reporter && tid == 0) report(KB200_STATUS_BAD_ROW, -1, KID_ATTN_PLAN);
  }
  const bool drop_all = sc.bad != 0;
  for (int base = 0; base < p.batch; base += NT) {
    const int b = base + tid;
    long long cnt_t = 0;
    int cnt_s = 0;
    if (b < p.batch) {
      int L = p.fixed_klen >= 0 ? (b == p.batch - 1 ? p.fixed_klen_last : p.fixed_klen) : p.seqused_k[b] - p.k_skip;
      const int L_rel = L;
      if (L < 0) L = 0;
      int sq, row0 = 0;
      if (p.cu_seqlens_q) {
        row0 = p.cu_seqlens_q[b];
        sq = p.cu_seqlens_q[b + 1] - row0;
      } else {
        sq = p.seqlen_q;
        if (p.seqused_q) sq = min(sq, p.seqused_q[b]);
      }
      if (sq < 0 || drop_all) sq = 0;
      // a query row that cannot see all of the skipped prefix under the causal mask (or a sequence
      // shorter than the prefix) breaks the caller's promise: results for it are undefined
      if (p.k_skip > 0 && L_rel < (p.causal ? sq : 0) && reporter) report(KB200_STATUS_BAD_PREFIX, b, KID_ATTN_PLAN);
      int t0 = 0;
      if (p.window_left >= 0) {
        int kmin = L - sq - p.window_left;
        if (kmin > 0) t0 = kmin / p.tile_n;
      }
      int ntile = (sq > 0 && L > 0) ? (L + p.tile_n - 1) / p.tile_n - t0 : 0;
      const int nmb = (p.group * sq + p.rows_per_seg - 1) / p.rows_per_seg;
      cnt_s = p.hkv * nmb;
      cnt_t = (long long)ntile * cnt_s;
      o.nt[b] = ntile;
      o.tile0[b] = t0;
      o.sq[b] = sq;
      o.qrow0[b] = row0;
      o.klen[b] = L;
    }
    // inclusive warp scans
    long long it = cnt_t;
    int is = cnt_s;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      long long ut = __shfl_up_sync(0xffffffffu, it, d);
      int us = __shfl_up_sync(0xffffffffu, is, d);
      if (lane >= d) { it += ut; is += us; }
    }
    if (lane == 31) { sc.warp_t[wid] = it; sc.warp_s[wid] = is; }
    __syncthreads();
    long long off_t = sc.carry_t;
    int off_s = sc.carry_s;
    for (int w = 0; w < wid; ++w) { off_t += sc.warp_t[w]; off_s += sc.warp_s[w]; }
    if (b < p.batch) {
      o.tile_cum[b] = off_t + it - cnt_t;
      o.seg_cum[b] = off_s + is - cnt_s;
    }
    __syncthreads();
    if (tid == NT - 1) { sc.carry_t = off_t + it; sc.carry_s = off_s + is; }
    __syncthreads();
  }
  if (tid == 0) {
    o.tile_cum[p.batch] = sc.carry_t;
    o.seg_cum[p.batch] = sc.carry_s;
  }
  __syncthreads();
}

__global__ void __launch_bounds__(256) attn_plan_kernel(const AttnParams p) {
  __shared__ PlanScan sc;
  pdl_wait();   // the plan arrays may still be read by the merge kernel of the previous call
  pdl_launch_dependents();
  const PlanOut o{p.tile_cum, p.seg_cum, p.nt, p.tile0, p.sq, p.qrow0, p.klen};
  build_plan<256>(p, o, sc, true);
}

// Plan of an attention CTA: built into shared memory at `plan_smem` (plan_in_kernel; CTA 0 also stores
// it in the scratch arrays for the merge kernel) or taken from the scratch arrays.  Block-wide.
template <int NT>
__device__ __forceinline__ PlanView attention_cta_plan(const AttnParams& p, uint8_t* plan_smem) {
  if (!p.plan_in_kernel) return PlanView{p.tile_cum, p.seg_cum, p.nt, p.tile0, p.sq, p.qrow0, p.klen};
  const int B = p.batch;
  long long* tc = reinterpret_cast<long long*>(plan_smem);
  int* ints = reinterpret_cast<int*>(tc + (B + 1));
  const PlanOut o{tc, ints, ints + (B + 1), ints + (B + 1) + B, ints + (B + 1) + 2 * B, ints + (B + 1) + 3 * B,
                  ints + (B + 1) + 4 * B};
  PlanScan& sc = *reinterpret_cast<PlanScan*>(plan_smem + (((B + 1) * 8 + (B + 1) * 4 + 5 * B * 4 + 7) & ~7));
  build_plan<NT>(p, o, sc, blockIdx.x == 0);
  if (blockIdx.x == 0) {
    for (int b = threadIdx.x; b <= B; b += NT) {
      p.tile_cum[b] = o.tile_cum[b];
      p.seg_cum[b] = o.seg_cum[b];
      if (b < B) {
        p.nt[b] = o.nt[b];
        p.tile0[b] = o.tile0[b];
        p.sq[b] = o.sq[b];
        p.qrow0[b] = o.qrow0[b];
        p.klen[b] = o.klen[b];
      }
    }
  }
  return PlanView{o.tile_cum, o.seg_cum, o.nt, o.tile0, o.sq, o.qrow0, o.klen};
}

// Position of a warp inside the flat tile space (identical on all 32 lanes).
struct Cursor {
  int b, seg, nseg, t, nt, tile0, L, sq, nmb, segbase, qr;   // qr: first packed query row of the sequence
};

__device__ __forceinline__ void cursor_load_seq(const AttnParams& p, const PlanView& pv, Cursor& c) {
  c.nt = pv.nt[c.b];
  c.tile0 = pv.tile0[c.b];
  c.L = pv.klen[c.b];
  c.sq = pv.sq[c.b];
  c.qr = p.cu_seqlens_q ? pv.qrow0[c.b] : 0;   // loaded with the rest: no dependent load where Q is addressed
  c.nmb = (p.group * c.sq + p.rows_per_seg - 1) / p.rows_per_seg;
  c.nseg = p.hkv * c.nmb;
  c.segbase = pv.seg_cum[c.b];
}

// Finds the sequence and segment that own flat tile g.  Called by all 32 lanes of a warp with
// the same g: the search over tile_cum is 32-way (one probe per lane, a vote per round), two
// dependent loads for up to 1024 sequences where a binary search would chain ten.
__device__ __forceinline__ void cursor_locate(const AttnParams& p, const PlanView& pv, Cursor& c, long long g) {
  const int lane = threadIdx.x & 31;
  int lo = 0, hi = p.batch;  // tile_cum[lo] <= g < tile_cum[hi]
  while (hi - lo > 1) {
    const int step = (hi - lo + 31) >> 5;
    const int idx = lo + (lane + 1) * step;
    const bool le = idx < hi && pv.tile_cum[idx] <= g;
    const int cnt = __popc(__ballot_sync(0xffffffffu, le));   // probes are monotone: the first cnt lanes vote yes
    const int nlo = lo + cnt * step;
    hi = min(hi, nlo + step);
    lo = nlo;
  }
  c.b = lo;
  cursor_load_seq(p, pv, c);
  const long long off = g - pv.tile_cum[lo];
  c.seg = (int)(off / c.nt);
  c.t = (int)(off - (long long)c.seg * c.nt);
}

// Moves to the next tile; only called while tiles remain, so a non-empty
// sequence always follows.
__device__ __forceinline__ void cursor_advance(const AttnParams& p, const PlanView& pv, Cursor& c) {
  if (++c.t < c.nt) return;
  c.t = 0;
  if (++c.seg < c.nseg) return;
  c.seg = 0;
  while (++c.b < p.batch) {
    cursor_load_seq(p, pv, c);
    if (c.nt > 0 && c.nseg > 0) return;
  }
  c.b = p.batch - 1;  // not reached when the caller counts tiles correctly
}

// What the merge kernel needs to know about the tile a worker's range starts at: written by lane 0 of
// every worker whose range starts inside [0, total), read by the merge block of that boundary.
__device__ __forceinline__ void write_boundary_record(const AttnParams& p, int w, const Cursor& c) {
  int4* rec = reinterpret_cast<int4*>(p.bound_rec + 8 * (size_t)w);
  rec[0] = make_int4(c.b, c.seg, c.t, c.nt);
  rec[1] = make_int4(c.sq, c.qr, c.segbase, c.nmb);
}

template <int RB>
__device__ __forceinline__ uint32_t swz(int row) {
  if constexpr (RB == 128) return row & 7;
  else if constexpr (RB == 64) return (row >> 1) & 3;
  else return (row >> 2) & 1;
}

// ---------------------------------------------------------------------------
// Copy side of a worker warp: walks the warp's tile range ahead of the math,
// one TMA box per (page, head, K|V, 128-byte half), page indices read one tile
// before the copy that needs them.
// ---------------------------------------------------------------------------
template <typename T, int KVB, bool GATHER>
struct TileProducer {
  static constexpr int TILE_N = T::TILE_N;
  static constexpr int RB = T::RB;
  static constexpr int NH = T::NH;
  const AttnParams& p;
  const PlanView& pv;
  const CUtensorMap* tmK;
  const CUtensorMap* tmV;
  uint32_t stage0, bar0;
  // page size and box height are powers of two: shifts instead of divisions on the per-tile path
  int lane, p_shift, box_shift, box_rows, nbox, hb_shift, my_tiles, issued, pg, h;
  const int32_t* pt_row;   // page-table row of the sequence the cursor is in
  Cursor pc;

  __device__ __forceinline__ TileProducer(const AttnParams& p_, const PlanView& pv_, const CUtensorMap* k,
                                          const CUtensorMap* v, uint32_t stage0_, uint32_t bar0_, int lane_,
                                          long long r0, int my_tiles_)
      : p(p_), pv(pv_), tmK(k), tmV(v), stage0(stage0_), bar0(bar0_), lane(lane_), my_tiles(my_tiles_), issued(0) {
    p_shift = 31 - __clz(p.page_size);
    box_rows = p.page_size < TILE_N ? p.page_size : TILE_N;
    box_shift = 31 - __clz(box_rows);
    hb_shift = (NH == 2 && !p.merged_halves) ? 1 : 0;   // log2 of the boxes per (page, K|V)
    nbox = (TILE_N >> box_shift) << (hb_shift + 1);
    cursor_locate(p, pv, pc, r0);
    enter_segment();
    pg = (!GATHER && lane < nbox) ? page_for(lane) : 0;
  }
  __device__ __forceinline__ void enter_segment() {
    h = pc.seg / pc.nmb;
    pt_row = p.page_table + (int64_t)pc.b * p.pt_rs;
  }
  __device__ __forceinline__ int page_for(int j) const {
    const int i = j >> (hb_shift + 1);
    const int key = (pc.tile0 + pc.t) * TILE_N + (i << box_shift);
    if (key >= pc.L) return 0;
    return pt_row[key >> p_shift];
  }
  // One tile, 16 bytes per cp.async: 256 chunks of K and 256 of V whatever the row length, eight of each per
  // lane.  Lane l looks up the pages of tokens l and l + 32 of the tile; the chunks get them by shuffle.
  __device__ __forceinline__ void issue_gather(int stage) {
    constexpr int CPR = T::ROW_BYTES / 16;     // chunks per row
    constexpr int CHUNKS = TILE_N * CPR;
    static_assert(CHUNKS % 32 == 0 && TILE_N <= 64, "tile geometry of the gather path");
    const uint32_t sbase = stage0 + (uint32_t)stage * T::STAGE_BYTES;
    const uint32_t bar = bar0 + 8u * stage;
    const int k0 = (pc.tile0 + pc.t) * TILE_N;
    int nvalid = pc.L - k0;
    if (nvalid > TILE_N) nvalid = TILE_N;
    const int pg_a = lane < nvalid ? pt_row[(k0 + lane) >> p_shift] : 0;
    const int pg_b = (TILE_N > 32 && lane + 32 < nvalid) ? pt_row[(k0 + lane + 32) >> p_shift] : 0;
#pragma unroll
    for (int c = lane; c < CHUNKS; c += 32) {
      const int tk = c / CPR, c16 = c % CPR;
      const int pa = __shfl_sync(0xffffffffu, pg_a, tk & 31), pb = __shfl_sync(0xffffffffu, pg_b, tk & 31);
      const int page = tk < 32 ? pa : pb;
      if (tk >= nvalid) continue;
      if ((unsigned)page >= (unsigned long long)p.n_pages) {   // never dereferenced: the tile keeps stale bytes there
        if (c16 == 0) report(KB200_STATUS_BAD_PAGE, page, KID_ATTN);
        continue;
      }
      const long long off = (long long)page * p.kv_ps_b + (long long)((k0 + tk) & (p.page_size - 1)) * p.kv_ts_b +
                            (long long)h * p.kv_hs_b + 16 * c16;
      uint32_t dst;
      if constexpr (NH == 2) dst = sbase + (uint32_t)(c16 >> 3) * (TILE_N * 128) + (uint32_t)tk * 128 + (uint32_t)(((c16 & 7) ^ (tk & 7)) << 4);
      else dst = sbase + (uint32_t)tk * RB + (uint32_t)((c16 ^ (int)swz<RB>(tk)) << 4);
      cp_async_16(dst, p.k_base + off);
      cp_async_16(dst + T::KV_TILE_BYTES, p.v_base + off);
    }
    cp_async_mbar_arrive(bar);
    __syncwarp();
    if (lane == 0) mbar_arrive_plain(bar);   // the arrival the barrier was initialised for; the 32 above are extra
    advance_after_issue();
  }
  __device__ __forceinline__ void advance_after_issue() {
    ++issued;
    if (issued < my_tiles) {
      cursor_advance(p, pv, pc);
      if (pc.t == 0) enter_segment();   // (a new segment, possibly of a new sequence)
      if constexpr (!GATHER) pg = lane < nbox ? page_for(lane) : 0;
    }
  }
  __device__ __forceinline__ void issue(int stage) {
    if constexpr (GATHER) { issue_gather(stage); return; }
    const uint32_t sbase = stage0 + (uint32_t)stage * T::STAGE_BYTES;
    const uint32_t bar = bar0 + 8u * stage;
    const int k0 = (pc.tile0 + pc.t) * TILE_N;
    int nvalid = pc.L - k0;
    if (nvalid > TILE_N) nvalid = TILE_N;
    const int nvb = (nvalid + box_rows - 1) >> box_shift;
    if (lane == 0) mbar_expect_tx(bar, (uint32_t)((nvb << box_shift) * T::ROW_BYTES * 2));
    __syncwarp();
    for (int j = lane; j < nbox; j += 32) {
      const int i = j >> (hb_shift + 1);
      if (i >= nvb) continue;
      const int sub = j & ((2 << hb_shift) - 1);
      const int kv = sub >> hb_shift, half = sub & ((1 << hb_shift) - 1);
      const int key = k0 + (i << box_shift);
      const int page = (j == lane) ? pg : page_for(j);
      if ((unsigned)page >= (unsigned long long)p.n_pages) report(KB200_STATUS_BAD_PAGE, page, KID_ATTN);
      const uint32_t dst = sbase + (uint32_t)kv * T::KV_TILE_BYTES + (uint32_t)half * (TILE_N * RB) +
                           (uint32_t)(i << box_shift) * RB;
      if (NH == 2 && p.merged_halves)   // (the box is the whole tile: [half][token][128 bytes], as two boxes would leave it)
        tma_load_5d(dst, kv ? tmV : tmK, bar, 0, key & (p.page_size - 1), 0, h, page);
      else
        tma_load_4d(dst, kv ? tmV : tmK, bar, half * (RB / KVB), key & (p.page_size - 1), h, page);
    }
    advance_after_issue();
  }
  __device__ __forceinline__ bool more() const { return issued < my_tiles; }
};

// ---------------------------------------------------------------------------
// The attention kernel.  KVB: bytes per K/V element (2: bf16/f16, 1: e4m3);
// BF16: operand type of the MMAs (bf16 when K/V are bf16, else f16).
// ---------------------------------------------------------------------------
template <int KVB, int HD, bool BF16, int NW, int NS, bool GATHER>
__global__ void __launch_bounds__(NW * 32, 1)
paged_attn_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                  const __grid_constant__ AttnParams p) {
  using T = AttnTile<KVB, HD, NW, NS>;
  constexpr int kAttnWarps = NW;
  constexpr int TILE_N = T::TILE_N;
  constexpr int RB = T::RB;
  constexpr int NT8 = TILE_N / 8;    // score n-tiles per tile
  constexpr int NKS = TILE_N / 16;   // k-steps of P V
  constexpr int NOT = HD / 8;        // output n-tiles
  constexpr int NQF = HD / 16;       // Q fragments (k-steps of Q K^T)
  constexpr float kLog2e = 1.4426950408889634f;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c4 = lane & 3, g8 = lane >> 2;
  const uint32_t my_stage0 = smem_base + (uint32_t)(warp * NS) * T::STAGE_BYTES;
  const uint32_t bar0 = smem_base + (uint32_t)(kAttnWarps * NS) * T::STAGE_BYTES +
                        (uint32_t)(warp * NS) * 8u;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kAttnWarps * NS; ++i)
      mbar_init(smem_base + (uint32_t)(kAttnWarps * NS) * T::STAGE_BYTES + 8u * i, 1);
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();
  pdl_launch_dependents();
  pdl_wait();   // the append (and a plan launch, if there was one) must have completed
  const PlanView plan = attention_cta_plan<NW * 32>(p, smem_raw + (smem_base - smem_u32(smem_raw)) + T::PLAN_OFF);
  // No block-wide barrier below this line: warps are independent workers.

  const long long total = plan.tile_cum[p.batch];
  const int w = blockIdx.x * kAttnWarps + warp;
  const long long r0 = (long long)w * total / p.n_workers;
  const long long r1 = (long long)(w + 1) * total / p.n_workers;
  if (r0 >= r1) {
    if (w > 0 && r0 < total) {   // an empty range still marks a boundary the merge kernel may have to handle
      Cursor c0;
      cursor_locate(p, plan, c0, r0);
      if (lane == 0) write_boundary_record(p, w, c0);
    }
    return;
  }
  const int my_tiles = (int)(r1 - r0);

  TileProducer<T, KVB, GATHER> prod(p, plan, &tmK, &tmV, my_stage0, bar0, lane, r0, my_tiles);
  Cursor cc = prod.pc;   // consumer side: starts where the producer starts
  if (lane == 0 && w > 0) write_boundary_record(p, w, cc);
  for (int s = 0; s < NS && prod.more(); ++s) prod.issue(s);

  uint32_t qf[NQF][4];
  float o[NOT][4];
  float m0 = 0.f, m1 = 0.f, l0 = 0.f, l1 = 0.f;
  float sl2 = 0.f, vscale = 1.f;
  int lim0 = 0, lim1 = 0, row0 = 0, row1 = 0, h = 0;
  bool valid0 = false, valid1 = false;
  bool fresh = true;
  long long piece_start = r0;

  for (int it = 0; it < my_tiles; ++it) {
    const long long g = r0 + it;
    if (fresh) {
      fresh = false;
      piece_start = g;
      const int mb = cc.seg % cc.nmb;
      h = cc.seg / cc.nmb;
      row0 = mb * kRowsPerSeg + g8;
      row1 = row0 + 8;
      const int nrows = p.group * cc.sq;
      valid0 = row0 < nrows;
      valid1 = row1 < nrows;
      const int j0 = row0 / p.group, j1 = row1 / p.group;
      const bool upper = p.causal || p.window_left >= 0;
      lim0 = upper ? cc.L - cc.sq + j0 : cc.L - 1;
      lim1 = upper ? cc.L - cc.sq + j1 : cc.L - 1;
      const float ksc = p.ks_vec ? p.ks_vec[h] : p.ks;
      vscale = p.vs_vec ? p.vs_vec[h] : p.vs;
      sl2 = p.softmax_scale * ksc * kLog2e;
      m0 = m1 = -INFINITY;
      l0 = l1 = 0.f;
#pragma unroll
      for (int i = 0; i < NOT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
      // Q fragments, straight from global memory (4 KB per segment at most)
      const int64_t qb = (int64_t)cc.b * p.q_bs;
      const char* q0 = p.q + 2 * (qb + (int64_t)(cc.qr + j0) * p.q_rs +
                                  (int64_t)(h * p.group + row0 % p.group) * p.q_hs);
      const char* q1 = p.q + 2 * (qb + (int64_t)(cc.qr + j1) * p.q_rs +
                                  (int64_t)(h * p.group + row1 % p.group) * p.q_hs);
      if constexpr (KVB == 2) {
#pragma unroll
        for (int ks = 0; ks < NQF; ++ks) {
          const int d = 16 * ks + 2 * c4;
          qf[ks][0] = valid0 ? *reinterpret_cast<const uint32_t*>(q0 + 2 * d) : 0u;
          qf[ks][1] = valid1 ? *reinterpret_cast<const uint32_t*>(q1 + 2 * d) : 0u;
          qf[ks][2] = valid0 ? *reinterpret_cast<const uint32_t*>(q0 + 2 * (d + 8)) : 0u;
          qf[ks][3] = valid1 ? *reinterpret_cast<const uint32_t*>(q1 + 2 * (d + 8)) : 0u;
        }
      } else {
        // e4m3 K rows are read four consecutive d per thread, so Q uses the same d order:
        // k-slots (2c, 2c+1) <-> d = 16*ch + 4c + {0,1}; (2c+8, 2c+9) <-> d = 16*ch + 4c + {2,3}
#pragma unroll
        for (int ch = 0; ch < NQF; ++ch) {
          const int d = 16 * ch + 4 * c4;
          uint2 a = valid0 ? *reinterpret_cast<const uint2*>(q0 + 2 * d) : make_uint2(0u, 0u);
          uint2 b = valid1 ? *reinterpret_cast<const uint2*>(q1 + 2 * d) : make_uint2(0u, 0u);
          if (p.q_is_bf16) {
            a.x = pack2<false>(bf16_bits_to_float(a.x & 0xffffu), bf16_bits_to_float(a.x >> 16));
            a.y = pack2<false>(bf16_bits_to_float(a.y & 0xffffu), bf16_bits_to_float(a.y >> 16));
            b.x = pack2<false>(bf16_bits_to_float(b.x & 0xffffu), bf16_bits_to_float(b.x >> 16));
            b.y = pack2<false>(bf16_bits_to_float(b.y & 0xffffu), bf16_bits_to_float(b.y >> 16));
          }
          qf[ch][0] = a.x; qf[ch][1] = b.x; qf[ch][2] = a.y; qf[ch][3] = b.y;
        }
      }
    }

    // Last tile of this segment and the next segment belongs to the same sequence: pull its Q rows
    // into L1 now, so that the loads at the segment switch do not wait for L2.
    if (cc.t == cc.nt - 1 && cc.seg + 1 < cc.nseg && it + 1 < my_tiles && (c4 < 2 || HD == 128)) {
      const int ns = cc.seg + 1, nh = ns / cc.nmb;
      const int r = (ns - nh * cc.nmb) * kRowsPerSeg + g8 + (c4 & 1) * 8;
      if (r < p.group * cc.sq)
        prefetch_l1(p.q + 2 * ((int64_t)cc.b * p.q_bs + (int64_t)(cc.qr + r / p.group) * p.q_rs +
                               (int64_t)(nh * p.group + r % p.group) * p.q_hs) + (c4 >> 1) * 128);
    }

    const int stage = it % NS;
    const uint32_t parity = (uint32_t)(it / NS) & 1u;
    if (!mbar_wait_bounded(bar0 + 8u * stage, parity)) {
      if (lane == 0) report(KB200_STATUS_WAIT_TIMEOUT, w, KID_ATTN);
      return;
    }
    const uint32_t kbase = my_stage0 + (uint32_t)stage * T::STAGE_BYTES;
    const uint32_t vbase = kbase + T::KV_TILE_BYTES;
    const int key0 = (cc.tile0 + cc.t) * TILE_N;

    // ---- S = Q K^T
    float s[NT8][4];
#pragma unroll
    for (int n = 0; n < NT8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
    if constexpr (KVB == 2) {
#pragma unroll
      for (int n = 0; n < NT8; ++n) {
        const int r = n * 8 + (lane & 7);
#pragma unroll
        for (int q4 = 0; q4 < HD / 32; ++q4) {
          const int ch = q4 * 4 + (lane >> 3);
          const uint32_t addr = kbase + (uint32_t)(ch >> 3) * (TILE_N * 128) + (uint32_t)r * 128 +
                                ((uint32_t)((ch & 7) ^ (r & 7)) << 4);
          uint32_t b0, b1, b2, b3;
          ldsm_x4(b0, b1, b2, b3, addr);
          mma16816<BF16>(s[n], qf[2 * q4], b0, b1);
          mma16816<BF16>(s[n], qf[2 * q4 + 1], b2, b3);
        }
      }
    } else {
#pragma unroll
      for (int n = 0; n < NT8; ++n) {
        const int r = n * 8 + (lane & 7);
#pragma unroll
        for (int q4 = 0; q4 < HD / 64; ++q4) {
          const int ch = q4 * 4 + (lane >> 3);
          const uint32_t addr = kbase + (uint32_t)r * RB + ((uint32_t)(ch ^ swz<RB>(r)) << 4);
          uint32_t x[4];
          ldsm_x4(x[0], x[1], x[2], x[3], addr);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t b0, b1;
            e4m3x4_to_f16x4(x[i], b0, b1);
            mma16816<false>(s[n], qf[q4 * 4 + i], b0, b1);
          }
        }
      }
    }

    // ---- mask (only tiles that touch a boundary)
    const int key_last = key0 + TILE_N - 1;
    const int min_lim = (p.causal || p.window_left >= 0) ? cc.L - cc.sq : cc.L - 1;
    const bool need_mask = key_last > min_lim || (p.window_left >= 0 && key0 < cc.L - 1 - p.window_left);
    if (need_mask) {
      const int lo0 = p.window_left >= 0 ? lim0 - p.window_left : 0;
      const int lo1 = p.window_left >= 0 ? lim1 - p.window_left : 0;
#pragma unroll
      for (int n = 0; n < NT8; ++n) {
        const int k = key0 + n * 8 + 2 * c4;
        if (k > lim0 || k < lo0) s[n][0] = -INFINITY;
        if (k + 1 > lim0 || k + 1 < lo0) s[n][1] = -INFINITY;
        if (k > lim1 || k < lo1) s[n][2] = -INFINITY;
        if (k + 1 > lim1 || k + 1 < lo1) s[n][3] = -INFINITY;
      }
    }

    // ---- online softmax (base 2)
    float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < NT8; ++n) {
      t0 = fmaxf(t0, fmaxf(s[n][0], s[n][1]));
      t1 = fmaxf(t1, fmaxf(s[n][2], s[n][3]));
    }
    t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1));
    t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
    t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1));
    t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
    const float mn0 = fmaxf(m0, t0), mn1 = fmaxf(m1, t1);
    if (__any_sync(0xffffffffu, mn0 > m0 || mn1 > m1)) {
      const float c0 = (m0 == -INFINITY) ? 0.f : ex2((m0 - mn0) * sl2);
      const float c1 = (m1 == -INFINITY) ? 0.f : ex2((m1 - mn1) * sl2);
      l0 *= c0;
      l1 *= c1;
#pragma unroll
      for (int i = 0; i < NOT; ++i) {
        o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1;
      }
      m0 = mn0;
      m1 = mn1;
    }
    const float ms0 = (m0 == -INFINITY) ? 0.f : m0 * sl2;
    const float ms1 = (m1 == -INFINITY) ? 0.f : m1 * sl2;
    uint32_t pf[NKS][4];
#pragma unroll
    for (int n = 0; n < NT8; ++n) {
      const float p0 = ex2(fmaf(s[n][0], sl2, -ms0));
      const float p1 = ex2(fmaf(s[n][1], sl2, -ms0));
      const float p2 = ex2(fmaf(s[n][2], sl2, -ms1));
      const float p3 = ex2(fmaf(s[n][3], sl2, -ms1));
      l0 += p0 + p1;
      l1 += p2 + p3;
      pf[n >> 1][(n & 1) * 2 + 0] = pack2<BF16>(p0, p1);
      pf[n >> 1][(n & 1) * 2 + 1] = pack2<BF16>(p2, p3);
    }

    // ---- O += P V.  Rows of V past the sequence end may hold anything (NaN
    // bit patterns included), so they are zeroed in the one tile that has them;
    // every other tile runs the mask-free instantiation.
    auto pv = [&](auto masked_tag) {
      constexpr bool MASKED = decltype(masked_tag)::value;
#pragma unroll
      for (int ks = 0; ks < NKS; ++ks) {
        uint32_t mk_lo = 0xffffffffu, mk_hi = 0xffffffffu;
        if constexpr (MASKED) {
          const int kv_left = cc.L - (key0 + 16 * ks);  // valid keys in this 16-key block
          mk_lo = (2 * c4 < kv_left ? 0x0000ffffu : 0u) | (2 * c4 + 1 < kv_left ? 0xffff0000u : 0u);
          mk_hi = (2 * c4 + 8 < kv_left ? 0x0000ffffu : 0u) | (2 * c4 + 9 < kv_left ? 0xffff0000u : 0u);
        }
        const int row = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
        if constexpr (KVB == 2) {
#pragma unroll
          for (int q2 = 0; q2 < HD / 16; ++q2) {
            const int ch = q2 * 2 + (lane >> 4);
            const uint32_t addr = vbase + (uint32_t)(ch >> 3) * (TILE_N * 128) + (uint32_t)row * 128 +
                                  ((uint32_t)((ch & 7) ^ (row & 7)) << 4);
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(b0, b1, b2, b3, addr);
            if constexpr (MASKED) { b0 &= mk_lo; b1 &= mk_hi; b2 &= mk_lo; b3 &= mk_hi; }
            mma16816<BF16>(o[2 * q2], pf[ks], b0, b1);
            mma16816<BF16>(o[2 * q2 + 1], pf[ks], b2, b3);
          }
        } else {
#pragma unroll
          for (int q2 = 0; q2 < HD / 32; ++q2) {
            const int ch = q2 * 2 + (lane >> 4);
            const uint32_t addr = vbase + (uint32_t)row * RB + ((uint32_t)(ch ^ swz<RB>(row)) << 4);
            uint32_t x0, x1, x2, x3;
            ldsm_x4_t(x0, x1, x2, x3, addr);
            if constexpr (MASKED) { x0 &= mk_lo; x1 &= mk_hi; x2 &= mk_lo; x3 &= mk_hi; }
            // word = [key 2c: d, d+1 | key 2c+1: d, d+1]  ->  [d: key 2c, 2c+1 | d+1: key 2c, 2c+1]
            x0 = __byte_perm(x0, 0, 0x3120);
            x1 = __byte_perm(x1, 0, 0x3120);
            x2 = __byte_perm(x2, 0, 0x3120);
            x3 = __byte_perm(x3, 0, 0x3120);
            uint32_t e0, o0, e1, o1;
            e4m3x4_to_f16x4(x0, e0, o0);
            e4m3x4_to_f16x4(x1, e1, o1);
            mma16816<false>(o[4 * q2 + 0], pf[ks], e0, e1);  // d = 16*(2*q2)   + 2g
            mma16816<false>(o[4 * q2 + 1], pf[ks], o0, o1);  // d = 16*(2*q2)   + 2g + 1
            e4m3x4_to_f16x4(x2, e0, o0);
            e4m3x4_to_f16x4(x3, e1, o1);
            mma16816<false>(o[4 * q2 + 2], pf[ks], e0, e1);  // d = 16*(2*q2+1) + 2g
            mma16816<false>(o[4 * q2 + 3], pf[ks], o0, o1);  // d = 16*(2*q2+1) + 2g + 1
          }
        }
      }
    };
    if (key0 + TILE_N > cc.L) pv(std::true_type{});
    else pv(std::false_type{});

    // ---- this stage has been read: refill it with the tile NS ahead
    __syncwarp();
    if (prod.more()) {
      fence_proxy_async();
      prod.issue(stage);
    }

    // ---- end of this warp's piece of the segment?
    const bool seg_end = cc.t == cc.nt - 1;
    if (seg_end || it == my_tiles - 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
      l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
      l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
      l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
      const bool whole = seg_end && (g - piece_start == cc.nt - 1);
      const int seg_id = cc.segbase + cc.seg;
      if (whole) {
        const float i0 = l0 > 0.f ? vscale / l0 : 0.f;
        const float i1 = l1 > 0.f ? vscale / l1 : 0.f;
        const int64_t ob = (int64_t)cc.b * p.o_bs;
        const int qr = cc.qr;
        const int j0 = row0 / p.group, j1 = row1 / p.group;
        const int hq0 = h * p.group + row0 % p.group, hq1 = h * p.group + row1 % p.group;
        char* out0 = p.out + 2 * (ob + (int64_t)(qr + j0) * p.o_rs + (int64_t)hq0 * p.o_hs);
        char* out1 = p.out + 2 * (ob + (int64_t)(qr + j1) * p.o_rs + (int64_t)hq1 * p.o_hs);
        const bool obf = KVB == 2 ? BF16 : (p.q_is_bf16 != 0);
        constexpr float kLn2 = 0.6931471805599453f;
        const float lse0 = l0 > 0.f ? m0 * sl2 * kLn2 + logf(l0) : -INFINITY;
        const float lse1 = l1 > 0.f ? m1 * sl2 * kLn2 + logf(l1) : -INFINITY;
        if constexpr (KVB == 2) {
#pragma unroll
          for (int i = 0; i < NOT; ++i) {
            const int d = 8 * i + 2 * c4;
            if (valid0) *reinterpret_cast<uint32_t*>(out0 + 2 * d) = pack2<BF16>(o[i][0] * i0, o[i][1] * i0);
            if (valid1) *reinterpret_cast<uint32_t*>(out1 + 2 * d) = pack2<BF16>(o[i][2] * i1, o[i][3] * i1);
          }
        } else {
#pragma unroll
          for (int ch = 0; ch < HD / 16; ++ch) {
            const int d = 16 * ch + 4 * c4;
            const float a0 = o[2 * ch][0] * i0, a1 = o[2 * ch + 1][0] * i0, a2 = o[2 * ch][1] * i0, a3 = o[2 * ch + 1][1] * i0;
            const float b0 = o[2 * ch][2] * i1, b1 = o[2 * ch + 1][2] * i1, b2 = o[2 * ch][3] * i1, b3 = o[2 * ch + 1][3] * i1;
            if (valid0)
              *reinterpret_cast<uint2*>(out0 + 2 * d) = obf ? make_uint2(pack2<true>(a0, a1), pack2<true>(a2, a3))
                                                            : make_uint2(pack2<false>(a0, a1), pack2<false>(a2, a3));
            if (valid1)
              *reinterpret_cast<uint2*>(out1 + 2 * d) = obf ? make_uint2(pack2<true>(b0, b1), pack2<true>(b2, b3))
                                                            : make_uint2(pack2<false>(b0, b1), pack2<false>(b2, b3));
          }
        }
        if (p.lse && c4 == 0) {
          if (valid0) p.lse[(int64_t)cc.b * p.lse_bs + (int64_t)hq0 * p.lse_hs + qr + j0] = lse0;
          if (valid1) p.lse[(int64_t)cc.b * p.lse_bs + (int64_t)hq1 * p.lse_hs + qr + j1] = lse1;
        }
      } else {
        // (rows past the segment's end are neither written here nor read by the merge: with one query token
        // and four heads per group that is three quarters of the partial)
        const int64_t slot = (int64_t)seg_id + w;
        float* po = p.part_o + slot * (kRowsPerSeg * HD);
        float* pml = p.part_ml + slot * (kRowsPerSeg * 2);
        if (c4 == 0) {
          if (valid0) *reinterpret_cast<float2*>(pml + g8 * 2) = make_float2((m0 == -INFINITY) ? -INFINITY : m0 * sl2, l0);
          if (valid1) *reinterpret_cast<float2*>(pml + (g8 + 8) * 2) = make_float2((m1 == -INFINITY) ? -INFINITY : m1 * sl2, l1);
        }
        if constexpr (KVB == 2) {
#pragma unroll
          for (int i = 0; i < NOT; ++i) {
            const int d = 8 * i + 2 * c4;
            if (valid0) *reinterpret_cast<float2*>(po + g8 * HD + d) = make_float2(o[i][0], o[i][1]);
            if (valid1) *reinterpret_cast<float2*>(po + (g8 + 8) * HD + d) = make_float2(o[i][2], o[i][3]);
          }
        } else {
#pragma unroll
          for (int ch = 0; ch < HD / 16; ++ch) {
            const int d = 16 * ch + 4 * c4;
            if (valid0)
              *reinterpret_cast<float4*>(po + g8 * HD + d) =
                  make_float4(o[2 * ch][0], o[2 * ch + 1][0], o[2 * ch][1], o[2 * ch + 1][1]);
            if (valid1)
              *reinterpret_cast<float4*>(po + (g8 + 8) * HD + d) =
                  make_float4(o[2 * ch][2], o[2 * ch + 1][2], o[2 * ch][3], o[2 * ch + 1][3]);
          }
        }
      }
      fresh = true;
    }
    if (it + 1 < my_tiles) cursor_advance(p, plan, cc);
  }
}

}  // namespace kb200
#include "paged_attention_rows32.cuh"
namespace kb200 {

// ---------------------------------------------------------------------------
// Decode kernel: segments of at most 8 query rows (GQA group x query positions),
// computed in the transposed form so that the 16-wide MMA dimension carries keys
// (for Q K^T) or head_dim (for P V) instead of mostly empty query rows:
//
//   S^T[keys x q] = K[keys x d] . Q^T[d x q]        A = K tile (ldmatrix), B = Q^T (registers)
//   O^T[d x q]   += V^T[d x keys] . P^T[keys x q]   A = V^T (ldmatrix.trans), B = P^T
//
// Compared with the general kernel this halves the MMAs per key, halves the
// accumulator registers (O^T is head_dim x 8) and drops the unused-row math.
// The softmax weights come out of the first product with keys along the thread's
// row index; movmatrix.trans turns them into the B fragment of the second.
// e4m3 K/V are widened to f16 in registers as in the general kernel; the d-order
// inside each 16-wide slice is permuted consistently between the operands
// (K: bytes 4c..4c+3 of a 16-byte chunk feed k-slots 2c,2c+1 and 2c+8,2c+9;
//  V: MMA row g is d = 16*chunk + 2g, row g+8 is d = 16*chunk + 2g + 1).
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
template <bool BF16>
__device__ __forceinline__ void mma16816r(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  if constexpr (BF16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

template <int KVB, int HD, bool BF16, int NW, int NS, bool GATHER>
__global__ void __launch_bounds__(NW * 32, 1)
paged_attn_decode_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                         const __grid_constant__ AttnParams p) {
  using T = AttnTile<KVB, HD, NW, NS>;
  constexpr int TILE_N = T::TILE_N;
  constexpr int RB = T::RB;
  constexpr int NMT = TILE_N / 16;  // 16-key blocks per tile
  constexpr int NDT = HD / 16;      // 16-wide head_dim slices
  constexpr float kLog2e = 1.4426950408889634f;
  static_assert(TILE_N % 16 == 0, "tile must hold whole 16-key blocks");
  // head_dim 256 only exists as several KV heads read as one (AttnParams::head_pack): e4m3 rows of 64 or 128
  // bytes in pools with pages of one or two tokens.  The products run over the wide head with block-sparse Q:
  // S^T = [K_0 | K_1 | ..] [Q_0^T ; Q_1^T ; ..] where Q_g^T is zero outside the rows of head g, so every column
  // of S^T is the score of its own head, and of O^T = [V_0 | V_1 | ..]^T P^T a column owns the slice of its head.
  // (the same for 16-bit pools with 128-byte rows: two heads of 64 as one of 128; plain 16-bit head_dim-128 pools
  // never run this kernel)
  constexpr bool PACKED = HD == 256 || (KVB == 2 && HD == 128);
  // e4m3 tile rows are RB bytes per 128-byte slab (two slabs when the row has 256 bytes)
  auto kv8_off = [](int r, int ch) -> uint32_t {
    if constexpr (T::NH == 2) return (uint32_t)(ch >> 3) * (TILE_N * 128) + (uint32_t)r * 128 + ((uint32_t)((ch & 7) ^ (r & 7)) << 4);
    else return (uint32_t)r * RB + ((uint32_t)(ch ^ (int)swz<RB>(r)) << 4);
  };

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c4 = lane & 3, g8 = lane >> 2;
  const uint32_t my_stage0 = smem_base + (uint32_t)(warp * NS) * T::STAGE_BYTES;
  const uint32_t bar0 = smem_base + (uint32_t)(NW * NS) * T::STAGE_BYTES + (uint32_t)(warp * NS) * 8u;
  if (threadIdx.x == 0) {
    for (int i = 0; i < NW * NS; ++i) mbar_init(smem_base + (uint32_t)(NW * NS) * T::STAGE_BYTES + 8u * i, 1);
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();
  pdl_launch_dependents();
  pdl_wait();   // the append (and a plan launch, if there was one) must have completed
  const PlanView plan = attention_cta_plan<NW * 32>(p, smem_raw + (smem_base - smem_u32(smem_raw)) + T::PLAN_OFF);
  // No block-wide barrier below this line: warps are independent workers.

  const long long total = plan.tile_cum[p.batch];
  const int w = blockIdx.x * NW + warp;
  const long long r0 = (long long)w * total / p.n_workers;
  const long long r1 = (long long)(w + 1) * total / p.n_workers;
  if (r0 >= r1) {
    if (w > 0 && r0 < total) {   // an empty range still marks a boundary the merge kernel may have to handle
      Cursor c0;
      cursor_locate(p, plan, c0, r0);
      if (lane == 0) write_boundary_record(p, w, c0);
    }
    return;
  }
  const int my_tiles = (int)(r1 - r0);

  TileProducer<T, KVB, GATHER> prod(p, plan, &tmK, &tmV, my_stage0, bar0, lane, r0, my_tiles);
  Cursor cc = prod.pc;   // consumer side: starts where the producer starts
  if (lane == 0 && w > 0) write_boundary_record(p, w, cc);
  for (int s = 0; s < NS && prod.more(); ++s) prod.issue(s);

  // lane-constant parts of the ldmatrix addresses
  const int mi = lane >> 3;                                  // which of the four 8x8 matrices this lane addresses
  const int k_row = (mi & 1) * 8 + (lane & 7);               // K: matrices (keys lo|hi) x (chunk, chunk+1)
  const int k_chunk = mi >> 1;
  const int v_row = KVB == 2 ? (mi >> 1) * 8 + (lane & 7) : (mi & 1) * 8 + (lane & 7);
  const int v_chunk = KVB == 2 ? (mi & 1) : (mi >> 1);

  uint32_t qb[NDT][2];   // Q^T B fragments: row g8 of the segment, one 16-wide d slice each
  float o[NDT][4];       // O^T: [d slice][ (d row g, q 2c) (d row g, q 2c+1) (d row g+8, q 2c) (d row g+8, q 2c+1) ]
  float m0 = 0.f, m1 = 0.f, l0 = 0.f, l1 = 0.f;   // running max / partial sum of query rows 2c and 2c+1
  float sl2 = 0.f, vscale = 1.f;
  int lim0 = 0, lim1 = 0, h = 0, mb = 0;
  bool fresh = true;
  long long piece_start = r0;

  for (int it = 0; it < my_tiles; ++it) {
    const long long g = r0 + it;
    if (fresh) {
      fresh = false;
      piece_start = g;
      mb = cc.seg % cc.nmb;
      h = cc.seg / cc.nmb;
      const int nrows = p.group * cc.sq;
      const bool upper = p.causal || p.window_left >= 0;
      const int q0 = mb * kDecodeRows + 2 * c4, q1 = q0 + 1;   // rows this thread accumulates
      lim0 = upper ? cc.L - cc.sq + q0 / p.group : cc.L - 1;
      lim1 = upper ? cc.L - cc.sq + q1 / p.group : cc.L - 1;
      const float ksc = p.ks_vec ? p.ks_vec[h] : p.ks;
      vscale = p.vs_vec ? p.vs_vec[h] : p.vs;
      sl2 = p.softmax_scale * ksc * kLog2e;
      m0 = m1 = -INFINITY;
      l0 = l1 = 0.f;
#pragma unroll
      for (int i = 0; i < NDT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
      // B fragments of Q^T: this thread supplies row (mb*8 + g8)
      const int qr = mb * kDecodeRows + g8;
      const bool qvalid = qr < nrows;
      // (h * group + g is the index of the query head with packed heads too: both count KV head by KV head)
      const char* qrow = p.q + 2 * ((int64_t)cc.b * p.q_bs + (int64_t)(cc.qr + qr / p.group) * p.q_rs +
                                    (int64_t)(h * p.group + qr % p.group) * p.q_hs);
      [[maybe_unused]] const int q_slice = PACKED ? (qr % p.group) / (p.group / p.head_pack) : 0;   // KV head inside the pack
      if constexpr (KVB == 2) {
#pragma unroll
        for (int ks = 0; ks < NDT; ++ks) {
          int d = 16 * ks + 2 * c4;
          bool mine = qvalid;
          if constexpr (PACKED) {   // zero outside the slice of the row's own KV head
            mine = qvalid && (16 * ks) / p.real_hd == q_slice;
            d -= q_slice * p.real_hd;
          }
          qb[ks][0] = mine ? *reinterpret_cast<const uint32_t*>(qrow + 2 * d) : 0u;
          qb[ks][1] = mine ? *reinterpret_cast<const uint32_t*>(qrow + 2 * (d + 8)) : 0u;
        }
      } else {
#pragma unroll
        for (int ch = 0; ch < NDT; ++ch) {
          int d = 16 * ch + 4 * c4;
          bool mine = qvalid;
          if constexpr (PACKED) {   // zero outside the slice of the row's own KV head
            mine = qvalid && (16 * ch) / p.real_hd == q_slice;
            d -= q_slice * p.real_hd;
          }
          uint2 a = mine ? *reinterpret_cast<const uint2*>(qrow + 2 * d) : make_uint2(0u, 0u);
          if (p.q_is_bf16) {
            a.x = pack2<false>(bf16_bits_to_float(a.x & 0xffffu), bf16_bits_to_float(a.x >> 16));
            a.y = pack2<false>(bf16_bits_to_float(a.y & 0xffffu), bf16_bits_to_float(a.y >> 16));
          }
          qb[ch][0] = a.x;
          qb[ch][1] = a.y;
        }
      }
    }

    // Last tile of this segment and the next segment belongs to the same sequence: pull its Q row
    // into L1 now, so that the loads at the segment switch do not wait for L2.
    if (!PACKED && cc.t == cc.nt - 1 && cc.seg + 1 < cc.nseg && it + 1 < my_tiles && (c4 == 0 || (HD == 128 && c4 == 1))) {
      const int ns = cc.seg + 1, nh = ns / cc.nmb;
      const int r = (ns - nh * cc.nmb) * kDecodeRows + g8;
      if (r < p.group * cc.sq)
        prefetch_l1(p.q + 2 * ((int64_t)cc.b * p.q_bs + (int64_t)(cc.qr + r / p.group) * p.q_rs +
                               (int64_t)(nh * p.group + r % p.group) * p.q_hs) + c4 * 128);
    }

    const int stage = it % NS;
    const uint32_t parity = (uint32_t)(it / NS) & 1u;
    if (!mbar_wait_bounded(bar0 + 8u * stage, parity)) {
      if (lane == 0) report(KB200_STATUS_WAIT_TIMEOUT, w, KID_ATTN);
      return;
    }
    const uint32_t kbase = my_stage0 + (uint32_t)stage * T::STAGE_BYTES;
    const uint32_t vbase = kbase + T::KV_TILE_BYTES;
    const int key0 = (cc.tile0 + cc.t) * TILE_N;

    // ---- S^T = K Q^T.  Two accumulator sets (even / odd d slices) keep dependent MMAs apart.
    float s[NMT][4], s2[NMT][4];
#pragma unroll
    for (int mt = 0; mt < NMT; ++mt) {
      s[mt][0] = s[mt][1] = s[mt][2] = s[mt][3] = 0.f;
      s2[mt][0] = s2[mt][1] = s2[mt][2] = s2[mt][3] = 0.f;
    }
    if constexpr (KVB == 2) {
#pragma unroll
      for (int ks = 0; ks < NDT; ++ks) {
#pragma unroll
        for (int mt = 0; mt < NMT; ++mt) {
          const int r = mt * 16 + k_row;
          const int ch = 2 * ks + k_chunk;
          const uint32_t addr = kbase + (uint32_t)(ch >> 3) * (TILE_N * 128) + (uint32_t)r * 128 +
                                ((uint32_t)((ch & 7) ^ (r & 7)) << 4);
          uint32_t a0, a1, a2, a3;
          ldsm_x4(a0, a1, a2, a3, addr);
          if (ks & 1) mma16816r<BF16>(s2[mt], a0, a1, a2, a3, qb[ks][0], qb[ks][1]);
          else mma16816r<BF16>(s[mt], a0, a1, a2, a3, qb[ks][0], qb[ks][1]);
        }
      }
    } else {
#pragma unroll
      for (int cp = 0; cp < NDT / 2; ++cp) {
#pragma unroll
        for (int mt = 0; mt < NMT; ++mt) {
          const int r = mt * 16 + k_row;
          const int ch = 2 * cp + k_chunk;
          const uint32_t addr = kbase + kv8_off(r, ch);
          uint32_t x0, x1, x2, x3;  // (keys lo, ch) (keys hi, ch) (keys lo, ch+1) (keys hi, ch+1)
          ldsm_x4(x0, x1, x2, x3, addr);
          uint32_t a0, a1, a2, a3;
          e4m3x4_to_f16x4(x0, a0, a2);
          e4m3x4_to_f16x4(x1, a1, a3);
          mma16816r<false>(s[mt], a0, a1, a2, a3, qb[2 * cp][0], qb[2 * cp][1]);
          e4m3x4_to_f16x4(x2, a0, a2);
          e4m3x4_to_f16x4(x3, a1, a3);
          mma16816r<false>(s2[mt], a0, a1, a2, a3, qb[2 * cp + 1][0], qb[2 * cp + 1][1]);
        }
      }
    }
#pragma unroll
    for (int mt = 0; mt < NMT; ++mt) {
      s[mt][0] += s2[mt][0]; s[mt][1] += s2[mt][1]; s[mt][2] += s2[mt][2]; s[mt][3] += s2[mt][3];
    }
    // s[mt] = { (key 16mt+g, q 2c), (key 16mt+g, q 2c+1), (key 16mt+g+8, q 2c), (key 16mt+g+8, q 2c+1) }

    // ---- mask (only tiles that touch a boundary)
    const int key_last = key0 + TILE_N - 1;
    const int min_lim = (p.causal || p.window_left >= 0) ? cc.L - cc.sq : cc.L - 1;
    if (key_last > min_lim || (p.window_left >= 0 && key0 < cc.L - 1 - p.window_left)) {
      const int lo0 = p.window_left >= 0 ? lim0 - p.window_left : 0;
      const int lo1 = p.window_left >= 0 ? lim1 - p.window_left : 0;
#pragma unroll
      for (int mt = 0; mt < NMT; ++mt) {
        const int ka = key0 + mt * 16 + g8, kb = ka + 8;
        if (ka > lim0 || ka < lo0) s[mt][0] = -INFINITY;
        if (ka > lim1 || ka < lo1) s[mt][1] = -INFINITY;
        if (kb > lim0 || kb < lo0) s[mt][2] = -INFINITY;
        if (kb > lim1 || kb < lo1) s[mt][3] = -INFINITY;
      }
    }

    // ---- online softmax over keys: keys run along g8 (and the m-tiles), so the row max
    // needs a reduction over lane bits 2..4
    float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
    for (int mt = 0; mt < NMT; ++mt) {
      t0 = fmaxf(t0, fmaxf(s[mt][0], s[mt][2]));
      t1 = fmaxf(t1, fmaxf(s[mt][1], s[mt][3]));
    }
#pragma unroll
    for (int d = 4; d < 32; d <<= 1) {
      t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, d));
      t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, d));
    }
    const float mn0 = fmaxf(m0, t0), mn1 = fmaxf(m1, t1);
    if (__any_sync(0xffffffffu, mn0 > m0 || mn1 > m1)) {
      const float c0 = (m0 == -INFINITY) ? 0.f : ex2((m0 - mn0) * sl2);
      const float c1 = (m1 == -INFINITY) ? 0.f : ex2((m1 - mn1) * sl2);
      l0 *= c0;
      l1 *= c1;
#pragma unroll
      for (int i = 0; i < NDT; ++i) {
        o[i][0] *= c0; o[i][1] *= c1; o[i][2] *= c0; o[i][3] *= c1;
      }
      m0 = mn0;
      m1 = mn1;
    }
    const float ms0 = (m0 == -INFINITY) ? 0.f : m0 * sl2;
    const float ms1 = (m1 == -INFINITY) ? 0.f : m1 * sl2;
    uint32_t pb[NMT][2];  // P^T B fragments per 16-key block
#pragma unroll
    for (int mt = 0; mt < NMT; ++mt) {
      const float p0 = ex2(fmaf(s[mt][0], sl2, -ms0));
      const float p1 = ex2(fmaf(s[mt][1], sl2, -ms1));
      const float p2 = ex2(fmaf(s[mt][2], sl2, -ms0));
      const float p3 = ex2(fmaf(s[mt][3], sl2, -ms1));
      l0 += p0 + p2;
      l1 += p1 + p3;
      pb[mt][0] = movmatrix_trans(pack2<BF16>(p0, p1));  // (keys 16mt+2c, +1 ; q g)
      pb[mt][1] = movmatrix_trans(pack2<BF16>(p2, p3));  // (keys 16mt+8+2c, +1 ; q g)
    }

    // ---- O^T += V^T P^T.  Rows of V past the sequence end may hold anything (NaN bit
    // patterns included): they are zeroed in the one tile that has them.
    auto pv = [&](auto masked_tag) {
      constexpr bool MASKED = decltype(masked_tag)::value;
#pragma unroll
      for (int mt = 0; mt < NMT; ++mt) {
        uint32_t mk_lo = 0xffffffffu, mk_hi = 0xffffffffu;
        if constexpr (MASKED) {
          const int kv_left = cc.L - (key0 + 16 * mt);
          mk_lo = (2 * c4 < kv_left ? 0x0000ffffu : 0u) | (2 * c4 + 1 < kv_left ? 0xffff0000u : 0u);
          mk_hi = (2 * c4 + 8 < kv_left ? 0x0000ffffu : 0u) | (2 * c4 + 9 < kv_left ? 0xffff0000u : 0u);
        }
        const int row = mt * 16 + v_row;
        if constexpr (KVB == 2) {
#pragma unroll
          for (int dt = 0; dt < NDT; ++dt) {
            const int ch = 2 * dt + v_chunk;
            const uint32_t addr = vbase + (uint32_t)(ch >> 3) * (TILE_N * 128) + (uint32_t)row * 128 +
                                  ((uint32_t)((ch & 7) ^ (row & 7)) << 4);
            uint32_t a0, a1, a2, a3;  // (keys lo, d lo) (keys lo, d hi) (keys hi, d lo) (keys hi, d hi)
            ldsm_x4_t(a0, a1, a2, a3, addr);
            if constexpr (MASKED) { a0 &= mk_lo; a1 &= mk_lo; a2 &= mk_hi; a3 &= mk_hi; }
            mma16816r<BF16>(o[dt], a0, a1, a2, a3, pb[mt][0], pb[mt][1]);
          }
        } else {
#pragma unroll
          for (int cp = 0; cp < NDT / 2; ++cp) {
            const int ch = 2 * cp + v_chunk;
            const uint32_t addr = vbase + kv8_off(row, ch);
            uint32_t x0, x1, x2, x3;  // (keys lo, ch) (keys hi, ch) (keys lo, ch+1) (keys hi, ch+1)
            ldsm_x4_t(x0, x1, x2, x3, addr);
            if constexpr (MASKED) { x0 &= mk_lo; x1 &= mk_hi; x2 &= mk_lo; x3 &= mk_hi; }
            // word = [key 2c: d, d+1 | key 2c+1: d, d+1]  ->  [d: key 2c, 2c+1 | d+1: key 2c, 2c+1]
            x0 = __byte_perm(x0, 0, 0x3120);
            x1 = __byte_perm(x1, 0, 0x3120);
            x2 = __byte_perm(x2, 0, 0x3120);
            x3 = __byte_perm(x3, 0, 0x3120);
            uint32_t a0, a1, a2, a3;
            e4m3x4_to_f16x4(x0, a0, a1);  // row g: d = 16ch + 2g ; row g+8: d = 16ch + 2g + 1 (keys lo)
            e4m3x4_to_f16x4(x1, a2, a3);  // same rows, keys hi
            mma16816r<false>(o[2 * cp], a0, a1, a2, a3, pb[mt][0], pb[mt][1]);
            e4m3x4_to_f16x4(x2, a0, a1);
            e4m3x4_to_f16x4(x3, a2, a3);
            mma16816r<false>(o[2 * cp + 1], a0, a1, a2, a3, pb[mt][0], pb[mt][1]);
          }
        }
      }
    };
    if (key0 + TILE_N > cc.L) pv(std::true_type{});
    else pv(std::false_type{});

    // ---- this stage has been read: refill it with the tile NS ahead
    __syncwarp();
    if (prod.more()) {
      fence_proxy_async();
      prod.issue(stage);
    }

    // ---- end of this warp's piece of the segment?
    const bool seg_end = cc.t == cc.nt - 1;
    if (seg_end || it == my_tiles - 1) {
#pragma unroll
      for (int d = 4; d < 32; d <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, d);
        l1 += __shfl_xor_sync(0xffffffffu, l1, d);
      }
      const bool whole = seg_end && (g - piece_start == cc.nt - 1);
      const int nrows = p.group * cc.sq;
      const int q0 = mb * kDecodeRows + 2 * c4, q1 = q0 + 1;
      const bool v0 = q0 < nrows, v1 = q1 < nrows;
      // element (slice i, half e) of this thread is d = dbase(i) + e * dstep
      constexpr int dstep = KVB == 2 ? 8 : 1;
      if (whole) {
        const float i0 = l0 > 0.f ? vscale / l0 : 0.f;
        const float i1 = l1 > 0.f ? vscale / l1 : 0.f;
        const int qrow_base = cc.qr;
        const int hq0 = h * p.group + q0 % p.group, hq1 = h * p.group + q1 % p.group;
        const int64_t ob = (int64_t)cc.b * p.o_bs;
        char* out0 = p.out + 2 * (ob + (int64_t)(qrow_base + q0 / p.group) * p.o_rs + (int64_t)hq0 * p.o_hs);
        char* out1 = p.out + 2 * (ob + (int64_t)(qrow_base + q1 / p.group) * p.o_rs + (int64_t)hq1 * p.o_hs);
        const bool obf = KVB == 2 ? BF16 : (p.q_is_bf16 != 0);
        constexpr float kLn2 = 0.6931471805599453f;
        float lse0 = l0 > 0.f ? m0 * sl2 * kLn2 + logf(l0) : -INFINITY;
        float lse1 = l1 > 0.f ? m1 * sl2 * kLn2 + logf(l1) : -INFINITY;
        {
#pragma unroll
          for (int i = 0; i < NDT; ++i) {
            int d = KVB == 2 ? 16 * i + g8 : 16 * i + 2 * g8;
            bool w0 = v0, w1 = v1;
            if constexpr (PACKED) {   // a column owns the slice of its KV head (both columns of a thread: the same pack)
              const int per = p.group / p.head_pack, sl = (16 * i) / p.real_hd;
              w0 = v0 && (q0 % p.group) / per == sl;
              w1 = v1 && (q1 % p.group) / per == sl;
              d -= sl * p.real_hd;
            }
            const float a0 = o[i][0] * i0, a2 = o[i][2] * i0, b1 = o[i][1] * i1, b3 = o[i][3] * i1;
            if constexpr (KVB == 2) {
              if (w0) {
                *reinterpret_cast<uint16_t*>(out0 + 2 * d) = (uint16_t)(pack2<BF16>(a0, 0.f) & 0xffffu);
                *reinterpret_cast<uint16_t*>(out0 + 2 * (d + dstep)) = (uint16_t)(pack2<BF16>(a2, 0.f) & 0xffffu);
              }
              if (w1) {
                *reinterpret_cast<uint16_t*>(out1 + 2 * d) = (uint16_t)(pack2<BF16>(b1, 0.f) & 0xffffu);
                *reinterpret_cast<uint16_t*>(out1 + 2 * (d + dstep)) = (uint16_t)(pack2<BF16>(b3, 0.f) & 0xffffu);
              }
            } else {
              if (w0) *reinterpret_cast<uint32_t*>(out0 + 2 * d) = obf ? pack2<true>(a0, a2) : pack2<false>(a0, a2);
              if (w1) *reinterpret_cast<uint32_t*>(out1 + 2 * d) = obf ? pack2<true>(b1, b3) : pack2<false>(b1, b3);
            }
          }
        }
        if (p.lse && g8 == 0) {
          if (v0) p.lse[(int64_t)cc.b * p.lse_bs + (int64_t)hq0 * p.lse_hs + qrow_base + q0 / p.group] = lse0;
          if (v1) p.lse[(int64_t)cc.b * p.lse_bs + (int64_t)hq1 * p.lse_hs + qrow_base + q1 / p.group] = lse1;
        }
      } else {
        const int64_t slot = (int64_t)(cc.segbase + cc.seg) + w;
        float* po = p.part_o + slot * (kRowsPerSeg * HD);
        float* pml = p.part_ml + slot * (kRowsPerSeg * 2);
        const int rl0 = 2 * c4, rl1 = rl0 + 1;  // row inside the segment
        // (rows past the segment's end are neither written here nor read by the merge)
        const int nrows_seg = p.group * cc.sq - mb * kDecodeRows;
        const bool wv0 = rl0 < nrows_seg, wv1 = rl1 < nrows_seg;
        if (g8 == 0) {
          if (wv0) *reinterpret_cast<float2*>(pml + rl0 * 2) = make_float2((m0 == -INFINITY) ? -INFINITY : m0 * sl2, l0);
          if (wv1) *reinterpret_cast<float2*>(pml + rl1 * 2) = make_float2((m1 == -INFINITY) ? -INFINITY : m1 * sl2, l1);
        }
#pragma unroll
        for (int i = 0; i < NDT; ++i) {
          const int d = KVB == 2 ? 16 * i + g8 : 16 * i + 2 * g8;
          if constexpr (KVB == 2) {
            if (wv0) {
              po[rl0 * HD + d] = o[i][0];
              po[rl0 * HD + d + dstep] = o[i][2];
            }
            if (wv1) {
              po[rl1 * HD + d] = o[i][1];
              po[rl1 * HD + d + dstep] = o[i][3];
            }
          } else {
            if (wv0) *reinterpret_cast<float2*>(po + rl0 * HD + d) = make_float2(o[i][0], o[i][2]);
            if (wv1) *reinterpret_cast<float2*>(po + rl1 * HD + d) = make_float2(o[i][1], o[i][3]);
          }
        }
      }
      fresh = true;
    }
    if (it + 1 < my_tiles) cursor_advance(p, plan, cc);
  }
}

// ---------------------------------------------------------------------------
// Merge.  A segment that lies inside one warp's tile range was normalised and written by the
// attention kernel.  Only a segment cut by a range boundary left partials, so the blocks stride
// over the W - 1 boundaries, not over the segments: boundary w (the first tile of worker w) takes
// part when it falls strictly inside a segment, and ALL the boundaries that cut one segment share
// its work items (4 consecutive d of one query row each) -- a batch of a few long sequences has
// few segments, each cut by a hundred boundaries, and must not be merged by a handful of blocks.
// A second loop zero-fills the rows of sequences without visible keys.
// ---------------------------------------------------------------------------
constexpr int kMergeCoopParts = 32;   // from this many partials per segment on, a warp shares an item

template <int HD>
__global__ void __launch_bounds__(128) attn_merge_kernel(const AttnParams p) {
  pdl_wait();
  pdl_launch_dependents();
  const long long total = p.tile_cum[p.batch];
  constexpr float kLn2 = 0.6931471805599453f;
  constexpr int kQuads = HD / 4;
  const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
  // x * n_workers / total and w * total / n_workers: 32-bit divisions whenever the products fit (a 64-bit division
  // is a call of a hundred instructions, and every block has a chain of them before its first load)
  const bool narrow = total * p.n_workers < (1ll << 31);
  auto muldiv = [&](long long a, long long b, long long c) -> long long {
    return narrow ? (long long)((uint32_t)(a * b) / (uint32_t)c) : a * b / c;
  };
  if (total > 0) {
    for (int w = blockIdx.x + 1; w < p.n_workers; w += gridDim.x) {
      const long long g = muldiv(w, total, p.n_workers);
      if (g <= 0 || g >= total) continue;
      // where tile g lies: the record the worker that starts there left (no search, one load)
      const int4* rec = reinterpret_cast<const int4*>(p.bound_rec + 8 * (size_t)w);
      const int4 ra = rec[0], rb = rec[1];
      Cursor c;
      c.b = ra.x; c.seg = ra.y; c.t = ra.z; c.nt = ra.w;
      c.sq = rb.x; c.qr = rb.y; c.segbase = rb.z; c.nmb = rb.w;
      if (c.t == 0) continue;       // the boundary coincides with the segment's first tile: not a cut
      const long long t0 = g - c.t, t1 = t0 + c.nt;   // the segment's tiles
      const int seg = c.segbase + c.seg;
      // workers wf .. wl hold the segment's tiles; the boundaries wf + 1 .. wl cut it, this one is number k of nb
      const int wf = narrow ? (int)(((uint32_t)(t0 + 1) * (uint32_t)p.n_workers - 1u) / (uint32_t)total)
                            : (int)(((t0 + 1) * p.n_workers - 1) / total);
      const int wl = narrow ? (int)(((uint32_t)t1 * (uint32_t)p.n_workers - 1u) / (uint32_t)total)
                            : (int)((t1 * p.n_workers - 1) / total);
      const int nb = wl - wf, k = w - wf - 1;
      const int b = c.b, sq = c.sq;
      const int h = c.seg / c.nmb, mb = c.seg - h * c.nmb;
      const int nrows = p.group * sq;
      const float vscale = p.vs_vec ? p.vs_vec[h] : p.vs;
      const int qr = c.qr;
      // A worker between wf and wl whose range is empty (fewer tiles than workers) wrote nothing.
      const bool all_have = total >= p.n_workers;
      auto has_tiles = [&](int wi) {
        return all_have || muldiv(wi, total, p.n_workers) < muldiv(wi + 1, total, p.n_workers);
      };
      auto ml_of = [&](int wi, int sub, int r16) {
        return p.part_ml + (((int64_t)seg + wi) * p.seg_blocks + sub) * (kRowsPerSeg * 2) + r16 * 2;
      };
      auto o_of = [&](int wi, int sub, int r16, int d) {
        return p.part_o + (((int64_t)seg + wi) * p.seg_blocks + sub) * (kRowsPerSeg * HD) + r16 * HD + d;
      };
      const int n_items = p.rows_per_seg * kQuads;
      // Few partials: one thread per item.  Many: one warp per item (the item is then uniform over the warp), its
      // lanes striding over the partials.  One loop serves both: the kernel is a chain of latencies, and a second
      // copy of the loop body costs more in instruction fetches than it saves.
      const bool coop = nb + 1 >= kMergeCoopParts;
      const int item_step = coop ? nb * 4 : nb * 128;
      const int wi0 = coop ? wf + lane : wf, wi_step = coop ? 32 : 1;
      for (int item = coop ? k * 4 + wp : k * 128 + threadIdx.x; item < n_items; item += item_step) {
        const int rl = item / kQuads, d = (item - rl * kQuads) * 4;
        const int row = mb * p.rows_per_seg + rl;
        if (row >= nrows) continue;
        int d_out = d;
        if (p.head_pack > 1) {   // packed heads: a row owns the slice of its own KV head
          const int sl = (row % p.group) / (p.group / p.head_pack);
          if (d / p.real_hd != sl) continue;
          d_out = d - sl * p.real_hd;
        }
        const int sub = rl >> 4, r16 = rl & 15;   // 16-row slot of the row (32-row segments have two per worker)
        float M = -INFINITY;
        for (int wi = wi0; wi <= wl; wi += wi_step)   // (not unrolled: measured slower, the kernel is a chain of fetches)
          if (has_tiles(wi)) M = fmaxf(M, *ml_of(wi, sub, r16));
        if (coop) {
#pragma unroll
          for (int s = 16; s > 0; s >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, s));
        }
        float L = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (M != -INFINITY) {
          for (int wi = wi0; wi <= wl; wi += wi_step) {   // the partial loads of an item are independent
            if (!has_tiles(wi)) continue;
            const float2 ml = *reinterpret_cast<const float2*>(ml_of(wi, sub, r16));
            if (ml.x == -INFINITY) continue;
            const float wgt = ex2(ml.x - M);
            const float4 o = *reinterpret_cast<const float4*>(o_of(wi, sub, r16, d));
            L += wgt * ml.y;
            acc.x += wgt * o.x; acc.y += wgt * o.y; acc.z += wgt * o.z; acc.w += wgt * o.w;
          }
        }
        if (coop) {
#pragma unroll
          for (int s = 16; s > 0; s >>= 1) {
            L += __shfl_xor_sync(0xffffffffu, L, s);
            acc.x += __shfl_xor_sync(0xffffffffu, acc.x, s);
            acc.y += __shfl_xor_sync(0xffffffffu, acc.y, s);
            acc.z += __shfl_xor_sync(0xffffffffu, acc.z, s);
            acc.w += __shfl_xor_sync(0xffffffffu, acc.w, s);
          }
          if (lane != 0) continue;
        }
        const float inv = L > 0.f ? vscale / L : 0.f;
        const int j = row / p.group, hq = h * p.group + row % p.group;
        const float4 r = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        const int64_t oi = (int64_t)b * p.o_bs + (int64_t)(qr + j) * p.o_rs + (int64_t)hq * p.o_hs + d_out;
        uint2 packed;
        if (p.q_is_bf16) packed = make_uint2(pack2<true>(r.x, r.y), pack2<true>(r.z, r.w));
        else packed = make_uint2(pack2<false>(r.x, r.y), pack2<false>(r.z, r.w));
        *reinterpret_cast<uint2*>(p.out + 2 * oi) = packed;
        if (p.lse && d_out == 0)
          p.lse[(int64_t)b * p.lse_bs + (int64_t)hq * p.lse_hs + qr + j] = L > 0.f ? M * kLn2 + logf(L) : -INFINITY;
      }
    }
  }
  // sequences with query rows but no visible keys: zeros
  for (int b = blockIdx.x; b < p.batch; b += gridDim.x) {
    const int sq = p.sq[b];
    if (p.nt[b] > 0 || sq <= 0) continue;
    const int qr = p.qrow0[b];
    const int zq = (p.head_pack > 1 ? p.real_hd : HD) / 4;   // (a query head's row has real_hd elements with packed heads too)
    const int items = sq * p.hq * zq;
    for (int item = threadIdx.x; item < items; item += 128) {
      const int d = (item % zq) * 4, rh = item / zq;
      const int hq = rh % p.hq, j = rh / p.hq;
      const int64_t oi = (int64_t)b * p.o_bs + (int64_t)(qr + j) * p.o_rs + (int64_t)hq * p.o_hs + d;
      *reinterpret_cast<uint2*>(p.out + 2 * oi) = make_uint2(0u, 0u);   // +0.0 in either 16-bit type
      if (p.lse && d == 0) p.lse[(int64_t)b * p.lse_bs + (int64_t)hq * p.lse_hs + qr + j] = -INFINITY;
    }
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

struct TmapKey {
  const void* base;
  int64_t page_stride, token_stride, head_stride, n_pages;
  int32_t page_size, hkv, hd, dtype, device;
  int32_t box_rows = 0;   // filled in by get_pool_tmap
  int32_t merged = 0;     // 5-D map whose box spans both 128-byte halves of a 256-byte row
  bool operator==(const TmapKey& o) const {
    return box_rows == o.box_rows && merged == o.merged && base == o.base && page_stride == o.page_stride && token_stride == o.token_stride &&
           head_stride == o.head_stride && n_pages == o.n_pages && page_size == o.page_size &&
           hkv == o.hkv && hd == o.hd && dtype == o.dtype && device == o.device;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = std::hash<const void*>()(k.base);
    auto mix = [&](uint64_t v) { h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2); };
    mix((uint64_t)k.page_stride); mix((uint64_t)k.token_stride); mix((uint64_t)k.head_stride);
    mix((uint64_t)k.n_pages); mix((uint64_t)k.page_size); mix((uint64_t)k.hkv); mix((uint64_t)k.hd);
    mix((uint64_t)k.dtype); mix((uint64_t)k.device); mix((uint64_t)k.box_rows); mix((uint64_t)k.merged);
    return h;
  }
};

// One tensor map per pool view: dims (innermost first) D, P, H_kv, n_pages;
// box = (128 bytes of D, min(P, TILE_N) tokens, 1 head, 1 page), 128-byte swizzle.
inline int get_pool_tmap(const TmapKey& key_in, int tile_n, bool merged, CUtensorMap* out) {
  TmapKey key = key_in;
  key.box_rows = key.page_size < tile_n ? key.page_size : tile_n;
  key.merged = merged ? 1 : 0;
  static std::mutex mu;
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  {
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return KB200_OK; }
  }
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return fail(KB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const int es = dtype_size(key.dtype);
  const int row_bytes = key.hd * es;
  const int rb = row_bytes > 128 ? 128 : row_bytes;
  const int box_rows = key.box_rows;
  cuuint64_t dims[4] = {(cuuint64_t)key.hd, (cuuint64_t)key.page_size, (cuuint64_t)key.hkv, (cuuint64_t)key.n_pages};
  cuuint64_t strides[3] = {(cuuint64_t)(key.token_stride * es), (cuuint64_t)(key.head_stride * es),
                           (cuuint64_t)(key.page_stride * es)};
  cuuint32_t box[4] = {(cuuint32_t)(rb / es), (cuuint32_t)box_rows, 1u, 1u};
  cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  CUtensorMapDataType dt = key.dtype == KB200_DTYPE_E4M3 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                           : key.dtype == KB200_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                           : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMapSwizzle sw = rb == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                          : rb == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
  CUtensorMap tm;
  CUresult r;
  if (merged) {
    // a 256-byte row as two 128-byte halves: dims 64 elements, token, half (stride 128 bytes), head, page
    cuuint64_t dims5[5] = {64u, (cuuint64_t)key.page_size, 2u, (cuuint64_t)key.hkv, (cuuint64_t)key.n_pages};
    cuuint64_t strides5[4] = {(cuuint64_t)(key.token_stride * es), 128u, (cuuint64_t)(key.head_stride * es),
                              (cuuint64_t)(key.page_stride * es)};
    cuuint32_t box5[5] = {64u, (cuuint32_t)box_rows, 2u, 1u, 1u};
    cuuint32_t estr5[5] = {1u, 1u, 1u, 1u, 1u};
    r = enc(&tm, dt, 5, const_cast<void*>(key.base), dims5, strides5, box5, estr5, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    r = enc(&tm, dt, 4, const_cast<void*>(key.base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) return fail(KB200_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  {
    std::lock_guard<std::mutex> lk(mu);
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, tm);
  }
  *out = tm;
  return KB200_OK;
}

struct DeviceInfo { int sms = 0; };
inline DeviceInfo& device_info(int dev) {
  static DeviceInfo info[64];
  return info[dev & 63];
}

inline int tile_n_for(int kv_dtype, int head_dim, int nw) {
  const int raw = kAttnStageBytes(nw) / (2 * head_dim * dtype_size(kv_dtype));
  return raw > 64 ? 64 : raw;
}

// Worker warps per CTA: 8 (16-bit K/V on the 16-row kernel: HBM-bound with 2 stages of 8 KB per warp) or 12
// (e4m3 K/V, and the transposed decode kernel: more warps to hide the MMA / conversion latencies); chosen in
// launch_attention_pass.  One warp per scheduler (4 warps, 16 KB stages) cannot hide its own latencies.
struct AttnWorkspace {
  size_t tile_cum, seg_cum, nt, tile0, sq, qrow0, klen, bound_rec, part_ml, part_o, total;
};

inline int64_t attn_max_segments(int64_t batch, int64_t total_q, int hq, int hkv) {
  const int group = hq / hkv;
  // sum over sequences of ceil(group * sq_b / 16) <= group * total_q / 16 + batch
  return (int64_t)hkv * ((group * total_q + kDecodeRows - 1) / kDecodeRows + batch);  // smallest segment size
}

// rows32: the call runs the 32-row kernel, whose (segment, worker) partials take two 16-row slots each.
inline AttnWorkspace attn_workspace_layout(int64_t batch, int64_t total_q, int hq, int hkv, int hd, int n_workers,
                                           bool rows32) {
  auto up = [](size_t x) { return (x + 255) & ~size_t(255); };
  AttnWorkspace w;
  size_t off = 0;
  w.tile_cum = off; off = up(off + sizeof(long long) * (batch + 1));
  w.seg_cum = off; off = up(off + sizeof(int) * (batch + 1));
  w.nt = off; off = up(off + sizeof(int) * batch);
  w.tile0 = off; off = up(off + sizeof(int) * batch);
  w.sq = off; off = up(off + sizeof(int) * batch);
  w.qrow0 = off; off = up(off + sizeof(int) * batch);
  w.klen = off; off = up(off + sizeof(int) * batch);
  // 16-row kernel: slot = segment + worker.  32-row kernel: slot = 2 * (segment + worker) + block, with at most
  // hkv * (group * total_q / 32 + batch) segments: twice that is within attn_max_segments + hkv * batch.
  const int64_t slots = attn_max_segments(batch, total_q, hq, hkv) + (rows32 ? hkv * batch + 2 * (int64_t)n_workers : n_workers);
  w.part_ml = off; off = up(off + sizeof(float) * slots * kRowsPerSeg * 2);
  w.part_o = off; off = up(off + sizeof(float) * slots * kRowsPerSeg * hd);
  w.bound_rec = off; off = up(off + sizeof(int) * 8 * n_workers);   // (split-KV kernels only, like the partials)
  w.total = off;
  return w;
}

inline int device_sm_count(int dev, int* sms) {
  DeviceInfo& di = device_info(dev);
  if (di.sms == 0) {
    int n = 0;
    KB200_CUDA_OK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    di.sms = n;
  }
  *sms = di.sms;
  return KB200_OK;
}

template <int KVB, int HD, bool BF16, int NW, int NS, bool GATHER>
inline int launch_attn_variant(const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p, int grid,
                               int dev, cudaStream_t stream) {
  using T = AttnTile<KVB, HD, NW, NS>;
  auto kern = paged_attn_kernel<KVB, HD, BF16, NW, NS, GATHER>;
  static SmemAttrOnce once;
  static_assert(T::SMEM_BYTES + plan_smem_bytes(kPlanSmemMaxBatch) <= 232448, "shared memory of the largest in-kernel plan");
  if (int rc = once.ensure(kern, T::SMEM_BYTES + plan_smem_bytes(kPlanSmemMaxBatch), dev)) return rc;
  const size_t smem = T::SMEM_BYTES + (p.plan_in_kernel ? plan_smem_bytes(p.batch) : 0);
  KB200_CUDA_OK(launch_kernel(kern, dim3(grid), dim3(NW * 32), smem, stream, tmK, tmV, p));
  return KB200_OK;
}

template <int KVB, int HD, bool BF16, int NW, int NS, bool GATHER>
inline int launch_decode_variant(const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p, int grid,
                                 int dev, cudaStream_t stream) {
  using T = AttnTile<KVB, HD, NW, NS>;
  auto kern = paged_attn_decode_kernel<KVB, HD, BF16, NW, NS, GATHER>;
  static SmemAttrOnce once;
  static_assert(T::SMEM_BYTES + plan_smem_bytes(kPlanSmemMaxBatch) <= 232448, "shared memory of the largest in-kernel plan");
  if (int rc = once.ensure(kern, T::SMEM_BYTES + plan_smem_bytes(kPlanSmemMaxBatch), dev)) return rc;
  const size_t smem = T::SMEM_BYTES + (p.plan_in_kernel ? plan_smem_bytes(p.batch) : 0);
  KB200_CUDA_OK(launch_kernel(kern, dim3(grid), dim3(NW * 32), smem, stream, tmK, tmV, p));
  return KB200_OK;
}

template <int KVB, int HD, bool BF16, bool GATHER>
inline int launch_rows32_variant(const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p, int grid,
                                 int dev, cudaStream_t stream) {
  using L = Rows32Smem<KVB, HD, 2>;
  auto kern = paged_attn_rows32_kernel<KVB, HD, BF16, 2, GATHER>;
  static SmemAttrOnce once;
  static_assert(L::SMEM_BYTES + plan_smem_bytes(kPlanSmemMaxBatch) <= 232448, "shared memory of the largest in-kernel plan");
  if (int rc = once.ensure(kern, L::SMEM_BYTES + plan_smem_bytes(kPlanSmemMaxBatch), dev)) return rc;
  const size_t smem = L::SMEM_BYTES + (p.plan_in_kernel ? plan_smem_bytes(p.batch) : 0);
  KB200_CUDA_OK(launch_kernel(kern, dim3(grid), dim3(256), smem, stream, tmK, tmV, p));
  return KB200_OK;
}

template <int KVB, bool BF16>
inline int launch_rows32_dispatch(bool d128, const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p,
                                  int grid, int dev, cudaStream_t stream) {
  if (d128) return p.gather ? launch_rows32_variant<KVB, 128, BF16, true>(tmK, tmV, p, grid, dev, stream)
                            : launch_rows32_variant<KVB, 128, BF16, false>(tmK, tmV, p, grid, dev, stream);
  return p.gather ? launch_rows32_variant<KVB, 64, BF16, true>(tmK, tmV, p, grid, dev, stream)
                  : launch_rows32_variant<KVB, 64, BF16, false>(tmK, tmV, p, grid, dev, stream);
}

template <int KVB, bool BF16, int HD>
inline int launch_decode_hd(int nw, const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p, int grid,
                            int dev, cudaStream_t stream) {
  (void)nw;   // the transposed kernel runs 12 warps
  if (p.gather) return launch_decode_variant<KVB, HD, BF16, 12, 2, true>(tmK, tmV, p, grid, dev, stream);
  return launch_decode_variant<KVB, HD, BF16, 12, 2, false>(tmK, tmV, p, grid, dev, stream);
}

template <int KVB, bool BF16>
inline int launch_decode_dispatch(bool d128, int nw, const CUtensorMap& tmK, const CUtensorMap& tmV,
                                  const AttnParams& p, int grid, int dev, cudaStream_t stream) {
  return d128 ? launch_decode_hd<KVB, BF16, 128>(nw, tmK, tmV, p, grid, dev, stream)
              : launch_decode_hd<KVB, BF16, 64>(nw, tmK, tmV, p, grid, dev, stream);
}

template <int KVB, bool BF16, int HD>
inline int launch_attn_hd(int nw, const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p, int grid,
                          int dev, cudaStream_t stream) {
  (void)nw;   // 12 warps for e4m3 K/V, 8 for 16-bit
  if constexpr (KVB == 1) {
    if (p.gather) return launch_attn_variant<KVB, HD, BF16, 12, 2, true>(tmK, tmV, p, grid, dev, stream);
    return launch_attn_variant<KVB, HD, BF16, 12, 2, false>(tmK, tmV, p, grid, dev, stream);
  } else {
    if (p.gather) return launch_attn_variant<KVB, HD, BF16, 8, 2, true>(tmK, tmV, p, grid, dev, stream);
    return launch_attn_variant<KVB, HD, BF16, 8, 2, false>(tmK, tmV, p, grid, dev, stream);
  }
}

template <int KVB, bool BF16>
inline int launch_attn_dispatch(bool d128, int nw, const CUtensorMap& tmK, const CUtensorMap& tmV,
                                const AttnParams& p, int grid, int dev, cudaStream_t stream) {
  return d128 ? launch_attn_hd<KVB, BF16, 128>(nw, tmK, tmV, p, grid, dev, stream)
              : launch_attn_hd<KVB, BF16, 64>(nw, tmK, tmV, p, grid, dev, stream);
}

// paged_prefill.cuh
bool prefill_enabled();
template <int HD, bool BF16, bool KV8>
int launch_prefill_variant(const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p, int grid, int dev,
                           cudaStream_t stream);
constexpr int kPrefillRowsPerSeg = 256, kPrefillTileKeys = 128, kPrefillMinPackedRows = 64;
// Packed query rows per sequence (per KV head) from which the prefill kernel serves a call.  Below, the split-KV
// kernels read a sequence's keys once per 32 rows and balance any mix of lengths over all SMs; the prefill kernel
// reads them once per 256 rows, but one CTA walks all keys of its rows and pays a fixed cost per CTA.  Measured
// per call, prefill | split-KV (32/8 heads unless noted; U[a, b] = context lengths):
//   16-bit pools, head_dim 128
//     36 rows: 256 x U[2k,16k] 1.46 | 3.28 ms, 64 x U[1k,8k] 0.28 | 0.48, 8 x U[2k,16k] 0.156 | 0.157          -> 33
//     20 .. 32 rows: 256 x U[2k,16k] 1.46 | 1.65, 64 x U[2k,4k] 0.154 | 0.174 .. 0.187, 128 x U[300,1200]
//       0.116 | 0.120 .. 0.139, 32 x U[300,1200] 0.036 | 0.081 .. 0.110, 512 x U[300,1200] 0.420 | 0.388 .. 0.429;
//       16 x U[2k,16k] 0.153 | 0.145, 8 x U[2k,16k] 0.150 | 0.120   -> 17 once there is a CTA (sequence x KV head) per SM
//   16-bit pools, head_dim 64
//     20 .. 32 rows: 512 x U[760,1000] 0.353 | 0.208 .. 0.219, 256 x U[2k,16k] 0.986 | 0.840 .. 0.850
//     48 rows: 512 x U[760,1000] 0.367 | 0.392, 64 x U[2k,16k] 0.318 | 0.427, 256 x U[2k,16k] 1.13 | 1.69;
//       32/32 heads, 64 x U[2k,16k] 1.08 | 1.63                                                                  -> 33
//   e4m3 pools, head_dim 128 (the prefill kernel widens tiles through shared memory)
//     without the key split (more than 128 rows per KV head somewhere in the launch): 64 rows: 256 x U[2k,16k]
//       2.69 | 2.44, 64 x: 0.84 | 0.71, 8 x: 0.33 | 0.14; 128 rows: 2.73 | 4.92, 0.85 | 1.36, 0.33 | 0.19           -> 65
//     with it: 40 rows: 256 x U[2k,16k] 1.77 | 2.39, 16 x: 0.206 | 0.171; 64 rows: 1.78 | 2.44, 0.204 | 0.179;
//       128 rows: 256 x 1.83, 16 x 0.210                            -> 33 once there is a CTA per SM (32 rows and
//       fewer stay with the 32-row kernel, which reads the keys once as well and spreads them over all SMs)
inline int prefill_min_rows(bool kv8) { return kv8 ? 65 : 33; }

// A TMA box must fill a multiple of 128 bytes of shared memory: page_size x min(row bytes, 128).  Pools
// that cannot offer that (page size 1 with 64-byte e4m3 rows) are served by the split-KV kernels' cp.async
// gather path.
inline bool tma_boxes_possible(const kb200_attn_args* a, int tile_n) {
  const int row_bytes = a->head_dim * dtype_size(a->kv_dtype);
  const int rb = row_bytes > 128 ? 128 : row_bytes;
  const int box_rows = a->page_size < tile_n ? a->page_size : tile_n;
  return (box_rows * rb) % 128 == 0;
}

// Which kernel serves a call: many query rows per sequence with 16-bit K/V (or a block mask) go to
// the tensor-memory prefill kernel, one CTA per 256 packed rows, no split over keys and no merge.
inline bool use_prefill_kernel(const kb200_attn_args* a) {
  if (a->q_visible_until != nullptr) return true;
  if (!prefill_enabled() || a->n_kv_heads <= 0) return false;
  if (!tma_boxes_possible(a, kPrefillTileKeys)) return false;   // (the prefill kernel has no gather path)
  // Packed rows: seqlen_q is only an upper bound (the reference's packed call passes none at all,
  // kestrel/ops/attention.py:69-86, and the shim then sets it to total_q); the mean rows per
  // sequence says which kernel has less work.
  int64_t rows = a->seqlen_q;
  if (a->cu_seqlens_q && a->batch > 0) rows = std::min<int64_t>(rows, (a->total_q + a->batch - 1) / a->batch);
  const int64_t packed_rows = (int64_t)(a->n_q_heads / a->n_kv_heads) * rows;
  const bool kv8 = a->kv_dtype == KB200_DTYPE_E4M3;
  if (packed_rows >= prefill_min_rows(kv8)) return true;
  // 17 .. 32 rows (33 .. 64 on e4m3 pools): with a CTA per SM at least, and only when the launch will get the
  // key-split variant (seqlen_q bounds every sequence's rows; a packed call without a bound keeps the 32-row kernel)
  if (a->head_dim == 128 && packed_rows > (kv8 ? 2 * kRowsPerSeg : kRowsPerSeg) &&
      (int64_t)(a->n_q_heads / a->n_kv_heads) * a->seqlen_q <= 128 /* rows of one Q tile */) {
    int sms = 0;
    return device_sm_count(a->device, &sms) == KB200_OK && a->batch * (int64_t)a->n_kv_heads >= sms;
  }
  return false;
}

// Scratch bytes this very call needs: the plan arrays, plus the split-KV partials unless the prefill
// kernel serves it.
// Several KV heads read as one wide head (AttnParams::head_pack): for e4m3 pools with pages of one or two tokens
// whose (token, head) rows have 64 or 128 bytes -- the reference's own FP8 geometry is page size 1, 32 KV heads of 64
// (kestrel/models/moondream/runtime.py:645-663, kestrel/models/moondream/config.py:25-31).  Per head, a tile is
// 64-byte pieces scattered over the pool, one page-table look-up per piece; four heads side by side make 256
// contiguous bytes per look-up.  Needs: one scale per layer (the reference's), heads side by side in the pool,
// at most 8 packed rows for the wide head.  Returns the number of heads per pack (1: none).
inline int attn_head_pack(const kb200_attn_args* a) {
  const bool kv8 = a->kv_dtype == KB200_DTYPE_E4M3;
  if (a->page_size > 2 || (kv8 && (a->k_scale_per_head || a->v_scale_per_head))) return 1;
  if (a->q_visible_until != nullptr || a->n_kv_heads <= 0) return 1;
  // wide rows of 256 bytes: four e4m3 heads of 64, two of 128, or two 16-bit heads of 64 (the reference's default
  // pools: page size 1, kestrel/config.py:164, MHA heads of 64)
  const int pack = kv8 ? (a->head_dim == 64 ? 4 : a->head_dim == 128 ? 2 : 1) : (a->head_dim == 64 ? 2 : 1);
  if (pack == 1 || a->n_kv_heads % pack != 0 || a->kv_head_stride != a->head_dim) return 1;
  if ((int64_t)(a->n_q_heads / a->n_kv_heads) * pack * a->seqlen_q > kDecodeRows) return 1;
  return pack;
}

// Segments of 17 to 32 packed rows (and what is left of longer ones below the prefill kernel's threshold) run the
// 32-row split-KV kernel: one pass over the keys per 32 rows instead of one per 16.
inline bool use_rows32_kernel(const kb200_attn_args* a) {
  if (a->n_kv_heads <= 0 || use_prefill_kernel(a)) return false;
  int64_t rows = a->seqlen_q;
  if (a->cu_seqlens_q && a->batch > 0) rows = std::min<int64_t>(rows, (a->total_q + a->batch - 1) / a->batch);
  return (int64_t)(a->n_q_heads / a->n_kv_heads) * rows > kRowsPerSeg;
}

inline uint64_t attn_pass_workspace_need(const kb200_attn_args* a, int sms) {
  const int pack = use_prefill_kernel(a) ? 1 : attn_head_pack(a);
  const AttnWorkspace wl = attn_workspace_layout(a->batch, a->total_q, a->n_q_heads, a->n_kv_heads / pack,
                                                 a->head_dim * pack, sms * kAttnMaxWarps, use_rows32_kernel(a));
  return use_prefill_kernel(a) ? wl.part_ml : wl.total;
}

// ---------------------------------------------------------------------------
// Shared cached prefix: the batch's common leading pages are read once.
//   pass 1  all B * Sq query rows as one sequence over the prefix keys, no mask (tensor-memory
//           prefill kernel), output and log-sum-exp into scratch
//   pass 2  every sequence over its remaining keys (page table and lengths shifted), output in
//           place, log-sum-exp into scratch (or the caller's buffer)
//   combine out = (o1 e^{l1} + o2 e^{l2}) / (e^{l1} + e^{l2})
// ---------------------------------------------------------------------------
inline bool shared_prefix_applies(const kb200_attn_args* a) {
  if (a->shared_prefix_pages <= 0) return false;
  if (a->cu_seqlens_q || a->seqused_q || a->window_left >= 0 || a->q_visible_until) return false;
  if (!prefill_enabled() || a->n_kv_heads <= 0 || a->n_q_heads % a->n_kv_heads != 0) return false;
  if ((int64_t)(a->n_q_heads / a->n_kv_heads) * a->batch * a->seqlen_q < kPrefillMinPackedRows) return false;
  if (a->batch * (int64_t)a->seqlen_q > 0x7fffffff / (a->n_q_heads / a->n_kv_heads)) return false;
  if (a->seqlen_q > 1 && a->q_batch_stride != (int64_t)a->seqlen_q * a->q_row_stride) return false;
  if ((int64_t)a->shared_prefix_pages * a->page_size > 0x3fffffff) return false;
  return true;
}

struct SharedPrefixPlan {
  kb200_attn_args pre, rest;   // the two passes
  int n_split, pages_first;    // the prefix pass as 1 or 2 sequences of prefix keys (pages_first: pages of the first)
  size_t o1, lse1, lse2, ws1, ws2, total;   // scratch layout
};

inline SharedPrefixPlan shared_prefix_plan(const kb200_attn_args* a, int sms) {
  auto up = [](size_t x) { return (x + 255) & ~size_t(255); };
  SharedPrefixPlan sp;
  const int64_t rows = a->batch * (int64_t)a->seqlen_q;
  sp.pre = *a;
  sp.pre.shared_prefix_pages = 0;
  sp.pre.batch = 1;
  sp.pre.total_q = rows;
  sp.pre.seqlen_q = (int32_t)rows;
  sp.pre.q_batch_stride = 0;
  sp.pre.q_row_stride = a->seqlen_q > 1 ? a->q_row_stride : a->q_batch_stride;
  sp.pre.o_batch_stride = 0;
  sp.pre.o_row_stride = (int64_t)a->n_q_heads * a->head_dim;
  sp.pre.o_head_stride = a->head_dim;
  sp.pre.seqused_k = nullptr;
  sp.pre.causal = 0;
  // Few CTAs (one per KV head and 256 packed rows): cut the prefix keys in two at a tile boundary and
  // run the halves as two sequences over the same query rows, so twice the SMs work half as long.
  sp.n_split = 1;
  sp.pages_first = a->shared_prefix_pages;
  {
    const int group = a->n_q_heads / a->n_kv_heads;
    const int64_t ctas = (int64_t)a->n_kv_heads * ((group * rows + kPrefillRowsPerSeg - 1) / kPrefillRowsPerSeg);
    const int pages_per_tile = kPrefillTileKeys / a->page_size;   // (0 for pages longer than a tile)
    if (pages_per_tile > 0 && 2 * ctas <= sms && a->shared_prefix_pages >= 4 * pages_per_tile) {
      const int tiles = (a->shared_prefix_pages + pages_per_tile - 1) / pages_per_tile;
      sp.pages_first = ((tiles + 1) / 2) * pages_per_tile;
      sp.n_split = 2;
      sp.pre.batch = 2;
      sp.pre.total_q = 2 * rows;
      sp.pre.pt_row_stride = sp.pages_first;   // the second sequence's row starts where the first one's pages end
      sp.pre.o_batch_stride = rows * a->n_q_heads * a->head_dim;
    }
  }
  sp.rest = *a;
  sp.rest.shared_prefix_pages = 0;
  sp.rest.page_table = a->page_table + a->shared_prefix_pages;
  size_t off = 0;
  sp.o1 = off; off = up(off + (size_t)sp.n_split * rows * a->n_q_heads * a->head_dim * 2);
  sp.lse1 = off; off = up(off + sizeof(float) * sp.n_split * rows * a->n_q_heads);
  sp.lse2 = off; off = up(off + sizeof(float) * rows * a->n_q_heads);
  sp.ws1 = off; off = up(off + attn_pass_workspace_need(&sp.pre, sms));
  sp.ws2 = off; off = up(off + attn_pass_workspace_need(&sp.rest, sms));
  sp.total = off;
  return sp;
}

// Scratch bytes this very call needs: the plan arrays, plus the split-KV partials unless the prefill
// kernel serves it; with a shared prefix, both passes' scratch plus the first pass's output.
inline uint64_t attn_workspace_need(const kb200_attn_args* a, int sms) {
  if (shared_prefix_applies(a)) return shared_prefix_plan(a, sms).total;
  return attn_pass_workspace_need(a, sms);
}

struct CombineParams {
  const char* o1;      // [n_pre][rows, hq, hd] contiguous, q's dtype: the prefix pass (one or two key ranges)
  char* out;           // the remainder pass's output, combined in place
  const float* lse1;   // [n_pre][hq, rows]
  float* lse2;         // [batch, hq, sq]; receives the combined value when write_lse is set
  int64_t o_bs, o_rs, o_hs;
  int64_t rows;
  int sq, hq, hd, q_is_bf16, write_lse, n_pre;
};

// one thread per 8 consecutive elements of one (row, head)
__global__ void __launch_bounds__(256) attn_combine_kernel(const CombineParams c) {
  pdl_wait();
  pdl_launch_dependents();
  const int chunks = c.hd / 8;
  const int64_t total = c.rows * c.hq * chunks;
  const int64_t o1_stride = c.rows * c.hq * c.hd * 2, l1_stride = c.rows * c.hq;   // second key range of the prefix
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int ch = (int)(i % chunks);
    const int64_t rh = i / chunks;
    const int h = (int)(rh % c.hq);
    const int64_t row = rh / c.hq;
    const int64_t b = row / c.sq;
    const int j = (int)(row - b * c.sq);
    const float l1 = c.lse1[(int64_t)h * c.rows + row];
    const float l1b = c.n_pre == 2 ? c.lse1[l1_stride + (int64_t)h * c.rows + row] : -INFINITY;
    float* l2p = c.lse2 + (b * c.hq + h) * c.sq + j;
    const float l2 = *l2p;
    const float m = fmaxf(fmaxf(l1, l1b), l2);
    float w1 = 0.f, w1b = 0.f, w2 = 0.f, lse = -INFINITY;
    if (m != -INFINITY) {
      const float e1 = __expf(l1 - m), e1b = __expf(l1b - m), e2 = __expf(l2 - m);   // exp(-inf) = 0
      const float inv = 1.f / (e1 + e1b + e2);
      w1 = e1 * inv;
      w1b = e1b * inv;
      w2 = e2 * inv;
      lse = m + logf(e1 + e1b + e2);
    }
    const char* src = c.o1 + 2 * ((row * c.hq + h) * c.hd + 8 * ch);
    const uint4 a = *reinterpret_cast<const uint4*>(src);
    const uint4 ab = c.n_pre == 2 ? *reinterpret_cast<const uint4*>(src + o1_stride) : make_uint4(0u, 0u, 0u, 0u);
    char* dst = c.out + 2 * (b * c.o_bs + j * c.o_rs + h * c.o_hs + 8 * ch);
    const uint4 d = *reinterpret_cast<const uint4*>(dst);
    const uint32_t* aw = reinterpret_cast<const uint32_t*>(&a);
    const uint32_t* bw = reinterpret_cast<const uint32_t*>(&ab);
    const uint32_t* dw = reinterpret_cast<const uint32_t*>(&d);
    uint4 r;
    uint32_t* rw = reinterpret_cast<uint32_t*>(&r);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float a0, a1, b0, b1, d0, d1;
      if (c.q_is_bf16) {
        a0 = bf16_bits_to_float(aw[e] & 0xffffu); a1 = bf16_bits_to_float(aw[e] >> 16);
        b0 = bf16_bits_to_float(bw[e] & 0xffffu); b1 = bf16_bits_to_float(bw[e] >> 16);
        d0 = bf16_bits_to_float(dw[e] & 0xffffu); d1 = bf16_bits_to_float(dw[e] >> 16);
        rw[e] = pack2<true>(a0 * w1 + b0 * w1b + d0 * w2, a1 * w1 + b1 * w1b + d1 * w2);
      } else {
        const __half2 ah = *reinterpret_cast<const __half2*>(&aw[e]), bh = *reinterpret_cast<const __half2*>(&bw[e]),
                      dh = *reinterpret_cast<const __half2*>(&dw[e]);
        a0 = __low2float(ah); a1 = __high2float(ah);
        b0 = __low2float(bh); b1 = __high2float(bh);
        d0 = __low2float(dh); d1 = __high2float(dh);
        rw[e] = pack2<false>(a0 * w1 + b0 * w1b + d0 * w2, a1 * w1 + b1 * w1b + d1 * w2);
      }
    }
    *reinterpret_cast<uint4*>(dst) = r;
    if (c.write_lse && ch == 0) *l2p = lse;
  }
}

inline int launch_attention_pass(const kb200_attn_args* a, int k_skip, int fixed_klen, int fixed_klen_last);

inline int launch_shared_prefix_attention(const kb200_attn_args* a) {
  int sms = 0;
  if (int rc = device_sm_count(a->device, &sms)) return rc;
  KB200_REQUIRE(a->q && a->out && a->page_table && a->seqused_k, "null pointer argument");
  KB200_REQUIRE(a->head_dim == 64 || a->head_dim == 128, "head_dim must be 64 or 128");
  SharedPrefixPlan sp = shared_prefix_plan(a, sms);
  if (!a->workspace || a->workspace_bytes < sp.total)
    return fail(KB200_ERR_WORKSPACE, "workspace too small: need %llu bytes, got %llu", (unsigned long long)sp.total,
                (unsigned long long)a->workspace_bytes);
  KB200_REQUIRE((reinterpret_cast<uintptr_t>(a->workspace) & 255) == 0, "workspace must be 256-byte aligned");
  char* ws = static_cast<char*>(a->workspace);
  const int k_skip = a->shared_prefix_pages * a->page_size;
  sp.pre.out = ws + sp.o1;
  sp.pre.lse = reinterpret_cast<float*>(ws + sp.lse1);
  sp.pre.workspace = ws + sp.ws1;
  sp.pre.workspace_bytes = sp.ws2 - sp.ws1;
  sp.rest.workspace = ws + sp.ws2;
  sp.rest.workspace_bytes = sp.total - sp.ws2;
  const int klen_first = sp.pages_first * a->page_size;
  if (int rc = launch_attention_pass(&sp.pre, 0, klen_first, sp.n_split == 2 ? k_skip - klen_first : klen_first)) return rc;
  const int64_t rows = a->batch * (int64_t)a->seqlen_q;
  sp.rest.lse = a->lse ? a->lse : reinterpret_cast<float*>(ws + sp.lse2);
  if (int rc = launch_attention_pass(&sp.rest, k_skip, -1, -1)) return rc;
  CombineParams c;
  c.o1 = ws + sp.o1;
  c.out = static_cast<char*>(a->out);
  c.lse1 = sp.pre.lse;
  c.lse2 = sp.rest.lse;
  c.o_bs = a->o_batch_stride; c.o_rs = a->o_row_stride; c.o_hs = a->o_head_stride;
  c.rows = rows;
  c.sq = a->seqlen_q; c.hq = a->n_q_heads; c.hd = a->head_dim;
  c.q_is_bf16 = a->q_dtype == KB200_DTYPE_BF16;
  c.write_lse = a->lse != nullptr;
  c.n_pre = sp.n_split;
  const int64_t items = c.rows * c.hq * (c.hd / 8);
  int64_t blocks = (items + 255) / 256;
  if (blocks > sms * 8) blocks = sms * 8;
  KB200_CUDA_OK(launch_kernel(attn_combine_kernel, dim3((unsigned)blocks), dim3(256), 0,
                              static_cast<cudaStream_t>(a->stream), c));
  return KB200_OK;
}

inline int launch_paged_attention(const kb200_attn_args* a) {
  KB200_REQUIRE(a != nullptr, "args is null");
  KB200_REQUIRE(a->struct_bytes == sizeof(kb200_attn_args), "kb200_attn_args size mismatch: got %u, built with %zu",
                a->struct_bytes, sizeof(kb200_attn_args));
  if (a->batch == 0 || a->total_q == 0) return KB200_OK;
  KB200_REQUIRE(a->shared_prefix_pages >= 0, "shared_prefix_pages must be non-negative");
  if (shared_prefix_applies(a)) return launch_shared_prefix_attention(a);
  return launch_attention_pass(a, 0, -1, -1);
}

// One attention pass.  k_skip / fixed_klen / fixed_klen_last: see AttnParams (0 / -1 / -1 for a plain call).
inline int launch_attention_pass(const kb200_attn_args* a, int k_skip, int fixed_klen, int fixed_klen_last) {
  KB200_REQUIRE(a != nullptr, "args is null");
  KB200_REQUIRE(a->struct_bytes == sizeof(kb200_attn_args), "kb200_attn_args size mismatch: got %u, built with %zu",
                a->struct_bytes, sizeof(kb200_attn_args));
  if (a->batch == 0 || a->total_q == 0) return KB200_OK;
  KB200_REQUIRE(a->batch > 0 && a->batch < (1 << 30), "batch out of range");
  KB200_REQUIRE(a->q && a->out && a->k_cache && a->v_cache && a->page_table && (a->seqused_k || fixed_klen >= 0),
                "null pointer argument");
  KB200_REQUIRE(a->q_dtype == KB200_DTYPE_F16 || a->q_dtype == KB200_DTYPE_BF16, "q must be F16 or BF16");
  KB200_REQUIRE(a->kv_dtype == KB200_DTYPE_E4M3 || a->kv_dtype == a->q_dtype,
                "K/V dtype must equal q dtype or be E4M3");
  if (a->head_dim != 64 && a->head_dim != 128)
    return fail(KB200_ERR_UNSUPPORTED, "head_dim %d is not supported (64 or 128)", a->head_dim);
  KB200_REQUIRE(a->n_kv_heads > 0 && a->n_q_heads > 0 && a->n_q_heads % a->n_kv_heads == 0,
                "n_q_heads must be a positive multiple of n_kv_heads");
  const int P = a->page_size;
  if (P <= 0 || P > 256 || (P & (P - 1)) != 0)
    return fail(KB200_ERR_UNSUPPORTED, "page_size %d is not supported (power of two, at most 256)", P);
  KB200_REQUIRE(a->seqlen_q > 0 && a->total_q > 0, "seqlen_q and total_q must be positive");
  // the scratch is sized from total_q: it must describe the rows the kernels will visit
  KB200_REQUIRE(a->cu_seqlens_q != nullptr || a->total_q == a->batch * (int64_t)a->seqlen_q,
                "total_q (%lld) must equal batch * seqlen_q (%lld) in the padded layout", (long long)a->total_q,
                (long long)(a->batch * (int64_t)a->seqlen_q));
  KB200_REQUIRE(a->n_pages > 0, "n_pages must be positive");
  const int es = dtype_size(a->kv_dtype);
  KB200_REQUIRE(aligned16(a->k_cache) && aligned16(a->v_cache), "K/V pools must be 16-byte aligned");
  KB200_REQUIRE((a->kv_page_stride * es) % 16 == 0 && (a->kv_token_stride * es) % 16 == 0 &&
                    (a->kv_head_stride * es) % 16 == 0,
                "K/V pool strides must be multiples of 16 bytes");
  KB200_REQUIRE(aligned16(a->q) && aligned16(a->out), "q and out must be 16-byte aligned");
  KB200_REQUIRE(a->q_row_stride % 8 == 0 && a->q_head_stride % 8 == 0 && a->q_batch_stride % 8 == 0 &&
                    a->o_row_stride % 8 == 0 && a->o_head_stride % 8 == 0 && a->o_batch_stride % 8 == 0,
                "q/out strides must be multiples of 8 elements");
  KB200_REQUIRE(a->softmax_scale > 0.f, "softmax_scale must be positive");

  int sms = 0;
  if (int rc = device_sm_count(a->device, &sms)) return rc;
  const int grid = sms;
  const bool prefill = use_prefill_kernel(a);
  // several KV heads read as one wide head (see attn_head_pack): from here on hkv, group and hd are the wide head's
  const int pack = prefill ? 1 : attn_head_pack(a);
  const int hkv = a->n_kv_heads / pack, hd = a->head_dim * pack;
  const int group = a->n_q_heads / hkv;
  // Segments of at most 8 query rows run the transposed decode kernel where the math, not HBM, limits the
  // 16-row kernel: e4m3 K/V (twice the keys per byte plus the widening), and 16-bit K/V with head_dim 64
  // (the same MMAs and twice the exponentials per byte as head_dim 128: with 8 warps the 16-row kernel waits
  // on its own dependent MMA / ALU chains there, 45 % of the DRAM rate on short contexts).  16-bit K/V with
  // head_dim 128 is within a few percent of the HBM roofline with the 16-row kernel already.
  const bool decode8 = !prefill && (int64_t)group * a->seqlen_q <= kDecodeRows &&
                       (a->kv_dtype == KB200_DTYPE_E4M3 || hd == 64 || pack > 1);
  // (12 warps x 2 stages; 8 x 3 and 6 x 4 -- more tiles in flight per warp, fewer warps -- measured 2 % and
  // 13 % slower on the short contexts of a shared-prefix batch)
  const bool rows32 = use_rows32_kernel(a);   // (8 warps: two output accumulators per thread need the registers)
  const int nw = rows32 ? 8 : (a->kv_dtype == KB200_DTYPE_E4M3 || decode8) ? 12 : 8;
  const int n_workers = grid * nw;
  const AttnWorkspace wl = attn_workspace_layout(a->batch, a->total_q, a->n_q_heads, hkv, hd, grid * kAttnMaxWarps, rows32);
  const uint64_t ws_need = attn_pass_workspace_need(a, sms);
  if (!a->workspace || a->workspace_bytes < ws_need)
    return fail(KB200_ERR_WORKSPACE, "workspace too small: need %llu bytes, got %llu", (unsigned long long)ws_need,
                (unsigned long long)a->workspace_bytes);
  KB200_REQUIRE((reinterpret_cast<uintptr_t>(a->workspace) & 255) == 0, "workspace must be 256-byte aligned");

  const bool block_mask = a->q_visible_until != nullptr;
  if (block_mask) {
    KB200_REQUIRE(a->causal != 0 && a->window_left < 0, "the block-bidirectional mask extends the causal mask: "
                                                       "causal must be set and no window given");
  }
  const int tile_n = prefill ? kPrefillTileKeys : tile_n_for(a->kv_dtype, hd, nw);
  // every TMA copy must land on a 128-byte boundary of shared memory; pools that cannot offer that go
  // through the split-KV kernels' cp.async gather path (the prefill kernel has none)
  // Pages of one or two tokens are gathered as well: a box per token (or two) costs the issuing warp more than
  // the sixteen 16-byte copies per lane of the gather.  Attention call, GB/s, boxes | gather, same GPU:
  //   bf16 D=128, 64 sequences U[1k, 8k]:  P=1 2450 | 4460   P=2 4000 | 4640   P=4 5380 | 4920   P=8 6170 | 5000
  //   e4m3 D=128, 32 sequences U[4k, 32k]: P=1 2970 | 4500   P=2 4620 | 5030   P=4 5800 | 5140   P=8 5430 | 5390
  constexpr int kGatherMaxPage = 2;
  const bool gather = !tma_boxes_possible(a, tile_n) || (!prefill && P <= kGatherMaxPage);
  if (gather && prefill)
    return fail(KB200_ERR_UNSUPPORTED, "a block mask on a pool with page_size %d and %d-byte rows is not supported", P,
                a->head_dim * es);
  TmapKey key{a->k_cache, a->kv_page_stride, a->kv_token_stride, a->kv_head_stride, a->n_pages,
              P, a->n_kv_heads, a->head_dim, a->kv_dtype, a->device};
  // 256-byte rows and pages at least a tile long: one box per (page, K|V) instead of one per half
  const bool merged = !prefill && a->head_dim * es == 256 && P >= tile_n;
  CUtensorMap tmK, tmV;
  if (gather) {
    memset(&tmK, 0, sizeof(tmK));
    memset(&tmV, 0, sizeof(tmV));
  } else {
    if (int rc = get_pool_tmap(key, tile_n, merged, &tmK)) return rc;
    key.base = a->v_cache;
    if (int rc = get_pool_tmap(key, tile_n, merged, &tmV)) return rc;
  }

  char* ws = static_cast<char*>(a->workspace);
  AttnParams p;
  p.q = static_cast<const char*>(a->q);
  p.out = static_cast<char*>(a->out);
  p.lse = a->lse;
  const bool packed = a->cu_seqlens_q != nullptr;
  p.q_bs = packed ? 0 : a->q_batch_stride;
  p.q_rs = a->q_row_stride;
  p.q_hs = a->q_head_stride;
  p.o_bs = packed ? 0 : a->o_batch_stride;
  p.o_rs = a->o_row_stride;
  p.o_hs = a->o_head_stride;
  p.lse_bs = packed ? 0 : (int64_t)a->n_q_heads * a->seqlen_q;
  p.lse_hs = packed ? a->total_q : a->seqlen_q;
  p.page_table = a->page_table;
  p.pt_rs = a->pt_row_stride;
  p.seqused_k = a->seqused_k;
  p.seqused_q = packed ? nullptr : a->seqused_q;
  p.cu_seqlens_q = a->cu_seqlens_q;
  p.q_vis = a->q_visible_until;
  p.q_vis_bs = packed ? 0 : a->q_visible_batch_stride;
  p.ks_vec = a->kv_dtype == KB200_DTYPE_E4M3 ? a->k_scale_per_head : nullptr;
  p.vs_vec = a->kv_dtype == KB200_DTYPE_E4M3 ? a->v_scale_per_head : nullptr;
  p.ks = a->kv_dtype == KB200_DTYPE_E4M3 ? a->k_scale : 1.f;
  p.vs = a->kv_dtype == KB200_DTYPE_E4M3 ? a->v_scale : 1.f;
  p.softmax_scale = a->softmax_scale;
  p.tile_cum = reinterpret_cast<long long*>(ws + wl.tile_cum);
  p.seg_cum = reinterpret_cast<int*>(ws + wl.seg_cum);
  p.nt = reinterpret_cast<int*>(ws + wl.nt);
  p.tile0 = reinterpret_cast<int*>(ws + wl.tile0);
  p.sq = reinterpret_cast<int*>(ws + wl.sq);
  p.qrow0 = reinterpret_cast<int*>(ws + wl.qrow0);
  p.klen = reinterpret_cast<int*>(ws + wl.klen);
  p.bound_rec = reinterpret_cast<int*>(ws + wl.bound_rec);
  p.part_ml = reinterpret_cast<float*>(ws + wl.part_ml);
  p.part_o = reinterpret_cast<float*>(ws + wl.part_o);
  p.n_pages = a->n_pages;
  p.batch = (int)a->batch;
  p.seqlen_q = a->seqlen_q;
  p.hq = a->n_q_heads;
  p.hkv = hkv;
  p.group = group;
  p.head_pack = pack;
  p.real_hd = a->head_dim;
  p.page_size = P;
  p.causal = a->causal != 0;
  p.window_left = a->window_left;
  p.q_is_bf16 = a->q_dtype == KB200_DTYPE_BF16;
  p.n_workers = n_workers;
  p.tile_n = tile_n;
  p.rows_per_seg = prefill ? kPrefillRowsPerSeg : decode8 ? kDecodeRows : rows32 ? 2 * kRowsPerSeg : kRowsPerSeg;
  p.seg_blocks = rows32 ? 2 : 1;
  p.uniform_nseg = (packed || a->seqused_q) ? 0
                   : hkv * ((group * a->seqlen_q + p.rows_per_seg - 1) / p.rows_per_seg);
  p.k_skip = k_skip;
  p.fixed_klen = fixed_klen;
  p.fixed_klen_last = fixed_klen_last;
  p.merged_halves = merged ? 1 : 0;
  p.total_q = a->total_q;
  p.gather = gather ? 1 : 0;
  p.k_base = static_cast<const char*>(a->k_cache);
  p.v_base = static_cast<const char*>(a->v_cache);
  p.kv_ps_b = a->kv_page_stride * es;
  p.kv_ts_b = a->kv_token_stride * es;
  p.kv_hs_b = a->kv_head_stride * es * pack;
  // the split-KV kernels build the plan themselves (every CTA, into shared memory) unless the batch is too large
  p.plan_in_kernel = (!prefill && a->batch <= kPlanSmemMaxBatch) ? 1 : 0;

  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  // sequences of fixed lengths on the prefill kernel (the prefix pass of a shared-prefix call) have
  // nothing to plan: the kernel derives its segments from the launch parameters
  const bool no_plan = prefill && fixed_klen >= 0 && p.uniform_nseg > 0;
  p.no_plan = no_plan ? 1 : 0;
  if (!no_plan && !p.plan_in_kernel) KB200_CUDA_OK(launch_kernel(attn_plan_kernel, dim3(1), dim3(256), 0, stream, p));

  int rc;
  const bool d128 = a->head_dim == 128;
  if (prefill) {
    const int64_t nseg = packed ? (int64_t)a->n_kv_heads * ((group * a->total_q + kPrefillRowsPerSeg - 1) / kPrefillRowsPerSeg + a->batch)
                                : a->batch * (int64_t)a->n_kv_heads * ((group * (int64_t)a->seqlen_q + kPrefillRowsPerSeg - 1) / kPrefillRowsPerSeg);
    KB200_REQUIRE(nseg <= 0x7fffffff, "too many segments");
    const bool bf = a->q_dtype == KB200_DTYPE_BF16;
    if (a->kv_dtype == KB200_DTYPE_E4M3) {
      if (d128) rc = bf ? launch_prefill_variant<128, true, true>(tmK, tmV, p, (int)nseg, a->device, stream)
                        : launch_prefill_variant<128, false, true>(tmK, tmV, p, (int)nseg, a->device, stream);
      else rc = bf ? launch_prefill_variant<64, true, true>(tmK, tmV, p, (int)nseg, a->device, stream)
                   : launch_prefill_variant<64, false, true>(tmK, tmV, p, (int)nseg, a->device, stream);
    } else {
      if (d128) rc = bf ? launch_prefill_variant<128, true, false>(tmK, tmV, p, (int)nseg, a->device, stream)
                        : launch_prefill_variant<128, false, false>(tmK, tmV, p, (int)nseg, a->device, stream);
      else rc = bf ? launch_prefill_variant<64, true, false>(tmK, tmV, p, (int)nseg, a->device, stream)
                   : launch_prefill_variant<64, false, false>(tmK, tmV, p, (int)nseg, a->device, stream);
    }
    return rc;   // every segment is written by its own CTA: nothing to merge
  }
  if (pack > 1 && a->kv_dtype == KB200_DTYPE_E4M3)   // (gather, at most 8 rows: the transposed kernel on the wide head)
    rc = launch_decode_variant<1, 256, false, 12, 2, true>(tmK, tmV, p, grid, a->device, stream);
  else if (pack > 1)
    rc = a->kv_dtype == KB200_DTYPE_BF16 ? launch_decode_variant<2, 128, true, 12, 2, true>(tmK, tmV, p, grid, a->device, stream)
                                         : launch_decode_variant<2, 128, false, 12, 2, true>(tmK, tmV, p, grid, a->device, stream);
  else if (rows32 && a->kv_dtype == KB200_DTYPE_E4M3)
    rc = launch_rows32_dispatch<1, false>(d128, tmK, tmV, p, grid, a->device, stream);
  else if (rows32)
    rc = a->kv_dtype == KB200_DTYPE_BF16 ? launch_rows32_dispatch<2, true>(d128, tmK, tmV, p, grid, a->device, stream)
                                         : launch_rows32_dispatch<2, false>(d128, tmK, tmV, p, grid, a->device, stream);
  else if (decode8 && a->kv_dtype == KB200_DTYPE_E4M3)
    rc = launch_decode_dispatch<1, false>(d128, nw, tmK, tmV, p, grid, a->device, stream);
  else if (decode8)   // 16-bit K/V, head_dim 64
    rc = a->kv_dtype == KB200_DTYPE_BF16
             ? launch_decode_hd<2, true, 64>(nw, tmK, tmV, p, grid, a->device, stream)
             : launch_decode_hd<2, false, 64>(nw, tmK, tmV, p, grid, a->device, stream);
  else if (a->kv_dtype == KB200_DTYPE_E4M3)
    rc = launch_attn_dispatch<1, false>(d128, nw, tmK, tmV, p, grid, a->device, stream);
  else if (a->kv_dtype == KB200_DTYPE_BF16)
    rc = launch_attn_dispatch<2, true>(d128, nw, tmK, tmV, p, grid, a->device, stream);
  else
    rc = launch_attn_dispatch<2, false>(d128, nw, tmK, tmV, p, grid, a->device, stream);
  if (rc) return rc;

  const int64_t max_seg = packed ? attn_max_segments(a->batch, a->total_q, a->n_q_heads, hkv)
                                 : a->batch * hkv * ((group * (int64_t)a->seqlen_q + p.rows_per_seg - 1) / p.rows_per_seg);
  KB200_REQUIRE(max_seg <= 0x7fffffff, "too many segments");
  // one block per range boundary (the only places where a segment can be cut), striding when there are more
  int64_t merge_blocks = std::max<int64_t>(n_workers - 1, 1);
  if (merge_blocks > (int64_t)sms * 16) merge_blocks = (int64_t)sms * 16;   // 16 x 128 threads fill an SM
  if (pack > 1 && hd == 256) KB200_CUDA_OK(launch_kernel(attn_merge_kernel<256>, dim3((unsigned)merge_blocks), dim3(128), 0, stream, p));
  else if (d128 || hd == 128) KB200_CUDA_OK(launch_kernel(attn_merge_kernel<128>, dim3((unsigned)merge_blocks), dim3(128), 0, stream, p));
  else KB200_CUDA_OK(launch_kernel(attn_merge_kernel<64>, dim3((unsigned)merge_blocks), dim3(128), 0, stream, p));
  return KB200_OK;
}

}  // namespace kb200
