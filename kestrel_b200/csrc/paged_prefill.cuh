// Paged prefill / append-prefill attention for sm_100a on the 5th-generation tensor
// cores: many query rows per sequence (a prompt chunk), K/V gathered through the
// page table.  This is the compute-bound mode of the same op the decode kernels
// serve (paged_attention.cuh); it is chosen when a sequence brings at least
// kPrefillMinRows packed query rows and K/V are 16-bit.
//
// One CTA = one (sequence, KV head, block of 128 packed query rows); packed row
// r = j * group + g is query position j of head h * group + g, so one pass over
// the keys serves the whole GQA group.  Per 128-key tile:
//
//   TMA warp      K and V page boxes -> 128-byte-swizzled shared memory (2 stages)
//   MMA warp      S = Q K^T   (tcgen05.mma, M=128 N=128, operands from shared
//                 memory descriptors, accumulator in tensor memory), then
//                 O_tile = P V with P read back from shared memory; S and O_tile
//                 are double-buffered in tensor memory so the next Q K^T runs
//                 under the softmax of the current tile
//   4 softmax warps  one row per thread: tcgen05.ld of S, mask, online softmax
//                 (fp32, base 2), P written to shared memory as the A operand of
//                 the second product; O accumulates in registers
//
// Every wait on a shared-memory barrier is bounded; a wait that runs out is
// recorded in the device status word and the CTA leaves through the common exit,
// which frees its tensor memory.
#pragma once

#include "paged_attention.cuh"

namespace kb200 {

constexpr int kPrefillRows = 128;     // packed query rows per CTA (MMA M)
constexpr int kPrefillKeys = 128;     // keys per tile (MMA N of the first product)
constexpr int kPrefillStages = 2;     // K/V ring depth
constexpr int kPrefillMinRows = 64;   // packed rows per sequence from which this kernel is used
constexpr int kPrefillThreads = 192;  // 4 softmax warps, 1 TMA warp, 1 MMA warp

template <int HD>
struct PrefillSmem {
  static constexpr int NH = HD * 2 / 128;                       // 128-byte slabs per row
  static constexpr int SLAB = kPrefillRows * 128;               // bytes of one 128-row slab
  static constexpr int Q_BYTES = NH * SLAB;
  static constexpr int KV_TILE = NH * kPrefillKeys * 128;       // K (or V) tile
  static constexpr int STAGE = 2 * KV_TILE;
  static constexpr int P_BYTES = 2 * SLAB;                      // 128 rows x 128 keys, 16-bit
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_KV = Q_BYTES;
  static constexpr int OFF_P = OFF_KV + kPrefillStages * STAGE;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  static constexpr int N_BARS = 4 * kPrefillStages + 10;
  static constexpr int OFF_TMEM = OFF_BAR + 8 * N_BARS;
  static constexpr int BYTES = OFF_TMEM + 16 + 1024;            // + alignment slack
};

// ---- tcgen05 / tensor memory helpers ---------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], 16-bit operands, fp32 accumulate
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread i of the warp gets lane (lane base + i)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  tc_wait_ld();
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor, 128-byte swizzle; offsets in bytes.
//   K-major operand  (rows of 128 bytes along K, 8-row groups 1024 bytes apart): lbo unused (1), sbo = 1024
//   MN-major operand (rows of 128 bytes along MN, one row per K index):          lbo = distance between
//                     64-element column slabs, sbo = 1024 (8 K indices)
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;   // descriptor version of this architecture
  d |= 2ull << 61;   // 128-byte swizzle
  return d;
}
// Instruction descriptor, kind::f16: fp32 accumulator, A/B both F16 (0) or BF16 (1), A K-major,
// B K-major or MN-major, M = 128.
__host__ __device__ constexpr uint32_t umma_idesc(bool bf16, bool b_mn_major, int n) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((b_mn_major ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kPrefillRows >> 4) << 24);
}

template <int HD, bool BF16>
__global__ void __launch_bounds__(kPrefillThreads, 1)
paged_prefill_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                     const __grid_constant__ AttnParams p) {
  using SM = PrefillSmem<HD>;
  constexpr int NH = SM::NH;
  constexpr int NS = kPrefillStages;
  constexpr int BN = kPrefillKeys;
  constexpr float kLog2e = 1.4426950408889634f;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t S_COL = 0, O_COL = 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));   // generic pointer to the aligned base
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // barrier map
  const uint32_t bar = sbase + SM::OFF_BAR;
  auto B_KFULL = [&](int s) { return bar + 8u * s; };
  auto B_VFULL = [&](int s) { return bar + 8u * (NS + s); };
  auto B_KVEMPTY = [&](int s) { return bar + 8u * (2 * NS + s); };
  auto B_SREADY = [&](int b) { return bar + 8u * (3 * NS + b); };
  auto B_SFREE = [&](int b) { return bar + 8u * (3 * NS + 2 + b); };
  auto B_OREADY = [&](int b) { return bar + 8u * (3 * NS + 4 + b); };
  auto B_OFREE = [&](int b) { return bar + 8u * (3 * NS + 6 + b); };
  const uint32_t B_PREADY = bar + 8u * (3 * NS + 8);
  const uint32_t B_PFREE = bar + 8u * (3 * NS + 9);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sgen + SM::OFF_TMEM);

  pdl_launch_dependents();
  pdl_wait();   // the plan, and the append before it, must have completed

  // ---- which segment is this CTA?
  const int seg = blockIdx.x;
  if (seg >= p.seg_cum[p.batch]) return;   // uniform over the CTA; nothing allocated yet
  int b;
  if (p.uniform_nseg > 0) {
    b = seg / p.uniform_nseg;
  } else {
    int lo = 0, hi = p.batch;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (p.seg_cum[mid] <= seg) lo = mid; else hi = mid;
    }
    b = lo;
  }
  const int sq = p.sq[b], L = p.klen[b], qrow0 = p.qrow0[b];
  const int nrows = p.group * sq;
  const int nmb = (nrows + kPrefillRows - 1) / kPrefillRows;
  const int sib = seg - p.seg_cum[b];
  const int h = sib / nmb, mb = sib - h * nmb;
  const int row_first = mb * kPrefillRows;
  const int row_last = min(nrows, row_first + kPrefillRows) - 1;
  const bool upper = p.causal || p.window_left >= 0;
  const int j_first = row_first / p.group, j_last = row_last / p.group;
  int k_end = upper ? min(L, L - sq + j_last + 1) : L;      // keys [k_begin, k_end) can be visible
  if (k_end < 0) k_end = 0;
  int k_begin = 0;
  if (p.window_left >= 0) k_begin = max(0, L - sq + j_first - p.window_left);
  const int tile_begin = k_begin / BN;
  const int n_tiles = k_end > tile_begin * BN ? (k_end - tile_begin * BN + BN - 1) / BN : 0;

  // ---- set-up: barriers, tensor memory, Q tile
  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(B_KFULL(s), 1);
      mbar_init(B_VFULL(s), 1);
      mbar_init(B_KVEMPTY(s), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(B_SREADY(i), 1);
      mbar_init(B_SFREE(i), 128);
      mbar_init(B_OREADY(i), 1);
      mbar_init(B_OFREE(i), 128);
    }
    mbar_init(B_PREADY, 128);
    mbar_init(B_PFREE, 1);
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc(sbase + SM::OFF_TMEM, TMEM_COLS);
    tmem_relinquish();
  }
  {
    // Q rows -> shared memory in the K-major 128-byte-swizzled operand layout; rows past the
    // segment's end are zero
    constexpr int CH = HD * 2 / 16;   // 16-byte chunks per row
    for (int i = tid; i < kPrefillRows * CH; i += kPrefillThreads) {
      const int r = i / CH, c = i - r * CH;
      const int row = row_first + r;
      uint4 val = make_uint4(0u, 0u, 0u, 0u);
      if (row < nrows) {
        const int j = row / p.group, g = row - j * p.group;
        const char* src = p.q + 2 * ((int64_t)b * p.q_bs + (int64_t)(qrow0 + j) * p.q_rs +
                                     (int64_t)(h * p.group + g) * p.q_hs) + 16 * c;
        val = *reinterpret_cast<const uint4*>(src);
      }
      const uint32_t off = SM::OFF_Q + (uint32_t)(c >> 3) * SM::SLAB + (uint32_t)r * 128 + (uint32_t)(((c & 7) ^ (r & 7)) << 4);
      *reinterpret_cast<uint4*>(sgen + off) = val;
    }
    fence_proxy_async();   // generic-proxy writes above are read by the tensor core (async proxy)
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // =========================== TMA producer ===========================
    const int P = p.page_size;
    const int p_shift = 31 - __clz(P);
    const int box_rows = P < BN ? P : BN;
    const int box_shift = 31 - __clz(box_rows);
    const int boxes_per_tile = BN >> box_shift;
    bool ok = true;
    for (int it = 0; it < n_tiles && ok; ++it) {
      const int s = it % NS;
      if (it >= NS) ok = mbar_wait_bounded(B_KVEMPTY(s), (uint32_t)((it / NS) - 1) & 1u);
      if (!ok) { if (lane == 0) report(KB200_STATUS_WAIT_TIMEOUT, it, KID_PREFILL); break; }
      const int key0 = (tile_begin + it) * BN;
      int nvalid = L - key0;
      if (nvalid > BN) nvalid = BN;
      const int nvb = (nvalid + box_rows - 1) >> box_shift;
      const uint32_t bytes = (uint32_t)((nvb << box_shift) * HD * 2);
      if (lane == 0) {
        mbar_expect_tx(B_KFULL(s), bytes);
        mbar_expect_tx(B_VFULL(s), bytes);
      }
      __syncwarp();
      const uint32_t kdst = sbase + SM::OFF_KV + (uint32_t)s * SM::STAGE;
      const uint32_t vdst = kdst + SM::KV_TILE;
      // K boxes first so the first product can start before V has landed
      for (int kv = 0; kv < 2; ++kv) {
        for (int j = lane; j < boxes_per_tile * NH; j += 32) {
          const int i = j / NH, half = j - i * NH;
          if (i >= nvb) continue;
          const int key = key0 + (i << box_shift);
          const int page = p.page_table[(int64_t)b * p.pt_rs + (key >> p_shift)];
          if ((unsigned)page >= (unsigned long long)p.n_pages) report(KB200_STATUS_BAD_PAGE, page, KID_PREFILL);
          const uint32_t dst = (kv ? vdst : kdst) + (uint32_t)half * (BN * 128) + (uint32_t)(i << box_shift) * 128;
          tma_load_4d(dst, kv ? &tmV : &tmK, kv ? B_VFULL(s) : B_KFULL(s), half * 64, key & (P - 1), h, page);
        }
      }
    }
  } else if (warp == 5) {
    // =========================== MMA issuer ===========================
    constexpr uint32_t IDESC_QK = umma_idesc(BF16, false, BN);
    constexpr uint32_t IDESC_PV = umma_idesc(BF16, true, HD);
    const uint32_t q_addr = sbase + SM::OFF_Q;
    const uint32_t p_addr = sbase + SM::OFF_P;
    bool ok = true;
    auto pv = [&](int j) {
      const int s = j % NS;
      ok = ok && mbar_wait_bounded(B_PREADY, (uint32_t)j & 1u);
      ok = ok && mbar_wait_bounded(B_VFULL(s), (uint32_t)(j / NS) & 1u);
      if (ok && j >= 2) ok = mbar_wait_bounded(B_OFREE(j & 1), (uint32_t)((j >> 1) - 1) & 1u);
      if (!ok) return;
      const uint32_t v_addr = sbase + SM::OFF_KV + (uint32_t)s * SM::STAGE + SM::KV_TILE;
      const int key0 = (tile_begin + j) * BN;
      int nvalid = L - key0;
      if (nvalid > BN) nvalid = BN;
      const int ksteps = (nvalid + 15) >> 4;
      if (nvalid & 15) {
        // rows of V between the sequence end and the end of its 16-key block may hold anything
        // (NaN bit patterns included) and would poison 0 * V: zero them
        const int r0 = nvalid, r1 = ksteps << 4;
        for (int i = lane; i < (r1 - r0) * NH * 8; i += 32) {
          const int r = r0 + i / (NH * 8), c = i % (NH * 8);
          *reinterpret_cast<uint4*>(sgen + (v_addr - sbase) + (uint32_t)(c >> 3) * (BN * 128) + (uint32_t)r * 128 +
                                    (uint32_t)((c & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);   // a whole row: swizzle is irrelevant
        }
        fence_proxy_async();
        __syncwarp();
      }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t o_tmem = tmem_base + O_COL + (uint32_t)(j & 1) * HD;
        for (int k = 0; k < ksteps; ++k) {
          const uint64_t da = umma_desc(p_addr + (uint32_t)(k >> 2) * SM::SLAB + (uint32_t)(k & 3) * 32, 16, 1024);
          const uint64_t db = umma_desc(v_addr + (uint32_t)k * 2048, BN * 128, 1024);
          umma_f16(o_tmem, da, db, IDESC_PV, k > 0 ? 1u : 0u);
        }
        tc_commit(B_OREADY(j & 1));
        tc_commit(B_KVEMPTY(s));
        tc_commit(B_PFREE);
      }
      __syncwarp();
    };
    for (int it = 0; it < n_tiles && ok; ++it) {
      const int s = it % NS;
      ok = mbar_wait_bounded(B_KFULL(s), (uint32_t)(it / NS) & 1u);
      if (ok && it >= 2) ok = mbar_wait_bounded(B_SFREE(it & 1), (uint32_t)((it >> 1) - 1) & 1u);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t k_addr = sbase + SM::OFF_KV + (uint32_t)s * SM::STAGE;
        const uint32_t s_tmem = tmem_base + S_COL + (uint32_t)(it & 1) * BN;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t da = umma_desc(q_addr + (uint32_t)(k >> 2) * SM::SLAB + (uint32_t)(k & 3) * 32, 16, 1024);
          const uint64_t db = umma_desc(k_addr + (uint32_t)(k >> 2) * (BN * 128) + (uint32_t)(k & 3) * 32, 16, 1024);
          umma_f16(s_tmem, da, db, IDESC_QK, k > 0 ? 1u : 0u);
        }
        tc_commit(B_SREADY(it & 1));
      }
      __syncwarp();
      if (it > 0) pv(it - 1);
    }
    if (ok && n_tiles > 0) pv(n_tiles - 1);
    if (!ok && lane == 0) report(KB200_STATUS_WAIT_TIMEOUT, seg, KID_PREFILL);
  } else {
    // =========================== softmax: one row per thread ===========================
    const int r = tid;                       // row inside the block == tensor-memory lane
    const int row = row_first + r;
    const bool valid = row < nrows;
    const int j = valid ? row / p.group : j_last;
    const int g = valid ? row - j * p.group : 0;
    const int lim = upper ? L - sq + j : L - 1;                       // last visible key
    const int lo = p.window_left >= 0 ? lim - p.window_left : 0;       // first visible key
    const float ksc = p.ks_vec ? p.ks_vec[h] : p.ks;
    const float vscale = p.vs_vec ? p.vs_vec[h] : p.vs;
    const float sl2 = p.softmax_scale * ksc * kLog2e;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    float o[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int it = 0; it < n_tiles; ++it) {
      const int buf = it & 1;
      ok = mbar_wait_bounded(B_SREADY(buf), (uint32_t)(it >> 1) & 1u);
      if (!ok) break;
      tc_fence_after();
      const uint32_t s_tmem = tmem_base + lane_base + S_COL + (uint32_t)buf * BN;
      const int key0 = (tile_begin + it) * BN;
      const bool need_mask = key0 + BN - 1 > lim || key0 < lo;
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        float v[32];
        tmem_ld32(s_tmem + c * 32, v);
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kk = key0 + c * 32 + i;
            if (kk > lim || kk < lo) v[i] = -INFINITY;
          }
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) mx = fmaxf(mx, v[i]);
      }
      const float m_new = fmaxf(m, mx);
      const float alpha = (m == -INFINITY) ? 0.f : ex2((m - m_new) * sl2);   // m_new >= m; both -inf cannot reach ex2
      const float ms = (m_new == -INFINITY) ? 0.f : m_new * sl2;
      // the P buffer is free once the second product of the previous tile has completed
      if (it > 0) {
        ok = mbar_wait_bounded(B_PFREE, (uint32_t)(it - 1) & 1u);
        if (!ok) break;
      }
      // pass 2: weights -> shared memory (A operand of P V), row sum
      float lsum = 0.f;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        float v[32];
        tmem_ld32(s_tmem + c * 32, v);
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const int kk = key0 + c * 32 + i;
          float p0 = ex2(fmaf(v[i], sl2, -ms));
          float p1 = ex2(fmaf(v[i + 1], sl2, -ms));
          if (need_mask) {
            if (kk > lim || kk < lo) p0 = 0.f;
            if (kk + 1 > lim || kk + 1 < lo) p1 = 0.f;
          }
          lsum += p0 + p1;
          w[i >> 1] = pack2<BF16>(p0, p1);
        }
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int ch = c * 4 + q4;   // 16-byte chunk of this row's 256 bytes
          const uint32_t off = SM::OFF_P + (uint32_t)(ch >> 3) * SM::SLAB + (uint32_t)r * 128 +
                               (uint32_t)(((ch & 7) ^ (r & 7)) << 4);
          *reinterpret_cast<uint4*>(sgen + off) = make_uint4(w[4 * q4], w[4 * q4 + 1], w[4 * q4 + 2], w[4 * q4 + 3]);
        }
      }
      // S has been read twice: the buffer may be overwritten by the product two tiles ahead
      tc_fence_before();
      mbar_arrive(B_SFREE(buf));
      fence_proxy_async();
      mbar_arrive(B_PREADY);
      // fold in the previous tile's O while the tensor core works on this one
      if (it > 0) {
        const int pb = (it - 1) & 1;
        ok = mbar_wait_bounded(B_OREADY(pb), (uint32_t)((it - 1) >> 1) & 1u);
        if (!ok) break;
        tc_fence_after();
        const uint32_t o_tmem = tmem_base + lane_base + O_COL + (uint32_t)pb * HD;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          float v[32];
          tmem_ld32(o_tmem + c * 32, v);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c * 32 + i] += v[i];
        }
        tc_fence_before();
        mbar_arrive(B_OFREE(pb));
      }
      if (alpha != 1.f) {
#pragma unroll
        for (int i = 0; i < HD; ++i) o[i] *= alpha;
      }
      l = l * alpha + lsum;
      m = m_new;
    }
    if (ok && n_tiles > 0) {
      const int pb = (n_tiles - 1) & 1;
      ok = mbar_wait_bounded(B_OREADY(pb), (uint32_t)((n_tiles - 1) >> 1) & 1u);
      if (ok) {
        tc_fence_after();
        const uint32_t o_tmem = tmem_base + lane_base + O_COL + (uint32_t)pb * HD;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          float v[32];
          tmem_ld32(o_tmem + c * 32, v);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c * 32 + i] += v[i];
        }
        tc_fence_before();
      }
    }
    if (!ok) {
      if (lane == 0) report(KB200_STATUS_WAIT_TIMEOUT, seg, KID_PREFILL);
    } else if (valid) {
      const float inv = l > 0.f ? vscale / l : 0.f;
      const int hq = h * p.group + g;
      char* dst = p.out + 2 * ((int64_t)b * p.o_bs + (int64_t)(qrow0 + j) * p.o_rs + (int64_t)hq * p.o_hs);
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) {
        uint4 w;
        w.x = pack2<BF16>(o[8 * c + 0] * inv, o[8 * c + 1] * inv);
        w.y = pack2<BF16>(o[8 * c + 2] * inv, o[8 * c + 3] * inv);
        w.z = pack2<BF16>(o[8 * c + 4] * inv, o[8 * c + 5] * inv);
        w.w = pack2<BF16>(o[8 * c + 6] * inv, o[8 * c + 7] * inv);
        *reinterpret_cast<uint4*>(dst + 16 * c) = w;
      }
      if (p.lse) {
        constexpr float kLn2 = 0.6931471805599453f;
        p.lse[(int64_t)b * p.lse_bs + (int64_t)hq * p.lse_hs + qrow0 + j] =
            l > 0.f ? m * sl2 * kLn2 + logf(l) : -INFINITY;
      }
    }
  }

  // ---- common exit: every role comes here, then the allocating warp frees the tensor memory
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

inline bool prefill_enabled() {
  static const bool on = [] {
    const char* e = getenv("KB200_PREFILL");
    return !(e && e[0] == '0');
  }();
  return on;
}

template <int HD, bool BF16>
inline int launch_prefill_variant(const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p, int grid,
                                  int dev, cudaStream_t stream) {
  using SM = PrefillSmem<HD>;
  auto kern = paged_prefill_kernel<HD, BF16>;
  static bool done[64] = {};
  if (!done[dev & 63]) {
    KB200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::BYTES));
    done[dev & 63] = true;
  }
  KB200_CUDA_OK(launch_kernel(kern, dim3(grid), dim3(kPrefillThreads), SM::BYTES, stream, tmK, tmV, p));
  return KB200_OK;
}

}  // namespace kb200
