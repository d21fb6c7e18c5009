// Paged prefill / append-prefill attention for sm_100a on the 5th-generation tensor
// cores: many query rows per sequence (a prompt chunk), K/V gathered through the
// page table.  This is the compute-bound mode of the same op the decode kernels
// serve (paged_attention.cuh); it is chosen when a sequence brings at least
// 33 packed query rows per KV head (65 on e4m3 pools; 17 with 16-bit head_dim-128 pools and a CTA per SM).  K/V pools are 16-bit or FP8 e4m3 (see KV8 below).
//
// One CTA = one (sequence, KV head, block of 256 packed query rows) = two Q tiles of
// 128 rows; packed row r = j * group + g is query position j of head h * group + g,
// so one pass over the keys serves the whole GQA group.  Per 128-key tile:
//
//   2 TMA warps     K and V page boxes -> 128-byte-swizzled shared memory (a ring of
//                   K_0 V_0 K_1 V_1 ... tiles shared by both Q tiles; one warp issues the K
//                   tiles, the other the V tiles)
//   MMA warp        S_x = Q_x K^T (tcgen05.mma, M=128 N=128, operands from shared-memory
//                   descriptors, accumulator in tensor memory) and O_x += P_x V with
//                   P_x read from tensor memory (it overlays S_x), which halves the
//                   shared-memory operand traffic of that product; the two Q tiles alternate
//                   (PV_A QK_A PV_B QK_B) so one tile's products run under the other's
//                   softmax
//   2 x 4 softmax   one row per thread: tcgen05.ld of S, mask, online softmax (fp32,
//   warps           base 2), P written back over S as packed 16-bit pairs (tcgen05.st), the
//                   A operand of the second product.  O stays in tensor memory; the running
//                   maximum is raised (and O rescaled through tcgen05.ld/st) only when
//                   it grew by more than 2^8, so weights stay bounded and the rescale
//                   is rare
//
// Every wait on a shared-memory barrier is bounded; a wait that runs out is
// recorded in the device status word and the CTA leaves through the common exit,
// which frees its tensor memory.
#pragma once

#include "paged_attention.cuh"

namespace kb200 {

constexpr int kPfTileRows = 128;    // packed query rows per Q tile (MMA M)
constexpr int kPfCtaRows = 256;     // two Q tiles per CTA
constexpr int kPrefillKeys = 128;   // keys per tile (MMA N of the first product)
// 2 x 4 softmax warps (0-7), a TMA warp (8), the MMA warp (9), then either a second TMA warp (10: 16-bit
// pools, where it takes the V tiles) or 4 warps (10-13: FP8 pools) that widen the tiles to 16 bits
constexpr int kPfCopyThreads = 288;   // warps 0-7 and 9 copy Q and meet at the set-up barrier
constexpr int pf_threads(bool kv8) { return kv8 ? 448 : 352; }

template <int HD, bool KV8>
struct PrefillSmem {
  static constexpr int NH = HD * 2 / 128;                       // 128-byte slabs per 16-bit row
  static constexpr int SLAB = kPfTileRows * 128;                // bytes of one 128-row slab
  static constexpr int Q_TILE = NH * SLAB;
  static constexpr int KV_TILE = NH * kPrefillKeys * 128;       // one K or V tile, 16-bit
  // 16-bit K/V tiles in flight (K0 V0 K1 V1 ...); with FP8 pools they are filled by the widening warps
  static constexpr int RING = KV8 ? (HD == 128 ? 3 : 6) : (HD == 128 ? 5 : 8);
  static constexpr int RB8 = HD;                                // bytes of one e4m3 row (128 or 64)
  static constexpr int STG_TILE = kPrefillKeys * RB8;           // one e4m3 tile as the TMA delivers it
  static constexpr int NSTG = KV8 ? (HD == 128 ? 4 : 8) : 0;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_KV = 2 * Q_TILE;
  static constexpr int OFF_STG = OFF_KV + RING * KV_TILE;
  static constexpr int OFF_BAR = OFF_STG + NSTG * STG_TILE;
  static constexpr int RINGB = RING + 1;                        // barrier pairs: the key split borrows Q tile B as one more ring slot
  static constexpr int N_BARS = 2 * RINGB + 6 + 2 * NSTG;
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
// D[tmem] (+)= A[tmem] * B[smem desc]: A is M x 16 with lane = row and two 16-bit elements per column
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
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

// the same load without the wait: the caller issues tc_wait_ld() before it reads v
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
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
}

// four tcgen05.ld of 32 columns each, one wait: a whole 128-column row
__device__ __forceinline__ void tmem_ld128(uint32_t taddr, float (&v)[128]) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t* r = reinterpret_cast<uint32_t*>(&v[32 * c]);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr + 32u * c)
        : "memory");
  }
  tc_wait_ld();
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
}
__device__ __forceinline__ void tmem_st16u(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Packed fp32 pairs (one instruction, two lanes) and the three-input maximum: the softmax warps
// are bound by instruction issue, and these halve the count of their arithmetic instructions.
__device__ __forceinline__ uint64_t pack_f32x2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Shared-memory matrix descriptors (64 bits), 128-byte swizzle, as the MMA warp builds them:
//   bits  0-13  start address >> 4        bits 16-29  leading byte offset >> 4
//   bits 32-45  stride byte offset >> 4   bits 46-47  descriptor version (1)   bits 61-63  swizzle mode (2 = 128 B)
//   K-major operand  (rows of 128 bytes along K, 8-row groups 1024 bytes apart): leading offset unused, stride 1024
//   MN-major operand (rows of 128 bytes along MN, one row per K index): leading offset = distance between
//                     64-element column slabs, stride 1024 (8 K indices)
// Instruction descriptor, kind::f16: fp32 accumulator, A/B both F16 (0) or BF16 (1), A K-major,
// B K-major or MN-major, M = 128.
__host__ __device__ constexpr uint32_t umma_idesc(bool bf16, bool b_mn_major, int n) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((b_mn_major ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kPfTileRows >> 4) << 24);
}

// BF16: dtype of q and out.  KV8: K/V pools hold e4m3 codes; the tiles are widened to f16 in shared memory
// (exact), the tensor core then runs on f16 operands (q is converted once, as in the decode kernels)
// and the dequantisation scales are folded into the softmax scale (K) and the final normalisation (V).
// SPLIT: no sequence of the launch brings more than 128 packed rows per KV head, so no CTA has rows in its
// second Q tile and the key split (below) is open to every CTA; the ring then has one slot more.
template <int HD, bool BF16, bool KV8, bool SPLIT>
__global__ void __launch_bounds__(pf_threads(KV8), 1)
paged_prefill_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                     const __grid_constant__ AttnParams p) {
  using SM = PrefillSmem<HD, KV8>;
  constexpr bool MMA_BF16 = BF16 && !KV8;   // operand type of both products
  constexpr int NH = SM::NH;
  constexpr int RING = SM::RING;
  // Under the key split Q tile B is unused and lies directly below the K/V ring: it becomes one more ring slot
  // (every key tile feeds one pipeline instead of two, so tiles are consumed twice as fast and the copies have
  // to run further ahead).
  static_assert(SM::Q_TILE == SM::KV_TILE && SM::OFF_KV == SM::OFF_Q + 2 * SM::Q_TILE, "Q tile B adjoins the ring");
  constexpr int RINGN = SPLIT ? RING + 1 : RING;
  constexpr uint32_t RING_OFF = SPLIT ? SM::OFF_Q + SM::Q_TILE : SM::OFF_KV;
  constexpr int BN = kPrefillKeys;
  constexpr float kLog2e = 1.4426950408889634f;
  constexpr float kRescaleStep = 8.f;   // the running maximum is only raised when it grew by 2^8
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t S_COL = 0, O_COL = 2 * BN;   // S_A, S_B, then O_A, O_B (128 columns reserved each)
  // head_dim 64 leaves 64 spare columns next to each O: P gets them instead of overlaying S, so the
  // next Q K^T of a tile can be issued before its P V and the tile's softmax restarts ~800 cycles earlier
  constexpr bool PSEP = HD == 64;
  constexpr uint32_t P_OFF = PSEP ? O_COL + 64 : S_COL;   // + x * 128: first column of P_x

  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));   // generic pointer to the aligned base
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // barrier map
  const uint32_t bar = sbase + SM::OFF_BAR;
  auto B_FULL = [&](int s) { return bar + 8u * s; };
  constexpr int RINGB = SM::RINGB;
  auto B_EMPTY = [&](int s) { return bar + 8u * (RINGB + s); };
  auto B_SREADY = [&](int x) { return bar + 8u * (2 * RINGB + x); };
  auto B_PREADY = [&](int x) { return bar + 8u * (2 * RINGB + 2 + x); };
  auto B_PVDONE = [&](int x) { return bar + 8u * (2 * RINGB + 4 + x); };
  auto B_SFULL = [&](int s) { return bar + 8u * (2 * RINGB + 6 + s); };               // e4m3 staging tiles
  auto B_SEMPTY = [&](int s) { return bar + 8u * (2 * RINGB + 6 + SM::NSTG + s); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sgen + SM::OFF_TMEM);

  pdl_launch_dependents();
  pdl_wait();   // the plan, and the append before it, must have completed

  // ---- which segment is this CTA?
  // CTAs are handed out in block order: taking the segments from the back puts the later row blocks
  // of a sequence, which see more keys under the causal mask, first and keeps the tail of the grid short
  // (sequences of fixed lengths, the prefix pass of a shared-prefix call, need no plan launch)
  const bool no_plan = p.no_plan != 0;
  const int seg = (no_plan ? p.batch * p.uniform_nseg : p.seg_cum[p.batch]) - 1 - (int)blockIdx.x;
  if (seg < 0) return;   // uniform over the CTA; nothing allocated yet
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
  const int sq = no_plan ? p.seqlen_q : p.sq[b];
  const int L = no_plan ? (b == p.batch - 1 ? p.fixed_klen_last : p.fixed_klen) : p.klen[b];
  const int qrow0 = no_plan ? 0 : p.qrow0[b];
  const int nrows = p.group * sq;
  const int nmb = (nrows + kPfCtaRows - 1) / kPfCtaRows;
  const int sib = seg - (no_plan ? b * p.uniform_nseg : p.seg_cum[b]);
  const int h = sib / nmb, mb = sib - h * nmb;
  const int row_first = mb * kPfCtaRows;
  const bool upper = p.causal || p.window_left >= 0;
  // key range [k_begin, k_end_x) that rows of Q tile x can see; tiles are counted from tile_begin
  const int j_first = row_first / p.group;
  int k_begin = 0;
  if (p.window_left >= 0) k_begin = max(0, L - sq + j_first - p.window_left);
  const int tile_begin = k_begin / BN;
  int n_x[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int r0 = row_first + x * kPfTileRows;
    if (r0 >= nrows) { n_x[x] = 0; continue; }
    const int r1 = min(nrows, r0 + kPfTileRows) - 1;
    int j1 = r1 / p.group;   // last query position of the tile; with a block mask it sees up to the end of its block
    if (p.q_vis) j1 = max(j1, min(sq - 1, p.q_vis[(int64_t)b * p.q_vis_bs + qrow0 + j1]));
    int k_end = upper ? min(L, L - sq + j1 + 1) : L;
    n_x[x] = k_end > tile_begin * BN ? (k_end - tile_begin * BN + BN - 1) / BN : 0;
  }
  const int n_tiles = max(n_x[0], n_x[1]);   // n_x[0] <= n_x[1] whenever tile B has rows (limits grow with the row)
  // Key split.  A CTA whose second Q tile has no rows (at most 128 packed rows per KV head: short chunks with few
  // heads per group, a verify step of a few dozen tokens) would run one dependent chain Q K^T -> softmax -> P V per
  // key tile with half of its warps and tensor memory idle.  Instead the two pipelines both work on Q tile A:
  // stream 0 takes the even key tiles, stream 1 the odd ones, each with its own S, P, O, maximum and sum, and the
  // two partial results are combined at the end.  Ring entries V_i to K_{i+2} (four in a row) are live at
  // once: the f16 ring of an e4m3 pool (three tiles) gets there with the borrowed Q tile.
  const bool split = SPLIT && n_x[0] >= 2;
  const int n_s[2] = {split ? (n_tiles + 1) >> 1 : n_x[0], split ? n_tiles >> 1 : n_x[1]};   // key tiles per pipeline

  // ---- set-up.  The TMA warp starts on the K/V tiles at once, so that they are in flight while the
  // other warps bring Q in and tensor memory is allocated.
  // =========================== TMA producer (warp 8) ===========================
  // ring entries alternate K_0, V_0, K_1, V_1, ...
  const int page_sz = p.page_size;
  const int p_shift = 31 - __clz(page_sz);
  const int box_rows = page_sz < BN ? page_sz : BN;
  const int box_shift = 31 - __clz(box_rows);
  const int boxes_per_tile = BN >> box_shift;
  // Page indices are fetched 32 table entries at a time (one per lane) and handed to the boxes by
  // shuffle, so a tile does not wait for its own dependent table load.
  int win_base = -1, win_page = 0;   // table slot of lane 0's entry; this lane's entry
  const int64_t pt_row = (int64_t)b * p.pt_rs;
  const int n_slots = (L + page_sz - 1) >> p_shift;   // table entries that hold pages of this sequence
  auto produce = [&](int idx) -> bool {   // warp-wide; false when the ring slot never came free
    constexpr int NSLOT = KV8 ? SM::NSTG : RINGN;
    const int s = idx % NSLOT;
    if (idx >= NSLOT && !mbar_wait_bounded(KV8 ? B_SEMPTY(s) : B_EMPTY(s), (uint32_t)((idx / NSLOT) - 1) & 1u)) {
      if (lane == 0) report(KB200_STATUS_WAIT_TIMEOUT, idx, KID_PREFILL);
      return false;
    }
    const int kv = idx & 1;
    const int key0 = (tile_begin + (idx >> 1)) * BN;
    int nvalid = L - key0;
    if (nvalid > BN) nvalid = BN;
    const int nvb = (nvalid + box_rows - 1) >> box_shift;
    const uint32_t full = KV8 ? B_SFULL(s) : B_FULL(s);
    const int slot0 = key0 >> p_shift;
    const bool windowed = boxes_per_tile <= 32;
    if (windowed && (win_base < 0 || slot0 < win_base || slot0 + boxes_per_tile > win_base + 32)) {
      win_base = slot0;
      win_page = win_base + lane < n_slots ? p.page_table[pt_row + win_base + lane] : 0;
    }
    constexpr int NHB = KV8 ? 1 : NH;                        // TMA boxes per row
    constexpr int ROWB = KV8 ? SM::RB8 : 128;                // bytes of one box row in shared memory
    if (lane == 0) mbar_expect_tx(full, (uint32_t)((nvb << box_shift) * HD * (KV8 ? 1 : 2)));
    __syncwarp();
    const uint32_t dst0 = KV8 ? sbase + SM::OFF_STG + (uint32_t)s * SM::STG_TILE
                              : sbase + RING_OFF + (uint32_t)s * SM::KV_TILE;
    for (int j0 = 0; j0 < boxes_per_tile * NHB; j0 += 32) {   // uniform trip count: the shuffle below is warp-wide
      const int j = j0 + lane;
      const int i = j / NHB, half = j - i * NHB;
      const int key = key0 + (i << box_shift);
      int page;
      if (windowed) page = __shfl_sync(0xffffffffu, win_page, ((key >> p_shift) - win_base) & 31);
      else page = (j < boxes_per_tile * NHB && i < nvb) ? p.page_table[pt_row + (key >> p_shift)] : 0;
      if (j >= boxes_per_tile * NHB || i >= nvb) continue;
      if ((unsigned)page >= (unsigned long long)p.n_pages) report(KB200_STATUS_BAD_PAGE, page, KID_PREFILL);
      const uint32_t dst = dst0 + (uint32_t)half * (BN * 128) + (uint32_t)(i << box_shift) * ROWB;
      tma_load_4d(dst, kv ? &tmV : &tmK, full, half * 64, key & (page_sz - 1), h, page);
    }
    return true;
  };
  if (tid == 0) {
    for (int s = 0; s < RINGB; ++s) {
      mbar_init(B_FULL(s), KV8 ? 128 : 1);   // filled by the TMA unit, or by the 128 widening threads
      mbar_init(B_EMPTY(s), 1);
    }
    for (int s = 0; s < SM::NSTG; ++s) {
      mbar_init(B_SFULL(s), 1);
      mbar_init(B_SEMPTY(s), 128);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(B_SREADY(x), 1);
      mbar_init(B_PREADY(x), 128);
      mbar_init(B_PVDONE(x), 1);
    }
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();   // barriers exist; nothing slow has started yet, so nobody waits here
  if (warp == 8 || (!KV8 && warp == 10)) {
    // 16-bit pools: two producer warps, one for the K tiles (even ring entries) and one for the V tiles;
    // issuing a tile's copies costs a warp ~130 cycles per box, too much for one warp at 32 boxes per
    // tile pair.  FP8 pools have half the boxes and one producer.  The other warps only meet the
    // producers again at the exit: their set-up barrier leaves them out.
    constexpr int NPROD = KV8 ? 1 : 2;
    for (int idx = warp == 8 ? 0 : 1; idx < 2 * n_tiles; idx += NPROD)
      if (!produce(idx)) break;
  } else if (KV8 && warp >= 10) {
    // =========================== widening warps (FP8 pools): one key row per thread ===========================
    // e4m3 tile as delivered by the TMA unit (rows of RB8 bytes, swizzled) -> f16 tile in the operand
    // layout of the MMAs (rows of 256 bytes in two 128-byte-swizzled slabs, or one slab for head_dim 64)
    constexpr int RB8 = SM::RB8;
    constexpr int NSTG = SM::NSTG > 0 ? SM::NSTG : 1;   // (this branch is only taken with a staging ring)
    const int r = (warp - 10) * 32 + lane;
    for (int idx = 0; idx < 2 * n_tiles; ++idx) {
      const int s8 = idx % NSTG, c = idx % RINGN;
      bool got = mbar_wait_bounded(B_SFULL(s8), (uint32_t)(idx / NSTG) & 1u);
      if (got && idx >= RINGN) got = mbar_wait_bounded(B_EMPTY(c), (uint32_t)((idx / RINGN) - 1) & 1u);
      if (!got) {
        if (lane == 0) report(KB200_STATUS_WAIT_TIMEOUT, idx, KID_PREFILL);
        break;
      }
      const uint8_t* src = sgen + SM::OFF_STG + s8 * SM::STG_TILE + r * RB8;
      uint8_t* dst = sgen + RING_OFF + c * SM::KV_TILE + r * 128;
#pragma unroll
      for (int ch = 0; ch < RB8 / 16; ++ch) {
        const uint4 x = *reinterpret_cast<const uint4*>(src + ((ch ^ (int)swz<RB8>(r)) << 4));
        uint4 lo4, hi4;   // elements 16ch .. 16ch+7 and 16ch+8 .. 16ch+15 as f16
        e4m3x4_to_f16x4(x.x, lo4.x, lo4.y);
        e4m3x4_to_f16x4(x.y, lo4.z, lo4.w);
        e4m3x4_to_f16x4(x.z, hi4.x, hi4.y);
        e4m3x4_to_f16x4(x.w, hi4.z, hi4.w);
        const int d0 = 2 * ch, d1 = 2 * ch + 1;   // 16-byte chunks of the f16 row
        *reinterpret_cast<uint4*>(dst + (d0 >> 3) * (BN * 128) + (((d0 & 7) ^ (r & 7)) << 4)) = lo4;
        *reinterpret_cast<uint4*>(dst + (d1 >> 3) * (BN * 128) + (((d1 & 7) ^ (r & 7)) << 4)) = hi4;
      }
      fence_proxy_async();          // the tensor core reads what was just written
      mbar_arrive(B_FULL(c));
      mbar_arrive(B_SEMPTY(s8));
    }
  } else {
    if (warp == 9) {
      tmem_alloc(sbase + SM::OFF_TMEM, TMEM_COLS);
      tmem_relinquish();
    }
    // Q rows -> shared memory in the K-major 128-byte-swizzled operand layout (tile A, then tile B);
    // rows past the segment's end are zero
    constexpr int CH = HD * 2 / 16;   // 16-byte chunks per row
    constexpr int NCOPY = kPfCopyThreads;
    constexpr int PER = (kPfCtaRows * CH + NCOPY - 1) / NCOPY;
    const int qt = tid < 256 ? tid : tid - 32;
    const int gshift = (p.group & (p.group - 1)) == 0 ? 31 - __clz(p.group) : -1;   // GQA groups are powers of two as a rule
    // all of a thread's loads are issued before the first store, so their latencies overlap
    uint4 val[PER];
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      const int i = qt + u * NCOPY;
      const int rr = i / CH, c = i - rr * CH;
      const int row = row_first + rr;
      val[u] = make_uint4(0u, 0u, 0u, 0u);
      if (i < kPfCtaRows * CH && row < nrows) {
        const int j = gshift >= 0 ? row >> gshift : row / p.group, g = row - j * p.group;
        const char* src = p.q + 2 * ((int64_t)b * p.q_bs + (int64_t)(qrow0 + j) * p.q_rs +
                                     (int64_t)(h * p.group + g) * p.q_hs) + 16 * c;
        val[u] = *reinterpret_cast<const uint4*>(src);
        if constexpr (KV8 && BF16) {   // bf16 -> f16 (exact unless |q| > 65504 or below the f16 subnormals)
          uint32_t* w32 = reinterpret_cast<uint32_t*>(&val[u]);
#pragma unroll
          for (int e = 0; e < 4; ++e)
            w32[e] = pack2<false>(bf16_bits_to_float(w32[e] & 0xffffu), bf16_bits_to_float(w32[e] >> 16));
        }
      }
    }
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      const int i = qt + u * NCOPY;
      if (i < kPfCtaRows * CH && !(SPLIT && i >= kPfTileRows * CH)) {   // (Q tile B is a ring slot under the key split)
        const int rr = i / CH, c = i - rr * CH;
        const int x = rr >> 7, r = rr & 127;
        const uint32_t off = SM::OFF_Q + (uint32_t)x * SM::Q_TILE + (uint32_t)(c >> 3) * SM::SLAB + (uint32_t)r * 128 +
                             (uint32_t)(((c & 7) ^ (r & 7)) << 4);
        *reinterpret_cast<uint4*>(sgen + off) = val[u];
      }
    }
    fence_proxy_async();   // generic-proxy writes above are read by the tensor core (async proxy)
    tc_fence_before();
    asm volatile("bar.sync 1, %0;" ::"n"(kPfCopyThreads) : "memory");   // warps 0-7 and 9
    tc_fence_after();
  }
  const uint32_t tmem_base = (warp == 8 || warp >= 10) ? 0u : *tmem_slot;

  if (warp == 8 || warp >= 10) {
    // (the producers and the widening warps have run to completion above)
  } else if (warp == 9) {
    // =========================== MMA issuer ===========================
    // Order per tile i:  PV_A(i)  QK_A(i+1)  PV_B(i)  QK_B(i+1): while one Q tile's softmax runs, the
    // tensor core works on the other's products.
    constexpr uint32_t IDESC_QK = umma_idesc(MMA_BF16, false, BN);
    constexpr uint32_t IDESC_PV = umma_idesc(MMA_BF16, true, HD);
    bool ok = true;
    auto kv_addr = [&](int idx) { return sbase + RING_OFF + (uint32_t)(idx % RINGN) * SM::KV_TILE; };
    auto kv_wait = [&](int idx) {
      ok = ok && mbar_wait_bounded(B_FULL(idx % RINGN), (uint32_t)(idx / RINGN) & 1u);
    };
    // Descriptors differ only in their start-address field (low 14 bits, units of 16 bytes): the
    // high word and the layout bits are built once, the per-step offsets are compile-time constants.
    constexpr uint32_t kDescHi = (uint32_t)((1024u >> 4) | (1u << 14) | (2u << 29));   // sbo = 1024, version, 128-byte swizzle
    constexpr uint32_t kLboK = (16u >> 4) << 16;                 // K-major operands: unused leading offset
    constexpr uint32_t kLboV = ((uint32_t)(BN * 128) >> 4) << 16;  // V (MN-major): distance between 64-column slabs
    auto mk = [](uint32_t lo) { return ((uint64_t)kDescHi << 32) | lo; };
    auto qk = [&](int x, int xq, int i) {   // S_x = Q_xq K_i^T
      tc_fence_after();
      if (lane == 0) {
        const uint32_t q_lo = ((sbase + SM::OFF_Q + (uint32_t)xq * SM::Q_TILE) >> 4) | kLboK;
        const uint32_t k_lo = (kv_addr(2 * i) >> 4) | kLboK;
        const uint32_t s_tmem = tmem_base + S_COL + (uint32_t)x * BN;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t oq = ((uint32_t)(k >> 2) * SM::SLAB + (uint32_t)(k & 3) * 32) >> 4;
          const uint32_t ok_ = ((uint32_t)(k >> 2) * (BN * 128) + (uint32_t)(k & 3) * 32) >> 4;
          umma_f16(s_tmem, mk(q_lo + oq), mk(k_lo + ok_), IDESC_QK, k > 0 ? 1u : 0u);
        }
        tc_commit(B_SREADY(x));
      }
      __syncwarp();
    };
    auto wait_p = [&](int x, int i) { ok = ok && mbar_wait_bounded(B_PREADY(x), (uint32_t)i & 1u); };
    auto pv = [&](int x, int i, int ksteps, bool acc) {   // O_x (+)= P_x V_i; acc: O_x holds earlier tiles
      if (!ok) return;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t p_tmem = tmem_base + P_OFF + (uint32_t)x * 128;   // (overlays the first 64 columns of S_x unless PSEP)
        const uint32_t v_lo = (kv_addr(2 * i + 1) >> 4) | kLboV;
        const uint32_t o_tmem = tmem_base + O_COL + (uint32_t)x * 128;
        if (ksteps == BN / 16) {
#pragma unroll
          for (int k = 0; k < BN / 16; ++k)
            umma_f16_ts(o_tmem, p_tmem + (uint32_t)k * 8, mk(v_lo + (uint32_t)k * (2048 >> 4)), IDESC_PV,
                        (acc || k > 0) ? 1u : 0u);
        } else {
          for (int k = 0; k < ksteps; ++k)
            umma_f16_ts(o_tmem, p_tmem + (uint32_t)k * 8, mk(v_lo + (uint32_t)k * (2048 >> 4)), IDESC_PV,
                        (acc || k > 0) ? 1u : 0u);
        }
        tc_commit(B_PVDONE(x));
      }
      __syncwarp();
    };
    // V rows between the sequence end and the end of its 16-key block may hold anything (NaN bit patterns
    // included) and would poison 0 * V: zero them (whole rows, so the swizzle does not matter)
    auto zero_v_tail = [&](int i, int nvalid, int ksteps) {
      const uint32_t v_off = kv_addr(2 * i + 1) - sbase;
      const int r0 = nvalid, r1 = ksteps << 4;
      for (int t = lane; t < (r1 - r0) * NH * 8; t += 32) {
        const int r = r0 + t / (NH * 8), c = t % (NH * 8);
        *reinterpret_cast<uint4*>(sgen + v_off + (uint32_t)(c >> 3) * (BN * 128) + (uint32_t)r * 128 +
                                  (uint32_t)((c & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
      }
      fence_proxy_async();
      __syncwarp();
    };
    if (split) {
      // pipeline x = i & 1 owns key tile i; per tile: P V of the tile, then Q K^T of the pipeline's next tile
      // (the other way round when P has columns of its own), while the other pipeline's softmax runs
      kv_wait(0);
      if (ok) {
        qk(0, 0, 0);
        if (lane == 0) tc_commit(B_EMPTY(0));
        __syncwarp();
        kv_wait(2);
      }
      if (ok) {
        qk(1, 0, 1);
        if (lane == 0) tc_commit(B_EMPTY(2 % RINGN));
        __syncwarp();
      }
      for (int i = 0; i < n_tiles && ok; ++i) {
        const int x = i & 1, li = i >> 1;
        kv_wait(2 * i + 1);
        if (!ok) break;
        int nvalid = L - (tile_begin + i) * BN;
        if (nvalid > BN) nvalid = BN;
        const int ksteps = (nvalid + 15) >> 4;
        if (nvalid & 15) zero_v_tail(i, nvalid, ksteps);
        const bool more = i + 2 < n_tiles;
        wait_p(x, li);
        if (!ok) break;
        if constexpr (PSEP) {
          if (more) {
            kv_wait(2 * (i + 2));
            if (!ok) break;
            qk(x, 0, i + 2);
          }
          pv(x, i, ksteps, li > 0);
        } else {
          pv(x, i, ksteps, li > 0);
          if (more) {
            kv_wait(2 * (i + 2));
            if (!ok) break;
            qk(x, 0, i + 2);
          }
        }
        if (lane == 0) {
          tc_commit(B_EMPTY((2 * i + 1) % RINGN));
          if (more) tc_commit(B_EMPTY((2 * i + 4) % RINGN));
        }
        __syncwarp();
      }
    } else if (n_tiles > 0) {
      kv_wait(0);
      if (ok) {
        if (n_x[0] > 0) qk(0, 0, 0);
        if (n_x[1] > 0) qk(1, 1, 0);
        if (lane == 0) tc_commit(B_EMPTY(0));
        __syncwarp();
      }
    }
    for (int i = 0; i < n_tiles && ok && !split; ++i) {
      kv_wait(2 * i + 1);
      if (!ok) break;
      const int key0 = (tile_begin + i) * BN;
      int nvalid = L - key0;
      if (nvalid > BN) nvalid = BN;
      const int ksteps = (nvalid + 15) >> 4;
      if (nvalid & 15) zero_v_tail(i, nvalid, ksteps);
      const bool more = i + 1 < n_tiles;
      if constexpr (PSEP) {
        // P_x has columns of its own: once the softmax has let go of S_x the next Q K^T goes first
        if (more) kv_wait(2 * (i + 1));
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (i < n_x[x]) {
            wait_p(x, i);
            if (!ok) break;
            if (i + 1 < n_x[x]) qk(x, x, i + 1);
            pv(x, i, ksteps, i > 0);
          }
        }
        if (!ok) break;
        if (lane == 0) {
          tc_commit(B_EMPTY((2 * i + 1) % RINGN));             // V_i has been read by both tiles
          if (more) tc_commit(B_EMPTY((2 * i + 2) % RINGN));   // K_{i+1} likewise
        }
        __syncwarp();
      } else {
        if (i < n_x[0]) { wait_p(0, i); pv(0, i, ksteps, i > 0); }
        if (more) kv_wait(2 * (i + 1));
        if (!ok) break;
        if (i + 1 < n_x[0]) qk(0, 0, i + 1);
        if (i < n_x[1]) { wait_p(1, i); pv(1, i, ksteps, i > 0); }
        if (!ok) break;
        if (lane == 0) tc_commit(B_EMPTY((2 * i + 1) % RINGN));   // V_i has been read by both tiles
        __syncwarp();
        if (more) {
          if (i + 1 < n_x[1]) qk(1, 1, i + 1);
          if (lane == 0) tc_commit(B_EMPTY((2 * i + 2) % RINGN));  // K_{i+1} likewise
          __syncwarp();
        }
      }
    }
    if (!ok && lane == 0) report(KB200_STATUS_WAIT_TIMEOUT, seg, KID_PREFILL);
  } else {
    // =========================== softmax: one row per thread, one warpgroup per Q tile ===========================
    const int x = warp >> 2;                 // Q tile (pipeline of the key split)
    const int r = tid & 127;                 // row inside the tile == tensor-memory lane
    const int row = row_first + (split ? 0 : x * kPfTileRows) + r;
    const bool valid = row < nrows;
    const int j = valid ? row / p.group : 0;
    const int g = valid ? row - j * p.group : 0;
    int jv = j;   // last row of this sequence whose key this row sees
    if (valid && p.q_vis) jv = max(j, min(sq - 1, p.q_vis[(int64_t)b * p.q_vis_bs + qrow0 + j]));
    // Rows past the segment's end are never written, and their tile must not hold the others back: no mask for
    // them (their Q rows are zero: every score is 0), and a warp without any row skips the arithmetic altogether.
    const int lim = valid ? (upper ? L - sq + jv : L - 1) : 0x3fffffff;             // last visible key
    const int lo = (valid && p.window_left >= 0) ? lim - p.window_left : 0;         // first visible key
    const bool warp_has_rows = row - lane < nrows;                                   // (the warp's first row)
    const float ksc = p.ks_vec ? p.ks_vec[h] : p.ks;
    const float vscale = p.vs_vec ? p.vs_vec[h] : p.vs;
    const float sl2 = p.softmax_scale * ksc * kLog2e;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_base + S_COL + (uint32_t)x * BN;
    const uint32_t o_tmem = tmem_base + lane_base + O_COL + (uint32_t)x * 128;
    const uint32_t p_st = tmem_base + lane_base + P_OFF + (uint32_t)x * 128;   // where this row's weights go
    const int n_mine = n_s[x];
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int it = 0; it < n_mine; ++it) {
      ok = mbar_wait_bounded(B_SREADY(x), (uint32_t)it & 1u);
      if (!ok) break;
      tc_fence_after();
      if (!warp_has_rows) {   // whatever S and P hold on these lanes only reaches rows of O that nobody reads
        // (still in step with the others on every barrier: a wait by parity must not fall two phases behind)
        if (it > 0) {
          ok = mbar_wait_bounded(B_PVDONE(x), (uint32_t)(it - 1) & 1u);
          if (!ok) break;
        }
        tc_fence_before();
        mbar_arrive(B_PREADY(x));
        continue;
      }
      const int key0 = (tile_begin + (split ? 2 * it + x : it)) * BN;
      const bool masked = key0 + BN - 1 > lim || key0 < lo;
      const int c_hi = lim - key0, c_lo = lo - key0;   // visible columns of this tile: c_lo <= column <= c_hi
      // pass 1: the row maximum; eight independent chains of three-input maxima (one chain of 128
      // dependent fmax would cost ~500 cycles)
      float mx8[8];
      if constexpr (KV8) {
        // (448 threads leave 128 registers per thread: 32 scores at a time, the next load in flight)
#pragma unroll
        for (int k = 0; k < 8; ++k) mx8[k] = -INFINITY;
        uint32_t raw[2][32];
        tmem_ld32_nowait(s_tmem, raw[0]);
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          tc_wait_ld();
          if (c + 1 < BN / 32) tmem_ld32_nowait(s_tmem + 32u * (c + 1), raw[(c + 1) & 1]);
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[c & 1][i]);
          if (masked) {
            if (c_lo <= 0) {   // only the upper limit cuts this tile (plain causal, or the window starts before it)
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (32 * c + i > c_hi) v[i] = -INFINITY;
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (32 * c + i > c_hi || 32 * c + i < c_lo) v[i] = -INFINITY;
            }
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) mx8[k] = max3(mx8[k], v[k], v[8 + k]);
#pragma unroll
          for (int k = 0; k < 8; ++k) mx8[k] = max3(mx8[k], v[16 + k], v[24 + k]);
        }
      } else {
        float s[BN];   // all 128 scores of the row at once
        tmem_ld128(s_tmem, s);
        if (masked) {
          if (c_lo <= 0) {   // only the upper limit cuts this tile (plain causal, or the window starts before it)
#pragma unroll
            for (int i = 0; i < BN; ++i)
              if (i > c_hi) s[i] = -INFINITY;
          } else {
#pragma unroll
            for (int i = 0; i < BN; ++i)
              if (i > c_hi || i < c_lo) s[i] = -INFINITY;
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) mx8[i] = s[i];
#pragma unroll
        for (int i = 8; i + 16 <= BN; i += 16) {
#pragma unroll
          for (int k = 0; k < 8; ++k) mx8[k] = max3(mx8[k], s[i + k], s[i + 8 + k]);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) mx8[k] = fmaxf(mx8[k], s[BN - 8 + k]);
      }
      const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])),
                             fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
      if (it == 0) {
        m = mx;   // the first product overwrites O: nothing to rescale
      } else {
        // the previous P V of this tile must have completed: P's buffer is free and O is at rest
        ok = mbar_wait_bounded(B_PVDONE(x), (uint32_t)(it - 1) & 1u);
        if (!ok) break;
        tc_fence_after();
        // Raise the running maximum only when it grew by more than 2^kRescaleStep (or was still
        // -inf): weights stay below 2^8 and O, kept in tensor memory, is rarely touched.
        const bool raise = mx > m && (m == -INFINITY || (mx - m) * sl2 > kRescaleStep);
        if (__any_sync(0xffffffffu, raise)) {
          const float f = raise ? (m == -INFINITY ? 0.f : ex2((m - mx) * sl2)) : 1.f;
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            float v[32];
            tmem_ld32(o_tmem + c * 32, v);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= f;
            tmem_st32(o_tmem + c * 32, v);
          }
          tc_wait_st();
          l *= f;
          if (raise) m = mx;
        }
      }
      const float ms = (m == -INFINITY) ? 0.f : m * sl2;
      float ls4[4] = {0.f, 0.f, 0.f, 0.f};   // independent partial row sums
      uint64_t ls2[4] = {0ull, 0ull, 0ull, 0ull};   // the same as packed pairs (bit pattern of 0.f, 0.f)
      const uint64_t sl2x2 = pack_f32x2(sl2, sl2), nmsx2 = pack_f32x2(-ms, -ms);
      // weights as packed 16-bit pairs over the first 64 columns of S_x: the A operand of P V.
      // S is read a second time, 32 columns at a time (keeping all 128 scores live across the
      // exponentials costs more in registers than the second read costs in time); chunk c of P
      // lands on columns [16c, 16c+16), inside S columns that are already in registers.
      uint32_t raw[2][32];   // the load of chunk c + 1 is in flight while chunk c is turned into weights
      tmem_ld32_nowait(s_tmem, raw[0]);
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        tc_wait_ld();
        if (c + 1 < BN / 32) tmem_ld32_nowait(s_tmem + 32u * (c + 1), raw[(c + 1) & 1]);
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[c & 1][i]);
        if (masked) {
          if (c_lo <= 0) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (32 * c + i > c_hi) v[i] = -INFINITY;
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (32 * c + i > c_hi || 32 * c + i < c_lo) v[i] = -INFINITY;
          }
        }
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(v[2 * i], v[2 * i + 1]), sl2x2, nmsx2), x0, x1);
          const float p0 = ex2(x0), p1 = ex2(x1);                  // exp2(-inf) = 0 for masked keys
          ls2[i & 3] = add_f32x2(ls2[i & 3], pack_f32x2(p0, p1));
          w[i] = pack2<MMA_BF16>(p0, p1);
        }
        tmem_st16u(p_st + 16u * c, w);
      }
      tc_wait_st();
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float a, b;
        unpack_f32x2(ls2[k], a, b);
        ls4[k] += a + b;
      }
      l += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
      // S has been read and P written: the tensor core may read P and then overwrite S
      tc_fence_before();
      mbar_arrive(B_PREADY(x));
    }
    if (ok && n_mine > 0) {
      ok = mbar_wait_bounded(B_PVDONE(x), (uint32_t)(n_mine - 1) & 1u);
      if (ok) tc_fence_after();
    }
    if (split) {
      // Combine the two pipelines.  Pipeline 1 parks its row (maximum in log2 units, sum, unnormalised O) in the
      // K/V ring, which is at rest once the last P V of both pipelines has completed; element (row, 4 columns c)
      // sits at (c * 128 + row) * 16 so that a warp's rows are side by side.
      uint8_t* xbuf = sgen + SM::OFF_KV;
      static_assert(HD * 512 + 128 * 8 <= RING * SM::KV_TILE, "the exchange buffer fits the K/V ring");
      const float m_own = (m == -INFINITY) ? -INFINITY : m * sl2;
      if (x == 1) {
        if (ok) ok = mbar_wait_bounded(B_PVDONE(0), (uint32_t)(n_s[0] - 1) & 1u);
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            float v[32];
            tmem_ld32(o_tmem + c * 32, v);
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *reinterpret_cast<float4*>(xbuf + ((c * 8 + q) * 128 + r) * 16) =
                  make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
          }
          *reinterpret_cast<float2*>(xbuf + HD * 512 + r * 8) = make_float2(m_own, l);
        }
      }
      if (!ok && lane == 0) report(KB200_STATUS_WAIT_TIMEOUT, seg, KID_PREFILL);
      asm volatile("bar.sync 2, 256;" ::: "memory");   // both softmax warpgroups, whatever happened above
      if (x == 0 && ok) {
        const float2 other = *reinterpret_cast<const float2*>(xbuf + HD * 512 + r * 8);
        const float M = fmaxf(m_own, other.x);
        const float w0 = (m_own == -INFINITY) ? 0.f : ex2(m_own - M);
        const float w1 = (other.x == -INFINITY) ? 0.f : ex2(other.x - M);
        const float lt = l * w0 + other.y * w1;
        const float inv = lt > 0.f ? vscale / lt : 0.f;
        const float f0 = w0 * inv, f1 = w1 * inv;
        const int hq = h * p.group + g;
        char* dst = p.out + 2 * ((int64_t)b * p.o_bs + (int64_t)(qrow0 + j) * p.o_rs + (int64_t)hq * p.o_hs);
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          float v[32];
          tmem_ld32(o_tmem + c * 32, v);
          if (valid) {
#pragma unroll
            for (int q8 = 0; q8 < 4; ++q8) {
              const float4 a = *reinterpret_cast<const float4*>(xbuf + ((c * 8 + 2 * q8) * 128 + r) * 16);
              const float4 bq = *reinterpret_cast<const float4*>(xbuf + ((c * 8 + 2 * q8 + 1) * 128 + r) * 16);
              uint4 w;
              w.x = pack2<BF16>(v[8 * q8 + 0] * f0 + a.x * f1, v[8 * q8 + 1] * f0 + a.y * f1);
              w.y = pack2<BF16>(v[8 * q8 + 2] * f0 + a.z * f1, v[8 * q8 + 3] * f0 + a.w * f1);
              w.z = pack2<BF16>(v[8 * q8 + 4] * f0 + bq.x * f1, v[8 * q8 + 5] * f0 + bq.y * f1);
              w.w = pack2<BF16>(v[8 * q8 + 6] * f0 + bq.z * f1, v[8 * q8 + 7] * f0 + bq.w * f1);
              *reinterpret_cast<uint4*>(dst + 64 * c + 16 * q8) = w;
            }
          }
        }
        if (valid && p.lse) {
          constexpr float kLn2 = 0.6931471805599453f;
          p.lse[(int64_t)b * p.lse_bs + (int64_t)hq * p.lse_hs + qrow0 + j] = lt > 0.f ? M * kLn2 + logf(lt) : -INFINITY;
        }
      }
    } else if (!ok) {
      if (lane == 0) report(KB200_STATUS_WAIT_TIMEOUT, seg, KID_PREFILL);
    } else if (row_first + x * kPfTileRows < nrows) {   // uniform per warpgroup: tensor-memory loads are warp-wide
      const float inv = l > 0.f ? vscale / l : 0.f;
      const int hq = h * p.group + g;
      char* dst = p.out + 2 * ((int64_t)b * p.o_bs + (int64_t)(qrow0 + j) * p.o_rs + (int64_t)hq * p.o_hs);
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        float v[32];
        if (n_mine > 0) {
          tmem_ld32(o_tmem + c * 32, v);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.f;
        }
        if (valid) {
#pragma unroll
          for (int q8 = 0; q8 < 4; ++q8) {
            uint4 w;
            w.x = pack2<BF16>(v[8 * q8 + 0] * inv, v[8 * q8 + 1] * inv);
            w.y = pack2<BF16>(v[8 * q8 + 2] * inv, v[8 * q8 + 3] * inv);
            w.z = pack2<BF16>(v[8 * q8 + 4] * inv, v[8 * q8 + 5] * inv);
            w.w = pack2<BF16>(v[8 * q8 + 6] * inv, v[8 * q8 + 7] * inv);
            *reinterpret_cast<uint4*>(dst + 64 * c + 16 * q8) = w;
          }
        }
      }
      if (valid && p.lse) {
        constexpr float kLn2 = 0.6931471805599453f;
        p.lse[(int64_t)b * p.lse_bs + (int64_t)hq * p.lse_hs + qrow0 + j] =
            l > 0.f ? m * sl2 * kLn2 + logf(l) : -INFINITY;
      }
    }
  }

  // ---- common exit: every role comes here, then the allocating warp frees the tensor memory
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
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

template <int HD, bool BF16, bool KV8, bool SPLIT>
inline int launch_prefill_split(const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p, int grid,
                                int dev, cudaStream_t stream) {
  using SM = PrefillSmem<HD, KV8>;
  auto kern = paged_prefill_kernel<HD, BF16, KV8, SPLIT>;
  static SmemAttrOnce once;
  if (int rc = once.ensure(kern, SM::BYTES, dev)) return rc;
  KB200_CUDA_OK(launch_kernel(kern, dim3(grid), dim3(pf_threads(KV8)), SM::BYTES, stream, tmK, tmV, p));
  return KB200_OK;
}

template <int HD, bool BF16, bool KV8>
inline int launch_prefill_variant(const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p, int grid,
                                  int dev, cudaStream_t stream) {
  // seqlen_q bounds the rows of every sequence (padded and packed layouts alike): at most 128 packed rows per
  // KV head means no CTA of the launch uses its second Q tile, and the key-split variant serves it
  if ((long long)p.group * p.seqlen_q <= kPfTileRows)
    return launch_prefill_split<HD, BF16, KV8, true>(tmK, tmV, p, grid, dev, stream);
  return launch_prefill_split<HD, BF16, KV8, false>(tmK, tmV, p, grid, dev, stream);
}

}  // namespace kb200
