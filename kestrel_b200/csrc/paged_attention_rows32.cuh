// Split-KV attention for segments of up to 32 query rows (17 .. 32 packed rows per KV head: an 8-token
// verify at GQA 4, a 4-token verify at GQA 8, short prompt chunks).  Included by paged_attention.cuh,
// whose helpers, plan, cursor and tile producer it uses.
//
// The 16-row kernel would visit such a sequence's keys once per block of 16 rows; here a warp keeps two
// 16-row blocks and runs both against every K/V tile it has brought into shared memory, so the keys cross
// HBM (and the shared-memory ring) once.  What that costs is registers: two output accumulators (2 x 16 x
// head_dim fp32) leave no room for the Q fragments, which therefore live in shared memory (32 rows per warp,
// 128-byte-swizzled, already in the operand order of the MMAs) and are re-read with ldmatrix, one k-step
// pair at a time, while the K fragments of that k-step are used for both blocks.  8 warps x 2 stages, the
// flat tile space, partials and merge of the 16-row kernel; a partial of a 32-row segment takes two
// 16-row slots.
#pragma once

namespace kb200 {

template <int KVB, int HD, int NS>
struct Rows32Smem {
  using T = AttnTile<KVB, HD, 8, NS>;
  static constexpr int Q_ROW_BYTES = HD * 2;
  static constexpr int Q_WARP_BYTES = 32 * Q_ROW_BYTES;
  static constexpr int Q_OFF = (8 * NS * T::STAGE_BYTES + 8 * NS * 8 + 127) & ~127;   // after stages and barriers
  static constexpr int PLAN_OFF = Q_OFF + 8 * Q_WARP_BYTES;
  static constexpr int SMEM_BYTES = PLAN_OFF + 1024;   // + plan_smem_bytes(batch) at launch
};

template <int KVB, int HD, bool BF16, int NS, bool GATHER>
__global__ void __launch_bounds__(256, 1)
paged_attn_rows32_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                         const __grid_constant__ AttnParams p) {
  constexpr int NW = 8;
  using T = AttnTile<KVB, HD, NW, NS>;
  using L = Rows32Smem<KVB, HD, NS>;
  constexpr int TILE_N = T::TILE_N;
  constexpr int RB = T::RB;
  constexpr int NT8 = TILE_N / 8;    // score n-tiles per tile
  constexpr int NKS = TILE_N / 16;   // k-steps of P V
  constexpr int NOT = HD / 8;        // output n-tiles
  constexpr int QCH = HD / 8;        // 16-byte chunks per Q row
  constexpr float kLog2e = 1.4426950408889634f;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c4 = lane & 3, g8 = lane >> 2;
  const uint32_t my_stage0 = smem_base + (uint32_t)(warp * NS) * T::STAGE_BYTES;
  const uint32_t bar0 = smem_base + (uint32_t)(NW * NS) * T::STAGE_BYTES + (uint32_t)(warp * NS) * 8u;
  const uint32_t q_smem = smem_base + L::Q_OFF + (uint32_t)warp * L::Q_WARP_BYTES;
  uint8_t* q_gen = smem_gen + L::Q_OFF + warp * L::Q_WARP_BYTES;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NW * NS; ++i) mbar_init(smem_base + (uint32_t)(NW * NS) * T::STAGE_BYTES + 8u * i, 1);
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();
  pdl_launch_dependents();
  pdl_wait();   // the append (and a plan launch, if there was one) must have completed
  const PlanView plan = attention_cta_plan<NW * 32>(p, smem_gen + L::PLAN_OFF);
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

  // Lane-dependent parts of the ldmatrix addresses.  A 16-byte chunk c of row r sits at chunk (c & 8) |
  // ((c & 7) ^ (r & 7)); c = (even constant of the unrolled loop) + (a lane bit), r & 7 = lane & 7 everywhere, so
  // the swizzled chunk is (constant & 7) ^ t with a per-lane t, and four values of it cover every constant.
  const uint32_t q_lane = q_smem + (uint32_t)(lane & 15) * L::Q_ROW_BYTES;
  uint32_t q_x[4], v_x[4], k_x[2];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    q_x[j] = (uint32_t)((2 * j) ^ ((lane >> 4) ^ (lane & 7))) << 4;
    v_x[j] = (uint32_t)((2 * j) ^ ((lane >> 4) ^ (lane & 7))) << 4;
  }
  k_x[0] = (uint32_t)(lane & 7) * 128 + ((uint32_t)((lane >> 3) ^ (lane & 7)) << 4);
  k_x[1] = (uint32_t)(lane & 7) * 128 + ((uint32_t)(((lane >> 3) ^ (lane & 7)) ^ 4) << 4);
  const uint32_t v_lane = (uint32_t)(((lane >> 3) & 1) * 8 + (lane & 7)) * 128;

  float o[2][NOT][4];
  float mx[2][2], ls[2][2];    // running maximum and sum of rows g8 / g8 + 8 of each block
  int lim[2][2], rowi[2][2];
  bool valid[2][2];
  float sl2 = 0.f, lazy = 0.f, vscale = 1.f;
  int h = 0;
  bool two = false;            // the second block has rows at all (warp-uniform)
  bool fresh = true;
  long long piece_start = r0;

  for (int it = 0; it < my_tiles; ++it) {
    const long long g = r0 + it;
    if (fresh) {
      fresh = false;
      piece_start = g;
      const int mb = cc.seg % cc.nmb;
      h = cc.seg / cc.nmb;
      const int nrows = p.group * cc.sq;
      two = nrows > mb * 32 + 16;
      const bool upper = p.causal || p.window_left >= 0;
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int r = mb * 32 + blk * 16 + hf * 8 + g8;
          rowi[blk][hf] = r;
          valid[blk][hf] = r < nrows;
          lim[blk][hf] = upper ? cc.L - cc.sq + r / p.group : cc.L - 1;
          mx[blk][hf] = -INFINITY;
          ls[blk][hf] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < NOT; ++i) o[blk][i][0] = o[blk][i][1] = o[blk][i][2] = o[blk][i][3] = 0.f;
      }
      const float ksc = p.ks_vec ? p.ks_vec[h] : p.ks;
      vscale = p.vs_vec ? p.vs_vec[h] : p.vs;
      sl2 = p.softmax_scale * ksc * kLog2e;
      lazy = 8.f / sl2;

      // Q rows of the segment into this warp's shared-memory slice: row r at r * Q_ROW_BYTES, 16-byte chunk
      // c at (c & ~7) | ((c & 7) ^ (r & 7)); rows past the segment end are zero rows.  Lanes of a half-warp
      // (head_dim 128) or a quarter-warp (64) read one row's chunks side by side.
      __syncwarp();   // every lane has finished reading the previous segment's rows
      const int64_t qb = (int64_t)cc.b * p.q_bs;
#pragma unroll
      for (int i = 0; i < QCH; ++i) {
        const int c = lane + 32 * i;
        const int r = c / QCH, gc = c % QCH;
        const int R = mb * 32 + r;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (R < nrows) {
          const int j = R / p.group, gq = R - j * p.group;
          v = *reinterpret_cast<const uint4*>(p.q + 2 * (qb + (int64_t)(cc.qr + j) * p.q_rs +
                                                         (int64_t)(h * p.group + gq) * p.q_hs) + 16 * gc);
        }
        uint8_t* row = q_gen + r * L::Q_ROW_BYTES;
        if constexpr (KVB == 2) {
          *reinterpret_cast<uint4*>(row + (((gc & ~7) | ((gc & 7) ^ (r & 7))) << 4)) = v;
        } else {
          // e4m3 K rows are read four consecutive d per thread, so within each group of 16 d Q is stored in the
          // k-slot order of the MMA: d = 4c + {0, 1} -> slots 2c, 2c + 1; d = 4c + {2, 3} -> slots 2c + 8, 2c + 9.
          // This chunk holds d = 8 * gc .. + 7: c = 2 * (gc & 1) and the next, of the group gc >> 1.
          if (p.q_is_bf16) {
            v.x = pack2<false>(bf16_bits_to_float(v.x & 0xffffu), bf16_bits_to_float(v.x >> 16));
            v.y = pack2<false>(bf16_bits_to_float(v.y & 0xffffu), bf16_bits_to_float(v.y >> 16));
            v.z = pack2<false>(bf16_bits_to_float(v.z & 0xffffu), bf16_bits_to_float(v.z >> 16));
            v.w = pack2<false>(bf16_bits_to_float(v.w & 0xffffu), bf16_bits_to_float(v.w >> 16));
          }
          const int grp = gc >> 1, byte = 8 * (gc & 1);
          const int ca = 2 * grp, cb = 2 * grp + 1;
          *reinterpret_cast<uint2*>(row + (((ca & ~7) | ((ca & 7) ^ (r & 7))) << 4) + byte) = make_uint2(v.x, v.z);
          *reinterpret_cast<uint2*>(row + (((cb & ~7) | ((cb & 7) ^ (r & 7))) << 4) + byte) = make_uint2(v.y, v.w);
        }
      }
      __syncwarp();
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

    // address of the A fragment (16 rows x 16 k-slots) of block blk, k-step ks
    auto q_frag_addr = [&](int blk, int ks) {   // (blk and ks are constants of the unrolled loops)
      return q_lane + q_x[ks & 3] + (uint32_t)(blk * 16 * L::Q_ROW_BYTES + ((2 * ks) & 8) * 16);
    };

    // ---- S = Q K^T for both blocks; every K fragment is loaded (and widened) once
    float s[2][NT8][4];
#pragma unroll
    for (int blk = 0; blk < 2; ++blk)
#pragma unroll
      for (int n = 0; n < NT8; ++n) s[blk][n][0] = s[blk][n][1] = s[blk][n][2] = s[blk][n][3] = 0.f;
    if constexpr (KVB == 2) {
#pragma unroll
      for (int q4 = 0; q4 < HD / 32; ++q4) {
        uint32_t qa[2][2][4];
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
          ldsm_x4(qa[blk][0][0], qa[blk][0][1], qa[blk][0][2], qa[blk][0][3], q_frag_addr(blk, 2 * q4));
          ldsm_x4(qa[blk][1][0], qa[blk][1][1], qa[blk][1][2], qa[blk][1][3], q_frag_addr(blk, 2 * q4 + 1));
        }
#pragma unroll
        for (int n = 0; n < NT8; ++n) {
          // row n * 8 + (lane & 7), chunk q4 * 4 + (lane >> 3) of the tile
          const uint32_t addr = kbase + k_x[q4 & 1] + (uint32_t)((q4 >> 1) * (TILE_N * 128) + n * 8 * 128);
          uint32_t b0, b1, b2, b3;
          ldsm_x4(b0, b1, b2, b3, addr);
#pragma unroll
          for (int blk = 0; blk < 2; ++blk) {
            mma16816<BF16>(s[blk][n], qa[blk][0], b0, b1);
            mma16816<BF16>(s[blk][n], qa[blk][1], b2, b3);
          }
        }
      }
    } else {
#pragma unroll
      for (int q4 = 0; q4 < HD / 64; ++q4) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {   // two 16-d groups at a time: their Q fragments of both blocks fit the registers
          uint32_t qa[2][2][4];
#pragma unroll
          for (int blk = 0; blk < 2; ++blk) {
            ldsm_x4(qa[blk][0][0], qa[blk][0][1], qa[blk][0][2], qa[blk][0][3], q_frag_addr(blk, q4 * 4 + 2 * hh));
            ldsm_x4(qa[blk][1][0], qa[blk][1][1], qa[blk][1][2], qa[blk][1][3], q_frag_addr(blk, q4 * 4 + 2 * hh + 1));
          }
#pragma unroll
          for (int n = 0; n < NT8; ++n) {
            const int r = n * 8 + (lane & 7);
            const int ch = q4 * 4 + 2 * hh + ((lane >> 3) & 1);   // (lanes 0-15 give the addresses of an x2)
            const uint32_t addr = kbase + (uint32_t)r * RB + ((uint32_t)(ch ^ swz<RB>(r)) << 4);
            uint32_t x0, x1;
            ldsm_x2(x0, x1, addr);
            uint32_t b0, b1;
            e4m3x4_to_f16x4(x0, b0, b1);
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
              mma16816<false>(s[blk][n], qa[blk][0], b0, b1);
            }
            e4m3x4_to_f16x4(x1, b0, b1);
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
              mma16816<false>(s[blk][n], qa[blk][1], b0, b1);
            }
          }
        }
      }
    }

    // ---- mask (only tiles that touch a boundary), online softmax (base 2), weights as A fragments
    const int key_last = key0 + TILE_N - 1;
    const int min_lim = (p.causal || p.window_left >= 0) ? cc.L - cc.sq : cc.L - 1;
    const bool need_mask = key_last > min_lim || (p.window_left >= 0 && key0 < cc.L - 1 - p.window_left);
    uint32_t pf[2][NKS][4];
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      if (need_mask) {
        const int lo0 = p.window_left >= 0 ? lim[blk][0] - p.window_left : 0;
        const int lo1 = p.window_left >= 0 ? lim[blk][1] - p.window_left : 0;
#pragma unroll
        for (int n = 0; n < NT8; ++n) {
          const int k = key0 + n * 8 + 2 * c4;
          if (k > lim[blk][0] || k < lo0) s[blk][n][0] = -INFINITY;
          if (k + 1 > lim[blk][0] || k + 1 < lo0) s[blk][n][1] = -INFINITY;
          if (k > lim[blk][1] || k < lo1) s[blk][n][2] = -INFINITY;
          if (k + 1 > lim[blk][1] || k + 1 < lo1) s[blk][n][3] = -INFINITY;
        }
      }
      float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
      for (int n = 0; n < NT8; ++n) {
        t0 = fmaxf(t0, fmaxf(s[blk][n][0], s[blk][n][1]));
        t1 = fmaxf(t1, fmaxf(s[blk][n][2], s[blk][n][3]));
      }
      t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1));
      t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
      t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1));
      t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
      // The reference maximum of a row is only raised when the scores outgrew it by more than 2^8 (`lazy`, in
      // score units): weights stay <= 256, exact after the final normalisation, and the 16 x head_dim rescale of
      // O is skipped for most tiles.
      float m0 = mx[blk][0], m1 = mx[blk][1];
      if (__any_sync(0xffffffffu, t0 > m0 + lazy || t1 > m1 + lazy)) {
        const float mn0 = fmaxf(m0, t0), mn1 = fmaxf(m1, t1);
        const float c0 = (m0 == -INFINITY) ? 0.f : ex2((m0 - mn0) * sl2);
        const float c1 = (m1 == -INFINITY) ? 0.f : ex2((m1 - mn1) * sl2);
        ls[blk][0] *= c0;
        ls[blk][1] *= c1;
#pragma unroll
        for (int i = 0; i < NOT; ++i) {
          o[blk][i][0] *= c0; o[blk][i][1] *= c0; o[blk][i][2] *= c1; o[blk][i][3] *= c1;
        }
        mx[blk][0] = m0 = mn0;
        mx[blk][1] = m1 = mn1;
      }
      const float ms0 = (m0 == -INFINITY) ? 0.f : m0 * sl2;
      const float ms1 = (m1 == -INFINITY) ? 0.f : m1 * sl2;
#pragma unroll
      for (int n = 0; n < NT8; ++n) {
        const float p0 = ex2(fmaf(s[blk][n][0], sl2, -ms0));
        const float p1 = ex2(fmaf(s[blk][n][1], sl2, -ms0));
        const float p2 = ex2(fmaf(s[blk][n][2], sl2, -ms1));
        const float p3 = ex2(fmaf(s[blk][n][3], sl2, -ms1));
        ls[blk][0] += p0 + p1;
        ls[blk][1] += p2 + p3;
        pf[blk][n >> 1][(n & 1) * 2 + 0] = pack2<BF16>(p0, p1);
        pf[blk][n >> 1][(n & 1) * 2 + 1] = pack2<BF16>(p2, p3);
      }
    }

    // ---- O += P V for both blocks; rows of V past the sequence end are zeroed in the one tile that has them
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
        [[maybe_unused]] const int row = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
        if constexpr (KVB == 2) {
#pragma unroll
          for (int q2 = 0; q2 < HD / 16; ++q2) {
            // row ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), chunk q2 * 2 + (lane >> 4)
            const uint32_t addr = vbase + v_lane + v_x[q2 & 3] + (uint32_t)((q2 >> 2) * (TILE_N * 128) + ks * 16 * 128);
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(b0, b1, b2, b3, addr);
            if constexpr (MASKED) { b0 &= mk_lo; b1 &= mk_hi; b2 &= mk_lo; b3 &= mk_hi; }
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
              mma16816<BF16>(o[blk][2 * q2], pf[blk][ks], b0, b1);
              mma16816<BF16>(o[blk][2 * q2 + 1], pf[blk][ks], b2, b3);
            }
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
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
              mma16816<false>(o[blk][4 * q2 + 0], pf[blk][ks], e0, e1);  // d = 16*(2*q2)   + 2g
              mma16816<false>(o[blk][4 * q2 + 1], pf[blk][ks], o0, o1);  // d = 16*(2*q2)   + 2g + 1
            }
            e4m3x4_to_f16x4(x2, e0, o0);
            e4m3x4_to_f16x4(x3, e1, o1);
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
              mma16816<false>(o[blk][4 * q2 + 2], pf[blk][ks], e0, e1);  // d = 16*(2*q2+1) + 2g
              mma16816<false>(o[blk][4 * q2 + 3], pf[blk][ks], o0, o1);  // d = 16*(2*q2+1) + 2g + 1
            }
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
      const bool whole = seg_end && (g - piece_start == cc.nt - 1);
      const int seg_id = cc.segbase + cc.seg;
      const bool obf = KVB == 2 ? BF16 : (p.q_is_bf16 != 0);
      constexpr float kLn2 = 0.6931471805599453f;
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
        if (blk == 1 && !two) continue;   // (no rows: nothing to write, and the merge reads no rows past the end)
        float l0 = ls[blk][0], l1 = ls[blk][1];
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
        const float m0 = mx[blk][0], m1 = mx[blk][1];
        if (whole) {
          const float i0 = l0 > 0.f ? vscale / l0 : 0.f;
          const float i1 = l1 > 0.f ? vscale / l1 : 0.f;
          const int64_t ob = (int64_t)cc.b * p.o_bs;
          const int qr = cc.qr;
          const int row0 = rowi[blk][0], row1 = rowi[blk][1];
          const bool valid0 = valid[blk][0], valid1 = valid[blk][1];
          const int j0 = row0 / p.group, j1 = row1 / p.group;
          const int hq0 = h * p.group + row0 % p.group, hq1 = h * p.group + row1 % p.group;
          char* out0 = p.out + 2 * (ob + (int64_t)(qr + j0) * p.o_rs + (int64_t)hq0 * p.o_hs);
          char* out1 = p.out + 2 * (ob + (int64_t)(qr + j1) * p.o_rs + (int64_t)hq1 * p.o_hs);
          if constexpr (KVB == 2) {
#pragma unroll
            for (int i = 0; i < NOT; ++i) {
              const int d = 8 * i + 2 * c4;
              if (valid0) *reinterpret_cast<uint32_t*>(out0 + 2 * d) = pack2<BF16>(o[blk][i][0] * i0, o[blk][i][1] * i0);
              if (valid1) *reinterpret_cast<uint32_t*>(out1 + 2 * d) = pack2<BF16>(o[blk][i][2] * i1, o[blk][i][3] * i1);
            }
          } else {
#pragma unroll
            for (int ch = 0; ch < HD / 16; ++ch) {
              const int d = 16 * ch + 4 * c4;
              const float a0 = o[blk][2 * ch][0] * i0, a1 = o[blk][2 * ch + 1][0] * i0, a2 = o[blk][2 * ch][1] * i0,
                          a3 = o[blk][2 * ch + 1][1] * i0;
              const float b0 = o[blk][2 * ch][2] * i1, b1 = o[blk][2 * ch + 1][2] * i1, b2 = o[blk][2 * ch][3] * i1,
                          b3 = o[blk][2 * ch + 1][3] * i1;
              if (valid0)
                *reinterpret_cast<uint2*>(out0 + 2 * d) = obf ? make_uint2(pack2<true>(a0, a1), pack2<true>(a2, a3))
                                                              : make_uint2(pack2<false>(a0, a1), pack2<false>(a2, a3));
              if (valid1)
                *reinterpret_cast<uint2*>(out1 + 2 * d) = obf ? make_uint2(pack2<true>(b0, b1), pack2<true>(b2, b3))
                                                              : make_uint2(pack2<false>(b0, b1), pack2<false>(b2, b3));
            }
          }
          if (p.lse && c4 == 0) {
            if (valid0) p.lse[(int64_t)cc.b * p.lse_bs + (int64_t)hq0 * p.lse_hs + qr + j0] =
                l0 > 0.f ? m0 * sl2 * kLn2 + logf(l0) : -INFINITY;
            if (valid1) p.lse[(int64_t)cc.b * p.lse_bs + (int64_t)hq1 * p.lse_hs + qr + j1] =
                l1 > 0.f ? m1 * sl2 * kLn2 + logf(l1) : -INFINITY;
          }
        } else {
          const int64_t slot = ((int64_t)seg_id + w) * 2 + blk;
          float* po = p.part_o + slot * (kRowsPerSeg * HD);
          float* pml = p.part_ml + slot * (kRowsPerSeg * 2);
          const bool wv0 = valid[blk][0], wv1 = valid[blk][1];   // rows past the end: not written, not read by the merge
          if (c4 == 0) {
            if (wv0) *reinterpret_cast<float2*>(pml + g8 * 2) = make_float2((m0 == -INFINITY) ? -INFINITY : m0 * sl2, l0);
            if (wv1) *reinterpret_cast<float2*>(pml + (g8 + 8) * 2) = make_float2((m1 == -INFINITY) ? -INFINITY : m1 * sl2, l1);
          }
          if constexpr (KVB == 2) {
#pragma unroll
            for (int i = 0; i < NOT; ++i) {
              const int d = 8 * i + 2 * c4;
              if (wv0) *reinterpret_cast<float2*>(po + g8 * HD + d) = make_float2(o[blk][i][0], o[blk][i][1]);
              if (wv1) *reinterpret_cast<float2*>(po + (g8 + 8) * HD + d) = make_float2(o[blk][i][2], o[blk][i][3]);
            }
          } else {
#pragma unroll
            for (int ch = 0; ch < HD / 16; ++ch) {
              const int d = 16 * ch + 4 * c4;
              if (wv0)
                *reinterpret_cast<float4*>(po + g8 * HD + d) =
                    make_float4(o[blk][2 * ch][0], o[blk][2 * ch + 1][0], o[blk][2 * ch][1], o[blk][2 * ch + 1][1]);
              if (wv1)
                *reinterpret_cast<float4*>(po + (g8 + 8) * HD + d) =
                    make_float4(o[blk][2 * ch][2], o[blk][2 * ch + 1][2], o[blk][2 * ch][3], o[blk][2 * ch + 1][3]);
            }
          }
        }
      }
      fresh = true;
    }
    if (it + 1 < my_tiles) cursor_advance(p, plan, cc);
  }
}

}  // namespace kb200
