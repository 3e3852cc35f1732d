// tcgen05 forward kernel for inputs that need no rotation in shared memory: q and k are either not
// rotated at all or are the rotated copies a streaming pass left behind (swa_fwd_rot).  Same mathematics,
// tile geometry, window mask and tensor-memory layout as fwd_kernel (swa_tc_fwd.cuh); what differs is who
// does what:
//
//   warp 0        TMA producer: query tile (double-buffered) and the ring of K / V halo blocks
//   warp 1        SCORE issuer: S = Q K^T (+ the window mask as 32 extra contraction columns)
//   warp 2        PV issuer:    O_g += P V with P read from tensor memory
//   warps 4-11    two softmax groups on alternate blocks, one thread per query row each, each with its own
//                 running maximum / sum and its own accumulator O_g
//   warps 12-15   one thread per row: window-mask penalty rows of every streamed block, and the EPILOGUE of
//                 every item: the two groups' partial results are merged (in an order fixed by block
//                 position), normalised and stored
//
// An item has only five to seven streamed blocks.  One warp issuing every MMA ran a dependent scalar
// instruction stream of about 2000 cycles per block while the tensor pipe needs less than half of
// that, and an epilogue inside the softmax groups idled both at every item boundary; hence two issuers
// (the order a single issuer gave for free becomes the barrier s_free) and epilogue warps.
// Measured and dropped: two threads per query row, each on half of every block's columns with the row maximum
// exchanged through shared memory (the softmax phase of a block halves, but both groups then work on the SAME
// block and the blocks of an item become strictly sequential: 1.47 ms per launch against 1.17 ms); rotating the
// query tile in warps 12-15 as well (about 400 dependent instructions
// per row cost 2700 cycles per item on the critical path, 1.1 ms per launch at the default workload,
// against 0.1 ms for a streaming pass over q), and a single warp writing all mask rows right behind the
// producer (four rows per lane made it the slowest role of the kernel).
//
// All waits are bounded; a timed-out wait raises a CTA-wide abort flag, every role runs its loops to the
// end without touching anything, TMEM is freed and the status word records it.
#pragma once

#include "swa_tc_fwd.cuh"

namespace swa {
namespace tc {

struct Fwd2Shared {
  uint64_t q_full[2], q_empty[2];
  uint64_t kv_full[kMaxStages], k_ready[kMaxStages], kv_empty[kMaxStages], kx_free[kMaxStages];
  uint64_t s_full[4], p_full[4], s_free[4], pv_done[2], o_full, o_free, ml_full[2], ml_empty[2];
  float ml[2][2][2][128];   // [item parity][group][maximum | sum][row]: handed to the epilogue warps
  uint32_t tmem_base;
  int abort_flag;
};

template <bool BF16>
__global__ void __launch_bounds__(kFwdThreads, 1)
fwd2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
            const __grid_constant__ CUtensorMap tm_v, KParams p, View4 o, float* __restrict__ lse) {
  using namespace ptx;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const Plan& pl = p.pl;
  const int N = pl.N;
  const uint32_t blk_bytes = (uint32_t)N * 128u;               // one 64-wide chunk of a streamed block
  const uint32_t q_bytes = p.qch * 16384u;
  const uint32_t k_stage = blk_bytes * p.qch, v_stage = blk_bytes * p.vch;
  const uint32_t kx_stage = (uint32_t)N * kXRowBytes;           // window-mask penalty rows of a streamed block
  const uint32_t o_cols = p.vch * 64u;                           // TMEM columns of one O accumulator
  const int nsb = pl.nsb;                                        // score buffers = look-ahead of the score MMAs
  // score buffer b at column s_stride*b (128-column strides when they fit, else packed), O_g behind them
  const uint32_t s_stride = (N <= 128 && nsb * 128u + 2 * o_cols <= kFwdTmemCols) ? 128u : (uint32_t)N;
  const uint32_t o_base = nsb * s_stride;
  uint8_t* q_smem = smem;                                        // two buffers
  uint8_t* qx_smem = q_smem + 2 * q_bytes;                      // window-mask indicator rows of a query tile
  uint8_t* k_smem = qx_smem + 128 * kXRowBytes;
  uint8_t* v_smem = k_smem + pl.stages * k_stage;
  uint8_t* kx_smem = v_smem + pl.stages * v_stage;
  Fwd2Shared* sh = reinterpret_cast<Fwd2Shared*>(kx_smem + pl.stages * kx_stage);
  PenView pen;                                                   // window-mask penalty parts of the current item's halo
  pen.row = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sh) + ((sizeof(Fwd2Shared) + 15) & ~size_t(15)));
  pen.col = pen.row + 2 * pl.pen_rows;
  pen.n_rows = pl.pen_rows;
  pen.n_cols = pl.pen_cols;
  volatile int* abort_flag = &sh->abort_flag;

  const int warp = threadIdx.x >> 5;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sh->q_full[s], 1);
      mbar_init(&sh->q_empty[s], 1);
      mbar_init(&sh->pv_done[s], 1);
      mbar_init(&sh->ml_full[s], 256);
      mbar_init(&sh->ml_empty[s], 128);
    }
    for (int s = 0; s < 4; ++s) {
      mbar_init(&sh->s_full[s], 1);
      mbar_init(&sh->p_full[s], 128);
      mbar_init(&sh->s_free[s], 1);
    }
    mbar_init(&sh->o_full, 1);
    mbar_init(&sh->o_free, 128);
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(&sh->kv_full[s], 1);
      mbar_init(&sh->k_ready[s], 128);
      mbar_init(&sh->kv_empty[s], 1);
      mbar_init(&sh->kx_free[s], 1);
    }
    sh->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, kFwdTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;

  bool ok = true;   // warp-uniform: a failed wait does not leave the loops, every later wait returns at once
  auto wait_spin = [&](uint64_t* bar, uint32_t parity) {
    const bool r = ok && mbar_wait<0>(bar, parity, abort_flag);
    ok = __all_sync(0xffffffffu, r);
  };
  auto wait_park = [&](uint64_t* bar, uint32_t parity) {
    const bool r = ok && mbar_wait<100>(bar, parity, abort_flag);
    ok = __all_sync(0xffffffffu, r);
  };
  const int n_items = p.n_items, tiles_per_head = pl.n_tiles_x * pl.n_tiles_y;

  // Registers follow the work: producer / issuer warpgroup 80, the two softmax warpgroups 152, the
  // rotation + mask + epilogue warpgroup keeps 128: (80 + 2 * 152 + 128) * 128 = 64 Ki.
  if (warp >= 4 && warp < 12) {
    setmaxnreg_inc<152>();
    // ------------------------------------------------------------------ softmax, one thread per query row and group
    const int lane = threadIdx.x & 31;
    const int g = (warp - 4) >> 2;                // group: takes the blocks whose stream position has parity g
    const int quarter = warp & 3;                 // TMEM lane quarter this warp may touch
    const int m = quarter * 32 + lane;
    const float none_thresh = -0.5f * p.mask_a * p.mask_b;     // a row maximum below this: every entry masked
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    const uint32_t o_tm = lane_base + o_base + g * o_cols;
    const float c2 = p.scale_log2;
    const int ng = N >> 4;                        // 16-column granules of a row
    uint32_t gbase = 0;                           // stream position of the current item's block 0
    uint32_t own_next = g, n_own = 0;             // this group's next block in the stream; blocks done so far
    int sbuf = g % nsb, spar = 0;                 // ... its score buffer and that buffer's barrier parity
    int tn = 0;
#pragma unroll 1
    for (int it = 0, item = blockIdx.x; item < n_items; ++it, item += gridDim.x) {
      const TilePos tp = tile_pos(p, item % tiles_per_head);
      // rows of the grid the 32 queries of this warp can see
      const int see_lo = tp.r0 + (quarter * 32) / pl.TW - p.wr, see_hi = tp.r0 + (quarter * 32 + 31) / pl.TW + p.wr;
      float m_used = -INFINITY, l = 0.f;
      int cnt = 0;                                // blocks of this item this group has handed to the PV MMA
#pragma unroll 1
      for (int j = (int)(own_next - gbase); j < tp.nblk; j += 2, own_next += 2, ++n_own, ++cnt) {
        const uint32_t s_tm = lane_base + sbuf * s_stride;
        uint64_t* const p_bar = &sh->p_full[sbuf];
        trace_ev(p, 2 + g, tn, m == 0 && it >= p.trace_it, 0 * 16 + (j & 15));
        wait_spin(&sh->s_full[sbuf], spar);
        trace_ev(p, 2 + g, tn, m == 0 && it >= p.trace_it, 1 * 16 + (j & 15));
        sbuf += 2;                                // two positions on in the ring of nsb buffers
        if (sbuf >= nsb) { sbuf -= nsb; spar ^= 1; }
        int band, cblk;
        block_pos(pl, j, band, cblk);
        const int blk_first = tp.hr_first + band * pl.KR, blk_last = blk_first + pl.KR - 1;
        const bool seen = !(blk_last < see_lo || blk_first > see_hi);
        if (ok) {
          tc_fence_after();
          uint32_t ra[16], rb[16];
          if (!seen) {
#pragma unroll
            for (int i = 0; i < 8; ++i) ra[i] = 0u;
#pragma unroll 1
            for (int c0 = 0; c0 < (N >> 1); c0 += 8) tmem_st8(s_tm + c0, ra);
          } else {
            // Two passes over the row in 16-column granules, the load of granule i+1 in flight while
            // granule i is worked on (a TMEM load takes ~150 cycles to come back).
            // pass 1: row maximum
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            tmem_ld16(s_tm, ra);
#pragma unroll 1
            for (int i = 0; i < ng; i += 2) {
              tmem_wait_ld();
              if (i + 1 < ng) tmem_ld16(s_tm + 16 * (i + 1), rb);
#pragma unroll
              for (int e = 0; e < 16; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(ra[e]));
              if (i + 1 < ng) {
                tmem_wait_ld();
                if (i + 2 < ng) tmem_ld16(s_tm + 16 * (i + 2), ra);
#pragma unroll
                for (int e = 0; e < 16; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(rb[e]));
              }
            }
            tmem_ld16(s_tm, ra);                            // first granule of pass 2, in flight during the bookkeeping
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            if (mx < none_thresh) mx = -INFINITY;
            // running max with lazy rescale: keep scaling by m_used until the true max exceeds it by 2^8
            bool need = false;
            float m_new = m_used;
            if (mx > m_used) {
              if (m_used == -INFINITY) m_used = mx;          // nothing accumulated yet for this row
              else if ((mx - m_used) * c2 > kRescaleThreshold) { need = true; m_new = mx; }
            }
            if (__any_sync(0xffffffffu, need) && cnt > 0) {
              // O_g must be at rest: wait for the PV MMA of this group's previous block, then scale the row
              wait_spin(&sh->pv_done[g], (n_own - 1) & 1);
              if (ok) {
                tc_fence_after();
                const float alpha = need ? exp2f((m_used - m_new) * c2) : 1.f;
                tmem_wait_ld();
#pragma unroll 1
                for (int c = 0; c < (int)o_cols; c += 16) {
                  tmem_ld16(o_tm + c, rb);
                  tmem_wait_ld();
#pragma unroll
                  for (int e = 0; e < 16; ++e) rb[e] = __float_as_uint(__uint_as_float(rb[e]) * alpha);
                  tmem_st16(o_tm + c, rb);
                }
                if (need) { m_used = m_new; l *= alpha; }
              }
            }
            const float mc = (m_used == -INFINITY) ? 0.f : m_used * c2;
            // pass 2: P = exp2(S*c - m), row sum, packed in place (P column c/2 <- S columns c, c+1)
            float ls4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
            for (int i = 0; i < ng; i += 2) {
              tmem_wait_ld();
              if (i + 1 < ng) tmem_ld16(s_tm + 16 * (i + 1), rb);
#pragma unroll
              for (int h = 0; h < 8; ++h) {
                const float p0 = exp2f(fmaf(__uint_as_float(ra[2 * h]), c2, -mc));
                const float p1 = exp2f(fmaf(__uint_as_float(ra[2 * h + 1]), c2, -mc));
                ls4[h & 3] += p0 + p1;
                ra[h] = pack2<BF16>(p0, p1);
              }
              tmem_st8(s_tm + 8 * i, ra);
              if (i + 1 < ng) {
                tmem_wait_ld();
                if (i + 2 < ng) tmem_ld16(s_tm + 16 * (i + 2), ra);
#pragma unroll
                for (int h = 0; h < 8; ++h) {
                  const float p0 = exp2f(fmaf(__uint_as_float(rb[2 * h]), c2, -mc));
                  const float p1 = exp2f(fmaf(__uint_as_float(rb[2 * h + 1]), c2, -mc));
                  ls4[h & 3] += p0 + p1;
                  rb[h] = pack2<BF16>(p0, p1);
                }
                tmem_st8(s_tm + 8 * (i + 1), rb);
              }
            }
            l += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
          }
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(p_bar);
        }
        trace_ev(p, 2 + g, tn, m == 0 && it >= p.trace_it, 2 * 16 + (j & 15));
      }
      // hand this group's running maximum and sum of the item to the epilogue warps
      if (it >= 2) wait_spin(&sh->ml_empty[it & 1], ((it >> 1) - 1) & 1);
      if (ok) {
        sh->ml[it & 1][g][0][m] = m_used;
        sh->ml[it & 1][g][1][m] = l;
        mbar_arrive(&sh->ml_full[it & 1]);
      }
      gbase += tp.nblk;
    }
  } else if (warp < 4) {
    setmaxnreg_dec<80>();
    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      if (elect_one()) {
        prefetch_tmap(&tm_q);
        prefetch_tmap(&tm_k);
        prefetch_tmap(&tm_v);
      }
      __syncwarp();
      int stage = 0, stage_par = 1;        // parity of the "empty" phase a refill of this stage waits for
      bool ring_full = false;              // all stages have been filled once
#pragma unroll 1
      for (int it = 0, item = blockIdx.x; item < n_items; ++it, item += gridDim.x) {
        const int bh = item / tiles_per_head, bi = bh / p.H, hi = bh - bi * p.H;
        const TilePos tp = tile_pos(p, item - bh * tiles_per_head);
        const int qb = it & 1;
        if (it >= 2) wait_park(&sh->q_empty[qb], ((it >> 1) - 1) & 1);
        if (ok && elect_one()) {
          mbar_arrive_expect_tx(&sh->q_full[qb], q_bytes);
#pragma unroll 1
          for (int c = 0; c < p.qch; ++c)
            tma_load_5d(q_smem + qb * q_bytes + c * 16384, &tm_q, &sh->q_full[qb], c * 64, tp.x0, tp.r0, hi, bi);
        }
        __syncwarp();
#pragma unroll 1
        for (int j = 0; j < tp.nblk; ++j) {
          if (ring_full) wait_park(&sh->kv_empty[stage], stage_par);
          if (ok && elect_one()) {
            mbar_arrive_expect_tx(&sh->kv_full[stage], k_stage + v_stage);
            int band, cblk;
            block_pos(pl, j, band, cblk);
            const int row = tp.hr_first + band * pl.KR, col = tp.hx0 + cblk * pl.KW;
#pragma unroll 1
            for (int c = 0; c < p.qch; ++c)
              tma_load_5d(k_smem + stage * k_stage + c * blk_bytes, &tm_k, &sh->kv_full[stage], c * 64, col, row, hi, bi);
#pragma unroll 1
            for (int c = 0; c < p.vch; ++c)
              tma_load_5d(v_smem + stage * v_stage + c * blk_bytes, &tm_v, &sh->kv_full[stage], c * 64, col, row, hi, bi);
          }
          __syncwarp();
          if (++stage == pl.stages) { stage = 0; stage_par ^= 1; ring_full = true; }
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------------ score issuer
      const uint32_t fmt = BF16 ? 1u : 0u;
      const uint32_t idesc_s = instr_desc(fmt, 128, N, 0, 0);
      const uint32_t hi_sw = smem_desc_hi(1024, true), hi_ns = smem_desc_hi(kXSbo, false);
      const uint64_t q_desc0 = smem_desc_from(smem_u32(q_smem), 16, hi_sw), k_desc0 = smem_desc_from(smem_u32(k_smem), 16, hi_sw),
                     qx_desc0 = smem_desc_from(smem_u32(qx_smem), kXLbo, hi_ns), kx_desc0 = smem_desc_from(smem_u32(kx_smem), kXLbo, hi_ns);
      const uint32_t k_stage16 = k_stage >> 4, kx_stage16 = kx_stage >> 4, blk16 = blk_bytes >> 4;
      int s_it = 0, s_j = 0, s_nblk = 1, s_stage = 0, s_stage_par = 0, s_buf = 0;
      uint32_t s_use = 0;                            // how often the ring of score buffers has wrapped
      int tn = 0;
      const bool tl = (threadIdx.x & 31) == 0;
      if (blockIdx.x < n_items) s_nblk = item_blocks(p, blockIdx.x, tiles_per_head);
#pragma unroll 1
      for (int s_item = blockIdx.x; s_item < n_items;) {
        const int qb = s_it & 1;
        trace_ev(p, 1, tn, tl && s_it >= p.trace_it, 2 * 16 + (s_j & 15));
        if (s_j == 0) wait_spin(&sh->q_full[qb], (s_it >> 1) & 1);
        wait_spin(&sh->kv_full[s_stage], s_stage_par);    // the block has landed ...
        wait_spin(&sh->k_ready[s_stage], s_stage_par);    // ... and its window-mask rows are written
        // the buffer is free once the PV MMA of the block that used it last has completed
        if (s_use >= 1) wait_spin(&sh->s_free[s_buf], (s_use - 1) & 1);
        if (ok) {
          tc_fence_after();
          if (elect_one()) {
            const uint32_t sd = tmem + s_buf * s_stride;
            uint64_t qd = q_desc0 + (uint64_t)(qb * (q_bytes >> 4)), kd = k_desc0 + (uint64_t)(s_stage * k_stage16);
            uint32_t acc = 0u;
#pragma unroll 1
            for (int c = 0; c < p.qch; ++c, qd += 1024 - 8, kd += blk16 - 8) {
#pragma unroll
              for (int k = 0; k < 4; ++k, qd += 2, kd += 2, acc = 1u) umma_ss(sd, qd, kd, idesc_s, acc);
            }
            const uint64_t kxd = kx_desc0 + (uint64_t)(s_stage * kx_stage16);
#pragma unroll
            for (int k = 0; k < 2; ++k)  // + indicator x penalty: the window mask
              umma_ss(sd, qx_desc0 + (uint64_t)(k * (kXStepBytes >> 4)), kxd + (uint64_t)(k * (kXStepBytes >> 4)), idesc_s, 1u);
            umma_commit(&sh->s_full[s_buf]);
            umma_commit(&sh->kx_free[s_stage]);                      // the mask rows of this stage may be overwritten
            if (s_j == s_nblk - 1) umma_commit(&sh->q_empty[qb]);   // last read of this query buffer
          }
          __syncwarp();
        }
        trace_ev(p, 1, tn, tl && s_it >= p.trace_it, 3 * 16 + (s_j & 15));
        if (++s_stage == pl.stages) { s_stage = 0; s_stage_par ^= 1; }
        if (++s_buf == nsb) { s_buf = 0; ++s_use; }
        if (++s_j == s_nblk) {
          s_j = 0;
          ++s_it;
          s_item += gridDim.x;
          if (s_item < n_items) s_nblk = item_blocks(p, s_item, tiles_per_head);
        }
      }
    } else if (warp == 2) {
      // ------------------------------------------------------------------ PV issuer: O_g += P V, P from tensor memory
      const uint32_t fmt = BF16 ? 1u : 0u;
      const uint32_t idesc_pv = instr_desc(fmt, 128, o_cols, 0, 1);
      const uint32_t hi_sw = smem_desc_hi(1024, true);
      const uint64_t v_desc0 = smem_desc_from(smem_u32(v_smem), blk_bytes, hi_sw);
      const uint32_t v_stage16 = v_stage >> 4;
      const int nks = N >> 4;
      int p_it = 0, p_j = 0, p_nblk = 1, p_stage = 0, p_buf = 0, p_buf_par = 0, p_grp = 0;
      int tn = 0;
      const bool tl = (threadIdx.x & 31) == 0;
      if (blockIdx.x < n_items) p_nblk = item_blocks(p, blockIdx.x, tiles_per_head);
#pragma unroll 1
      for (int p_item = blockIdx.x; p_item < n_items;) {
        const bool first = p_j < 2;                       // first block of this item for group p_grp: O_g starts over
        trace_ev(p, 6, tn, tl && p_it >= p.trace_it, 0 * 16 + (p_j & 15));
        wait_spin(&sh->p_full[p_buf], p_buf_par);
        if (first && p_it >= 1) wait_spin(&sh->o_free, (p_it - 1) & 1);   // the previous item's O_g has been read
        trace_ev(p, 6, tn, tl && p_it >= p.trace_it, 4 * 16 + (p_j & 15));
        if (ok) {
          tc_fence_after();
          if (elect_one()) {
            const uint32_t pa = tmem + p_buf * s_stride, od = tmem + o_base + p_grp * o_cols;
            uint64_t vd = v_desc0 + (uint64_t)(p_stage * v_stage16);
            uint32_t acc = first ? 0u : 1u;
#pragma unroll 1
            for (int ks = 0; ks < nks; ++ks, vd += 128, acc = 1u) umma_ts(od, pa + ks * 8, vd, idesc_pv, acc);
            umma_commit(&sh->s_free[p_buf]);
            umma_commit(&sh->kv_empty[p_stage]);
            umma_commit(&sh->pv_done[p_grp]);
            if (p_j == p_nblk - 1) umma_commit(&sh->o_full);
          }
          __syncwarp();
        }
        trace_ev(p, 6, tn, tl && p_it >= p.trace_it, 1 * 16 + (p_j & 15));
        p_grp ^= 1;
        if (++p_stage == pl.stages) p_stage = 0;
        if (++p_buf == nsb) { p_buf = 0; p_buf_par ^= 1; }
        if (++p_j == p_nblk) {
          p_j = 0;
          ++p_it;
          p_item += gridDim.x;
          if (p_item < n_items) p_nblk = item_blocks(p, p_item, tiles_per_head);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ query rotation, mask rows, epilogue (warps 12-15)
    const int t = (int)threadIdx.x - 384;          // 0..127: row of the query tile / of a streamed block
    const int quarter = warp & 3;
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    const float c2 = p.scale_log2;
    int tn = 0;
    write_indicator_row<BF16>(qx_smem, t, 0, 1, p);               // the same for every item
    const bool row_on = t < N;
    const int jr = t / pl.KW, jc = t % pl.KW;                     // this thread's row inside every streamed block
    // Epilogue of one item: merge the two groups' partial results of this thread's row and store it.
    // `gb` = stream position of the item's block 0, `nblk` = its blocks.
    auto epilogue = [&](int item, int it, uint32_t gb, int nblk) {
      const int bh = item / tiles_per_head, bi = bh / p.H, hi = bh - bi * p.H;
      const TilePos tp = tile_pos(p, item - bh * tiles_per_head);
      const int qr = tp.r0 + t / pl.TW, qx = tp.x0 + t % pl.TW;
      const bool q_in = qr < p.t_h && qx < p.Wtok;
      const int64_t tok = (int64_t)qr * p.Wtok + qx;
      const int par = it & 1;
      // the group that took the even blocks of the item, and how many blocks each parity had
      const int g_even = (int)(gb & 1u);
      const int cnt_e = (nblk + 1) >> 1, cnt_d = nblk >> 1;
      trace_ev(p, 5, tn, t == 0 && it >= p.trace_it, 0 * 16 + (it & 15));
      wait_spin(&sh->ml_full[par], (it >> 1) & 1);
      const float m_e = sh->ml[par][g_even][0][t], l_e = sh->ml[par][g_even][1][t];
      const float m_d = sh->ml[par][g_even ^ 1][0][t], l_d = sh->ml[par][g_even ^ 1][1][t];
      if (ok) mbar_arrive(&sh->ml_empty[par]);
      // Merge in an order fixed by the blocks' positions in the item (even ones first), not by which group
      // happened to get them: the result of a tile must not depend on the work that preceded it.
      const float mm = fmaxf(m_e, m_d);
      const float w_e = (m_e == -INFINITY) ? 0.f : exp2f((m_e - mm) * c2);
      const float w_d = (m_d == -INFINITY) ? 0.f : exp2f((m_d - mm) * c2);
      const float lt = fmaf(l_d, w_d, l_e * w_e);
      const float inv = 1.f / lt;
      const float f_e = w_e * inv, f_d = w_d * inv;
      const uint32_t o_even = lane_base + o_base + g_even * o_cols, o_odd = lane_base + o_base + (g_even ^ 1) * o_cols;
      T* orow = (T*)o.ptr + bi * o.s0 + hi * o.s1 + tok * o.s2;
      wait_spin(&sh->o_full, it & 1);
      trace_ev(p, 5, tn, t == 0 && it >= p.trace_it, 1 * 16 + (it & 15));
      if (ok) {
        tc_fence_after();
#pragma unroll 1
        for (int c0 = 0; c0 < p.dv; c0 += 32) {          // the real columns of O only
          uint32_t a[32], b[32];
          if (cnt_e > 0) tmem_ld32(o_even + c0, a);
          if (cnt_d > 0) tmem_ld32(o_odd + c0, b);
          tmem_wait_ld();
          if (c0 + 32 >= p.dv) {                       // everything has been read: the next item may accumulate
            tc_fence_before();
            mbar_arrive(&sh->o_free);
            trace_ev(p, 5, tn, t == 0 && it >= p.trace_it, 2 * 16 + (it & 15));
          }
          if (q_in) {
            uint4* dst = reinterpret_cast<uint4*>(orow + c0);
#pragma unroll
            for (int uu = 0; uu < 4; ++uu) {
              uint32_t w[4];
#pragma unroll
              for (int h = 0; h < 4; ++h) {
                const int i0 = uu * 8 + 2 * h;
                float v0 = 0.f, v1 = 0.f;
                if (cnt_e > 0) { v0 = __uint_as_float(a[i0]) * f_e; v1 = __uint_as_float(a[i0 + 1]) * f_e; }
                if (cnt_d > 0) { v0 = fmaf(__uint_as_float(b[i0]), f_d, v0); v1 = fmaf(__uint_as_float(b[i0 + 1]), f_d, v1); }
                w[h] = pack2<BF16>(v0, v1);
              }
              dst[uu] = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
        if (q_in) lse[(int64_t)bh * p.t_h * p.Wtok + tok] = mm * c2 + log2f(lt);
      }
      trace_ev(p, 5, tn, t == 0 && it >= p.trace_it, 3 * 16 + (it & 15));
    };

    int stage = 0, stage_par = 1;                    // parity of the "free" phase a rewrite of this stage's rows waits for
    bool ring_full = false;
    uint64_t pen_sig = ~0ull;                        // geometry the penalty tables in shared memory were built for
    uint32_t G = 0;                                  // stream position of the next block to prepare
    bool pend = false;                               // an item whose epilogue has not run yet
    int pend_item = 0, pend_it = 0, pend_nblk = 0;
    uint32_t pend_gb = 0, pend_G = 0;                // its first stream position; the position before which it runs
#pragma unroll 1
    for (int it = 0, item = blockIdx.x;; ++it, item += gridDim.x) {   // one extra round flushes the last epilogue
      const bool have = item < n_items;
      const int bh = have ? item / tiles_per_head : 0;
      TilePos tp;
      tp.r0 = tp.x0 = tp.hx0 = tp.hr_first = tp.hr_last = 0;
      tp.nblk = 0;
      if (have) tp = tile_pos(p, item - bh * tiles_per_head);
      const uint32_t gb = G;
      if (have) {
        // the tables depend only on how the halo is clipped by the grid: interior tiles share them
        const uint64_t sig = penalty_signature(p, tp);
        if (sig != pen_sig) {
          pen_sig = sig;
          named_bar_sync(5, 128);           // nobody still reads the previous tables
          build_penalty_view<BF16>(pen, t, p, tp, 128);
          named_bar_sync(5, 128);
        }
      }
#pragma unroll 1
      for (int j = 0;; ++j, ++G) {
        // These warps run ahead of the score MMAs by up to `stages` blocks (a stage's mask rows are free as soon as
        // the score MMA that read them has completed; the K / V data need not have landed).  The block at stream
        // position (last block of an item + score buffers + stages) is the first one they would have to wait for
        // until that item's last PV MMA has completed: the item's epilogue runs right before it (or at the end of
        // a later item that ends earlier, or after the last item), hidden behind that lead.
        const bool at_end = j >= tp.nblk;
        if (pend && (at_end || G >= pend_G)) {
          epilogue(pend_item, pend_it, pend_gb, pend_nblk);
          pend = false;
        }
        if (at_end) break;
        trace_ev(p, 4, tn, t == 0 && it >= p.trace_it, 0 * 16 + (j & 15));
        if (ring_full) wait_park(&sh->kx_free[stage], (uint32_t)stage_par);
        trace_ev(p, 4, tn, t == 0 && it >= p.trace_it, 1 * 16 + (j & 15));
        if (ok) {
          if (row_on) {
            int band, cblk;
            block_pos(pl, j, band, cblk);
            write_penalty_row_v(kx_smem + stage * kx_stage, t, pen, band * pl.KR + jr, cblk * pl.KW + jc, pl.TH >> 3, pl.TW >> 3);
          }
          fence_proxy_async_smem();
          mbar_arrive(&sh->k_ready[stage]);
        }
        trace_ev(p, 4, tn, t == 0 && it >= p.trace_it, 2 * 16 + (j & 15));
        if (++stage == pl.stages) { stage = 0; stage_par ^= 1; ring_full = true; }
      }
      if (!have) break;
      pend = true;
      pend_item = item;
      pend_it = it;
      pend_gb = gb;
      pend_nblk = tp.nblk;
      pend_G = G - 1 + (uint32_t)(pl.stages + nsb);
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // let whatever is still in flight (TMA, MMA) land before shared memory and TMEM are released
#pragma unroll 1
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    if (threadIdx.x == 0) report_abort(p.status, 6, 0);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kFwdTmemCols);
  }
}

}  // namespace tc
}  // namespace swa
