// tcgen05 backward kernels for inputs that need no rotation in shared memory: q and k are either
// not rotated at all or are the rotated copies an earlier kernel left behind (NE > 0: the gradients
// are rotated back to the un-rotated tensors in the epilogue).  Same mathematics, tile geometry,
// window mask and tensor-memory layout as bwd_kernel (swa_tc_bwd.cuh); what differs is who does what:
//
//   warp 0        TMA producer: resident tile (double-buffered) and the ring of streamed blocks
//   warp 1        SCORE issuer:  S = X_qk Y_qk^T (+ mask), dP = X_v Y_v^T into the block's (S, dP) pair
//   warp 2        ACCUMULATE issuer: dV += P^T dO, dK += dS^T Q  resp.  dQ += dS K, A operand in tensor memory
//   warps 4-11    two compute groups, one thread per resident row each, on alternate blocks
//   warps 12-15   one thread per row: window-mask penalty rows and lse / delta of every streamed block,
//                 and the EPILOGUE of every item (accumulators -> registers -> inverse rotation -> global)
//
// Why two issuers and epilogue warps: an item has only five to seven streamed blocks, and one warp that
// issues every MMA of the kernel runs a dependent scalar instruction stream of about 2000 cycles per block
// (waits, descriptor arithmetic, commits) next to busy compute warps, while the tensor pipe needs about
// 850 cycles for the same block; and an epilogue inside the compute groups idles both of them at every item
// boundary.  With the score and the accumulating MMAs issued by different warps the two instruction
// streams run side by side; the order the single issuer gave for free ("the accumulating MMAs of the
// block that used this pair last were issued before") becomes one more barrier, pair_free, that the
// accumulate issuer commits and the score issuer waits for.
// Measured and dropped: two compute threads per resident row, each on half of every block's columns (a block's
// compute phase halves, but both groups then work on the SAME block, the blocks of an item become strictly
// sequential and dK/dV went from 2.14 to 2.59 ms per launch).
//
// All waits are bounded; a timed-out wait raises a CTA-wide abort flag, every role runs its loops to the
// end without touching anything, TMEM is freed and the status word records it.
#pragma once

#include "swa_tc_bwd.cuh"

namespace swa {
namespace tc {

struct Bwd2Shared {
  uint64_t x_full[2], x_empty[2];
  uint64_t y_full[kMaxStages], y_ready[kMaxStages], y_empty[kMaxStages], yx_free[kMaxStages];
  uint64_t sd_full[2], ds_full[2], pair_free[2], acc_full, acc_free;
  uint64_t vec_ready[kMaxStages + 2];   // dK/dV: the lse / delta slot of a block is written (one barrier per slot)
  uint32_t tmem_base;
  int abort_flag;
  int abort_site;
};

// NE: width of the inverse rotation of dQ / dK in the epilogue (n_rdim / 8; 0 = none); TABS: the cos/sin
// tables are staged in shared memory (the planner does that when it costs no stage of the block ring).
template <bool BF16, bool DKDV, int NE, bool TABS>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd2_kernel(const __grid_constant__ CUtensorMap tm_xqk, const __grid_constant__ CUtensorMap tm_xv,
            const __grid_constant__ CUtensorMap tm_yqk, const __grid_constant__ CUtensorMap tm_yv, KParams p,
            const float* __restrict__ lse, const float* __restrict__ delta, View4 out_qk, View4 out_v) {
  using namespace ptx;
  constexpr int R = NE > 0 ? 8 * NE : 8;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const Plan& pl = p.pl;
  const int N = pl.N, nxb = pl.nxb;
  constexpr int nsb = 2;                                         // (S, dP) buffer pairs: group g owns pair g
  const uint32_t blk_bytes = (uint32_t)N * 128u;               // one 64-wide chunk of a streamed block
  const uint32_t xqk_bytes = p.qch * 16384u, xv_bytes = p.vch * 16384u, x_bytes = xqk_bytes + xv_bytes;
  const uint32_t yqk_stage = blk_bytes * p.qch, yv_stage = blk_bytes * p.vch;
  const uint32_t yx_stage = (uint32_t)N * kXRowBytes;
  uint8_t* x_smem = smem;                                        // nxb buffers of (qk chunks, v chunks)
  uint8_t* xx_smem = x_smem + nxb * x_bytes;                    // window-mask indicator rows of a resident tile
  uint8_t* yqk_smem = xx_smem + 128 * kXRowBytes;
  uint8_t* yv_smem = yqk_smem + pl.stages * yqk_stage;
  uint8_t* yx_smem = yv_smem + pl.stages * yv_stage;
  // -lse / delta of the streamed queries (dK/dV): a ring of stages + 2 slots [slot][-lse | delta][128], two deeper
  // than the block ring because the warps that fill it run ahead of the loads
  float* vec_smem = reinterpret_cast<float*>(yx_smem + pl.stages * yx_stage);
  const int vslots = pl.stages + 2;
  Bwd2Shared* sh = reinterpret_cast<Bwd2Shared*>(reinterpret_cast<uint8_t*>(vec_smem) + vslots * 1024);
  PenView pen;                                                   // window-mask penalty parts of the current item's halo
  pen.row = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sh) + ((sizeof(Bwd2Shared) + 15) & ~size_t(15)));
  pen.col = pen.row + 2 * pl.pen_rows;
  pen.n_rows = pl.pen_rows;
  pen.n_cols = pl.pen_cols;
  uint8_t* tab_smem = reinterpret_cast<uint8_t*>(pen.col + 2 * pl.pen_cols);   // cos/sin tables (TABS)
  volatile int* abort_flag = &sh->abort_flag;
  // tensor memory: buffer pair b = (S at 2N b, dP at 2N b + N), accumulators behind the pairs
  const uint32_t acc_qk = nsb * 2 * N, acc_v = acc_qk + p.qch * 64;

  const int warp = threadIdx.x >> 5;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sh->x_full[s], 1);
      mbar_init(&sh->x_empty[s], 1);
      mbar_init(&sh->sd_full[s], 1);
      mbar_init(&sh->ds_full[s], 128);
      mbar_init(&sh->pair_free[s], 1);
    }
    mbar_init(&sh->acc_full, 1);
    mbar_init(&sh->acc_free, 128);
    for (int s = 0; s < kMaxStages + 2; ++s) mbar_init(&sh->vec_ready[s], 128);
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(&sh->y_full[s], 1);
      mbar_init(&sh->y_ready[s], 128);
      mbar_init(&sh->y_empty[s], 1);
      mbar_init(&sh->yx_free[s], 1);
    }
    sh->abort_flag = 0;
    sh->abort_site = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, kBwdTmemCols);
    tmem_relinquish();
  }
  if constexpr (TABS) stage_rope_tables(tab_smem, p.rope, threadIdx.x, kBwdThreads);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;

  bool ok = true;   // warp-uniform: a failed wait does not leave the loops, every later wait returns at once
  auto wait_spin = [&](uint64_t* bar, uint32_t parity, int site) {
    const bool was = ok;
    const bool r = ok && mbar_wait<0>(bar, parity, abort_flag);
    ok = __all_sync(0xffffffffu, r);
    if (was && !ok && (threadIdx.x & 31) == 0) atomicCAS(&sh->abort_site, 0, site);
  };
  auto wait_park = [&](uint64_t* bar, uint32_t parity, int site) {
    const bool was = ok;
    const bool r = ok && mbar_wait<100>(bar, parity, abort_flag);
    ok = __all_sync(0xffffffffu, r);
    if (was && !ok && (threadIdx.x & 31) == 0) atomicCAS(&sh->abort_site, 0, site);
  };
  const int n_items = p.n_items, tiles_per_head = pl.n_tiles_x * pl.n_tiles_y;

  // Registers follow the work: producer / issuer warpgroup 80, the two compute warpgroups 152, the
  // mask + epilogue warpgroup keeps 128: (80 + 2 * 152 + 128) * 128 = 64 Ki.
  if (warp >= 4 && warp < 12) {
    setmaxnreg_inc<152>();
    // ------------------------------------------------------------------ P / dS, one thread per resident row and group
    const int lane = threadIdx.x & 31;
    const int g = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int m = quarter * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    const float c2 = p.scale_log2;
    const int ng = N >> 4;
    uint32_t gbase = 0, own_next = g;
    int tn = 0;
    const uint32_t s_tm = lane_base + g * 2 * N, d_tm = s_tm + N;
    uint64_t* const ds_bar = &sh->ds_full[g];
    int buf_par = 0;
    int vslot = g, vpar = 0;                       // slot of the lse / delta ring of this group's next block, its barrier parity
#pragma unroll 1
    for (int it = 0, item = blockIdx.x; item < n_items; ++it, item += gridDim.x) {
      const int bh = item / tiles_per_head;
      const TilePos tp = tile_pos(p, item - bh * tiles_per_head);
      const int see_lo = tp.r0 + (quarter * 32) / pl.TW - p.wr, see_hi = tp.r0 + (quarter * 32 + 31) / pl.TW + p.wr;
      float my_nlse = -INFINITY, my_delta = 0.f;     // dQ: -lse and delta of this thread's query
      if (!DKDV) {
        const int tr = tp.r0 + m / pl.TW, tx = tp.x0 + m % pl.TW;
        if (tr < p.t_h && tx < p.Wtok) {
          const int64_t at = (int64_t)bh * p.t_h * p.Wtok + (int64_t)tr * p.Wtok + tx;
          my_nlse = -__ldg(lse + at);
          my_delta = __ldg(delta + at);
        }
      }
#pragma unroll 1
      for (int j = (int)(own_next - gbase); j < tp.nblk; j += 2, own_next += 2) {
        trace_ev(p, 2 + g, tn, m == 0 && it >= p.trace_it, 0 * 16 + (j & 15));
        wait_spin(&sh->sd_full[g], buf_par, 7);
        trace_ev(p, 2 + g, tn, m == 0 && it >= p.trace_it, 1 * 16 + (j & 15));
        const float* vec = vec_smem + vslot * 256;
        // -lse / delta of the block's queries are staged.  One barrier per slot of that ring, not the stage's
        // y_ready: the warps that fill the slots run ahead of the block ring and may complete a stage's y_ready twice
        // before this warp has looked at it, but they cannot refill a slot before this warp has read it (see there).
        if (DKDV) wait_spin(&sh->vec_ready[vslot], vpar, 8);
        vslot += 2;
        if (vslot >= vslots) { vslot -= vslots; vpar ^= 1; }
        buf_par ^= 1;
        int band, cblk;
        block_pos(pl, j, band, cblk);
        const int blk_first = tp.hr_first + band * pl.KR, blk_last = blk_first + pl.KR - 1;
        const bool seen = !(blk_last < see_lo || blk_first > see_hi);
        if (ok) {
          tc_fence_after();
          uint32_t sa[16], sb[16], da[16], db[16];
          if (!seen) {            // none of this warp's 32 rows can see the block: P = dS = 0
#pragma unroll
            for (int i = 0; i < 8; ++i) sa[i] = 0u;
#pragma unroll 1
            for (int c0 = 0; c0 < (N >> 1); c0 += 8) {
              tmem_st8(s_tm + c0, sa);
              if (DKDV) tmem_st8(d_tm + c0, sa);
            }
          } else {
            // 16 columns at a time, the loads of the next 16 in flight while these are worked on
            auto work = [&](int i, uint32_t* s, uint32_t* d) {
              uint32_t wp[8];
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                float nl[4], dl[4];
                if constexpr (DKDV) {
                  const float4 a = *reinterpret_cast<const float4*>(vec + 16 * i + 4 * q4);
                  const float4 b = *reinterpret_cast<const float4*>(vec + 128 + 16 * i + 4 * q4);
                  nl[0] = a.x; nl[1] = a.y; nl[2] = a.z; nl[3] = a.w;
                  dl[0] = b.x; dl[1] = b.y; dl[2] = b.z; dl[3] = b.w;
                } else {
                  nl[0] = nl[1] = nl[2] = nl[3] = my_nlse;
                  dl[0] = dl[1] = dl[2] = dl[3] = my_delta;
                }
                float pv[4], dsv[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  pv[e] = exp2f(fmaf(__uint_as_float(s[4 * q4 + e]), c2, nl[e]));
                  dsv[e] = pv[e] * (__uint_as_float(d[4 * q4 + e]) - dl[e]);
                }
                s[2 * q4] = pack2<BF16>(dsv[0], dsv[1]);
                s[2 * q4 + 1] = pack2<BF16>(dsv[2], dsv[3]);
                if constexpr (DKDV) {
                  wp[2 * q4] = pack2<BF16>(pv[0], pv[1]);
                  wp[2 * q4 + 1] = pack2<BF16>(pv[2], pv[3]);
                }
              }
              if constexpr (DKDV) {
                tmem_st8(s_tm + 8 * i, wp);      // P^T over S^T
                tmem_st8(d_tm + 8 * i, s);       // dS^T over dP^T
              } else {
                tmem_st8(s_tm + 8 * i, s);       // dS over S
              }
            };
            tmem_ld16(s_tm, sa);
            tmem_ld16(d_tm, da);
#pragma unroll 1
            for (int i = 0; i < ng; i += 2) {
              tmem_wait_ld();
              if (i + 1 < ng) { tmem_ld16(s_tm + 16 * (i + 1), sb); tmem_ld16(d_tm + 16 * (i + 1), db); }
              work(i, sa, da);
              if (i + 1 < ng) {
                tmem_wait_ld();
                if (i + 2 < ng) { tmem_ld16(s_tm + 16 * (i + 2), sa); tmem_ld16(d_tm + 16 * (i + 2), da); }
                work(i + 1, sb, db);
              }
            }
          }
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(ds_bar);
        }
        trace_ev(p, 2 + g, tn, m == 0 && it >= p.trace_it, 2 * 16 + (j & 15));
      }
      gbase += tp.nblk;
    }
  } else if (warp < 4) {
    setmaxnreg_dec<80>();
    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      if (elect_one()) {
        prefetch_tmap(&tm_xqk);
        prefetch_tmap(&tm_xv);
        prefetch_tmap(&tm_yqk);
        prefetch_tmap(&tm_yv);
      }
      __syncwarp();
      int stage = 0, stage_par = 1;
      bool ring_full = false;
      int xb = 0, xb_par = 1;
      bool x_ring_full = false;
      int tn = 0;
      const bool tl = (threadIdx.x & 31) == 0;
#pragma unroll 1
      for (int it = 0, item = blockIdx.x; item < n_items; ++it, item += gridDim.x) {
        const int bh = item / tiles_per_head, bi = bh / p.H, hi = bh - bi * p.H;
        const TilePos tp = tile_pos(p, item - bh * tiles_per_head);
        if (x_ring_full) wait_park(&sh->x_empty[xb], xb_par, 1);
        if (ok && elect_one()) {
          mbar_arrive_expect_tx(&sh->x_full[xb], x_bytes);
          uint8_t* dst = x_smem + xb * x_bytes;
#pragma unroll 1
          for (int c = 0; c < p.qch; ++c) tma_load_5d(dst + c * 16384, &tm_xqk, &sh->x_full[xb], c * 64, tp.x0, tp.r0, hi, bi);
#pragma unroll 1
          for (int c = 0; c < p.vch; ++c) tma_load_5d(dst + xqk_bytes + c * 16384, &tm_xv, &sh->x_full[xb], c * 64, tp.x0, tp.r0, hi, bi);
        }
        __syncwarp();
        if (++xb == nxb) { xb = 0; xb_par ^= 1; x_ring_full = true; }
#pragma unroll 1
        for (int j = 0; j < tp.nblk; ++j) {
          trace_ev(p, 0, tn, tl && it >= p.trace_it, 0 * 16 + (j & 15));
          if (ring_full) wait_park(&sh->y_empty[stage], stage_par, 2);
          trace_ev(p, 0, tn, tl && it >= p.trace_it, 1 * 16 + (j & 15));
          if (ok && elect_one()) {
            mbar_arrive_expect_tx(&sh->y_full[stage], yqk_stage + yv_stage);
            int band, cblk;
            block_pos(pl, j, band, cblk);
            const int row = tp.hr_first + band * pl.KR, col = tp.hx0 + cblk * pl.KW;
#pragma unroll 1
            for (int c = 0; c < p.qch; ++c)
              tma_load_5d(yqk_smem + stage * yqk_stage + c * blk_bytes, &tm_yqk, &sh->y_full[stage], c * 64, col, row, hi, bi);
#pragma unroll 1
            for (int c = 0; c < p.vch; ++c)
              tma_load_5d(yv_smem + stage * yv_stage + c * blk_bytes, &tm_yv, &sh->y_full[stage], c * 64, col, row, hi, bi);
          }
          __syncwarp();
          if (++stage == pl.stages) { stage = 0; stage_par ^= 1; ring_full = true; }
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------------ score issuer: S (+ mask) and dP of every block
      const uint32_t fmt = BF16 ? 1u : 0u;
      const uint32_t idesc_s = instr_desc(fmt, 128, N, 0, 0);                 // both operands K-major
      const uint32_t hi_sw = smem_desc_hi(1024, true), hi_ns = smem_desc_hi(kXSbo, false);
      const uint64_t x_desc0 = smem_desc_from(smem_u32(x_smem), 16, hi_sw),
                     yqk_desc0 = smem_desc_from(smem_u32(yqk_smem), 16, hi_sw), yv_desc0 = smem_desc_from(smem_u32(yv_smem), 16, hi_sw),
                     xx_desc0 = smem_desc_from(smem_u32(xx_smem), kXLbo, hi_ns), yx_desc0 = smem_desc_from(smem_u32(yx_smem), kXLbo, hi_ns);
      const uint32_t yqk16 = yqk_stage >> 4, yv16 = yv_stage >> 4, yx16 = yx_stage >> 4, blk16 = blk_bytes >> 4, x16 = x_bytes >> 4;
      int s_it = 0, s_j = 0, s_nblk = 1, s_stage = 0, s_stage_par = 0, s_buf = 0, s_xb = 0, s_xb_par = 0;
      uint32_t G = 0;                                  // position in the CTA's stream of blocks
      int tn = 0;
      const bool tl = (threadIdx.x & 31) == 0;
      if (blockIdx.x < n_items) s_nblk = item_blocks(p, blockIdx.x, tiles_per_head);
#pragma unroll 1
      for (int s_item = blockIdx.x; s_item < n_items;) {
        trace_ev(p, 1, tn, tl && s_it >= p.trace_it, 2 * 16 + (s_j & 15));
        if (s_j == 0) wait_spin(&sh->x_full[s_xb], s_xb_par, 5);
        wait_spin(&sh->y_full[s_stage], s_stage_par, 12);    // the block has landed ...
        wait_spin(&sh->y_ready[s_stage], s_stage_par, 6);    // ... and its mask rows (and lse / delta) are written
        // the pair is free once the accumulating MMAs of the block that used it last have completed
        if (G >= 2) wait_spin(&sh->pair_free[s_buf], ((G >> 1) - 1) & 1, 11);
        if (ok) {
          tc_fence_after();
          if (elect_one()) {
            const uint32_t s_tm = tmem + s_buf * 2 * N, d_tm = s_tm + N;
            uint64_t xd = x_desc0 + (uint64_t)(s_xb * x16), yd = yqk_desc0 + (uint64_t)(s_stage * yqk16);
            uint32_t acc = 0u;
#pragma unroll 1
            for (int c = 0; c < p.qch; ++c, xd += 1024 - 8, yd += blk16 - 8) {
#pragma unroll
              for (int k = 0; k < 4; ++k, xd += 2, yd += 2, acc = 1u) umma_ss(s_tm, xd, yd, idesc_s, acc);
            }
            const uint64_t yxd = yx_desc0 + (uint64_t)(s_stage * yx16);
#pragma unroll
            for (int k = 0; k < 2; ++k)  // + indicator x penalty: the window mask
              umma_ss(s_tm, xx_desc0 + (uint64_t)(k * (kXStepBytes >> 4)), yxd + (uint64_t)(k * (kXStepBytes >> 4)), idesc_s, 1u);
            // xd now points at the v chunks of the resident tile
            yd = yv_desc0 + (uint64_t)(s_stage * yv16);
            acc = 0u;
#pragma unroll 1
            for (int c = 0; c < p.vch; ++c, xd += 1024 - 8, yd += blk16 - 8) {
#pragma unroll
              for (int k = 0; k < 4; ++k, xd += 2, yd += 2, acc = 1u) umma_ss(d_tm, xd, yd, idesc_s, acc);
            }
            umma_commit(&sh->sd_full[s_buf]);
            umma_commit(&sh->yx_free[s_stage]);                        // the mask rows of this stage may be overwritten
            if (s_j == s_nblk - 1) umma_commit(&sh->x_empty[s_xb]);   // last read of this resident buffer
          }
          __syncwarp();
        }
        trace_ev(p, 1, tn, tl && s_it >= p.trace_it, 3 * 16 + (s_j & 15));
        ++G;
        s_buf ^= 1;
        if (++s_stage == pl.stages) { s_stage = 0; s_stage_par ^= 1; }
        if (++s_j == s_nblk) {
          s_j = 0;
          ++s_it;
          s_item += gridDim.x;
          if (++s_xb == nxb) { s_xb = 0; s_xb_par ^= 1; }
          if (s_item < n_items) s_nblk = item_blocks(p, s_item, tiles_per_head);
        }
      }
    } else if (warp == 2) {
      // ------------------------------------------------------------------ accumulate issuer: A operands come from tensor memory
      const uint32_t fmt = BF16 ? 1u : 0u;
      const uint32_t idesc_qk = instr_desc(fmt, 128, p.qch * 64, 0, 1);       // dQ / dK: B = streamed qk tile, MN-major
      const uint32_t idesc_v = instr_desc(fmt, 128, p.vch * 64, 0, 1);        // dV: B = streamed dO tile, MN-major
      const uint32_t hi_sw = smem_desc_hi(1024, true);
      const uint64_t yqk_mn0 = smem_desc_from(smem_u32(yqk_smem), blk_bytes, hi_sw), yv_mn0 = smem_desc_from(smem_u32(yv_smem), blk_bytes, hi_sw);
      const uint32_t yqk16 = yqk_stage >> 4, yv16 = yv_stage >> 4;
      const int nks = N >> 4;
      int a_it = 0, a_j = 0, a_nblk = 1, a_stage = 0, a_buf = 0, a_buf_par = 0;
      int tn = 0;
      const bool tl = (threadIdx.x & 31) == 0;
      if (blockIdx.x < n_items) a_nblk = item_blocks(p, blockIdx.x, tiles_per_head);
#pragma unroll 1
      for (int a_item = blockIdx.x; a_item < n_items;) {
        trace_ev(p, 6, tn, tl && a_it >= p.trace_it, 0 * 16 + (a_j & 15));
        wait_spin(&sh->ds_full[a_buf], a_buf_par, 3);
        if (a_j == 0 && a_it >= 1) wait_spin(&sh->acc_free, (a_it - 1) & 1, 4);   // the previous item's accumulators have been read
        trace_ev(p, 6, tn, tl && a_it >= p.trace_it, 4 * 16 + (a_j & 15));
        if (ok) {
          tc_fence_after();
          if (elect_one()) {
            const uint32_t s_tm = tmem + a_buf * 2 * N, d_tm = s_tm + N;
            const uint32_t acc0 = a_j == 0 ? 0u : 1u;
            uint64_t bqk = yqk_mn0 + (uint64_t)(a_stage * yqk16);
            if constexpr (DKDV) {
              uint64_t bv = yv_mn0 + (uint64_t)(a_stage * yv16);
              uint32_t acc = acc0;
#pragma unroll 1
              for (int ks = 0; ks < nks; ++ks, bv += 128, acc = 1u) umma_ts(tmem + acc_v, s_tm + ks * 8, bv, idesc_v, acc);   // dV += P^T dO
              acc = acc0;
#pragma unroll 1
              for (int ks = 0; ks < nks; ++ks, bqk += 128, acc = 1u) umma_ts(tmem + acc_qk, d_tm + ks * 8, bqk, idesc_qk, acc);   // dK += dS^T Q
            } else {
              uint32_t acc = acc0;
#pragma unroll 1
              for (int ks = 0; ks < nks; ++ks, bqk += 128, acc = 1u) umma_ts(tmem + acc_qk, s_tm + ks * 8, bqk, idesc_qk, acc);   // dQ += dS K
            }
            umma_commit(&sh->pair_free[a_buf]);
            umma_commit(&sh->y_empty[a_stage]);
            if (a_j == a_nblk - 1) umma_commit(&sh->acc_full);
          }
          __syncwarp();
        }
        trace_ev(p, 6, tn, tl && a_it >= p.trace_it, 1 * 16 + (a_j & 15));
        if (++a_stage == pl.stages) a_stage = 0;
        a_buf ^= 1;
        if (a_buf == 0) a_buf_par ^= 1;
        if (++a_j == a_nblk) {
          a_j = 0;
          ++a_it;
          a_item += gridDim.x;
          if (a_item < n_items) a_nblk = item_blocks(p, a_item, tiles_per_head);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ mask rows + lse / delta of every block; epilogue of every item
    const int t = (int)threadIdx.x - 384;          // 0..127: row of the resident tile (epilogue) / of a streamed block (mask)
    const int quarter = warp & 3;
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    const bool rope_on = NE > 0 && p.rope.idx != nullptr;
    const float scale = p.sm_scale;
    const uint32_t tab_row = smem_u32(tab_smem), tab_col = tab_row + (uint32_t)p.rope.max_h * rope_tab_stride(R);
    int tn = 0;
    write_indicator_row<BF16>(xx_smem, t, 0, 1, p);               // the same for every item
    const bool row_on = t < N;
    const int jr = t / pl.KW, jc = t % pl.KW;                     // this thread's row inside every streamed block

    // Epilogue of one item: this thread's row of the accumulators goes tensor memory -> registers -> global 16 columns
    // (and, where rotated, their 16 partner columns) at a time.  Only a few dozen values are ever live: holding a
    // whole 64-column row made the rotating variants of this kernel 0.2 ms per launch slower than the plain ones
    // (register pressure in one role degrades the code of all roles of a kernel).  Tensor memory is released when
    // the last column has been read.
    int32_t pend_packed = -1;                        // packed RoPE index of this thread's row of the pending item
    auto epilogue = [&](int item, int it) {
      const int bh = item / tiles_per_head, bi = bh / p.H, hi = bh - bi * p.H;
      const TilePos tp = tile_pos(p, item - bh * tiles_per_head);
      const int tr = tp.r0 + t / pl.TW, tx = tp.x0 + t % pl.TW;
      const bool t_in = tr < p.t_h && tx < p.Wtok;
      const int64_t tok = (int64_t)tr * p.Wtok + tx;
      int irow = -1, icol = -1;
      if (rope_on && t_in) decode_idx(pend_packed, p.rope.max_h, p.rope.max_w, irow, icol);
      T* qk_row = (T*)out_qk.ptr + bi * out_qk.s0 + hi * out_qk.s1 + tok * out_qk.s2;
      const int dqk = p.dqk;                       // the real head dims: columns beyond them hold zeros and are not stored
      // rotated dims [0, 4R): row-angle pairs (i, i + R) in [0, 2R), column-angle pairs in [2R, 4R).  One rotated step =
      // NP pairs: columns [c0, c0 + NP) with their partners [c0 + R, c0 + R + NP).
      constexpr int NP = (R >= 16 && TABS) ? 16 : 8;   // tables in global memory: 8, the prefetched (cos, sin) values take registers
      constexpr int SPS = R / NP;                      // steps per segment
      const int nrot = (NE > 0 && rope_on) ? 2 * SPS : 0;
      // Tables in global memory (too large to stage): the (cos, sin) values of a step are fetched one step ahead --
      // those of the first step before the wait for the accumulators -- and the dV columns are stored between the
      // rotated steps, so that the L2 latency of the fetch is covered by work instead of being paid once per step.
      float4 cs[NP / 2];
      auto fetch = [&](int r) {
        if constexpr (NE > 0 && !TABS) {
          const int seg = r / SPS, i0 = (r - seg * SPS) * NP, pos = seg ? icol : irow;
          if (pos >= 0) {
            const float4* t4 = reinterpret_cast<const float4*>((seg ? p.rope.col_cs : p.rope.row_cs) + ((int64_t)pos * R + i0) * 2);
#pragma unroll
            for (int e = 0; e < NP / 2; ++e) cs[e] = __ldg(t4 + e);
          }
        }
      };
      if (nrot > 0) fetch(0);
      trace_ev(p, 5, tn, t == 0 && it >= p.trace_it, 0 * 16 + (it & 15));
      wait_spin(&sh->acc_full, it & 1, 9);
      trace_ev(p, 5, tn, t == 0 && it >= p.trace_it, 1 * 16 + (it & 15));
      if (ok) {
        tc_fence_after();
        [[maybe_unused]] T* v_row = qk_row;
        if constexpr (DKDV) v_row = (T*)out_v.ptr + bi * out_v.s0 + hi * out_v.s1 + tok * out_v.s2;
        const int dv = DKDV ? p.dv : 0;
        const uint32_t aqk = lane_base + acc_qk;
        const int v_per_step = nrot > 0 ? (dv / 16 + nrot - 1) / nrot : 0;   // dV chunks stored after every rotated step
        // ONE loop whose body holds the rotated step and the plain 16-column chunk once each: this code runs once per
        // item between long stretches of other roles' loops, so it is fetched cold every time, and what it costs is
        // its size (with a second and third inlined copy of the plain chunk the rotating dK/dV kernels were 8 % slower
        // than the plain ones although neither the table reads nor the arithmetic could be measured).
        int r = 0, v_owed = 0;                        // next rotated step; dV chunks still to store before it
        int cv = 0, cq = nrot * 2 * NP;               // next plain column of dV and of dQ / dK
#pragma unroll 1
        while (true) {
          if (r < nrot && v_owed == 0) {
            if constexpr (NE > 0) {
              const int seg = r / SPS, i0 = (r - seg * SPS) * NP, pos = seg ? icol : irow;
              const int c0 = 2 * seg * R + i0;
              uint32_t a[NP], b[NP];
              float x0[NP], x1[NP];
              if constexpr (NP == 16) { tmem_ld16(aqk + c0, a); tmem_ld16(aqk + c0 + R, b); }
              else { tmem_ld8(aqk + c0, a); tmem_ld8(aqk + c0 + R, b); }
              tmem_wait_ld();
              ++r;
              if (r == nrot && cv >= dv && cq >= dqk) { tc_fence_before(); mbar_arrive(&sh->acc_free); }
#pragma unroll
              for (int e = 0; e < NP; ++e) { x0[e] = __uint_as_float(a[e]) * scale; x1[e] = __uint_as_float(b[e]) * scale; }
              if (pos >= 0) {
                [[maybe_unused]] const uint32_t ta = (seg ? tab_col : tab_row) + (uint32_t)pos * rope_tab_stride(R) + i0 * 8;
#pragma unroll
                for (int e = 0; e < NP; e += 2) {
                  float4 c;                            // (cos, sin) of pairs e and e + 1
                  if constexpr (TABS) {
                    const uint4 u = lds128(ta + (e >> 1) * 16);
                    c = make_float4(__uint_as_float(u.x), __uint_as_float(u.y), __uint_as_float(u.z), __uint_as_float(u.w));
                  } else {
                    c = cs[e >> 1];
                  }
                  const float p0 = x0[e], q0 = x1[e], p1 = x0[e + 1], q1 = x1[e + 1];
                  x0[e] = p0 * c.x + q0 * c.y;
                  x1[e] = q0 * c.x - p0 * c.y;
                  x0[e + 1] = p1 * c.z + q1 * c.w;
                  x1[e + 1] = q1 * c.z - p1 * c.w;
                }
              }
              if (r < nrot) fetch(r);
              if (t_in) {
                if constexpr (NP == 16) {
                  store16<BF16>(qk_row + c0, x0);
                  store16<BF16>(qk_row + c0 + R, x1);
                } else {
                  *reinterpret_cast<uint4*>(qk_row + c0) = make_uint4(pack2<BF16>(x0[0], x0[1]), pack2<BF16>(x0[2], x0[3]),
                                                                      pack2<BF16>(x0[4], x0[5]), pack2<BF16>(x0[6], x0[7]));
                  *reinterpret_cast<uint4*>(qk_row + c0 + R) = make_uint4(pack2<BF16>(x1[0], x1[1]), pack2<BF16>(x1[2], x1[3]),
                                                                          pack2<BF16>(x1[4], x1[5]), pack2<BF16>(x1[6], x1[7]));
                }
              }
              v_owed = v_per_step;
            }
            continue;
          }
          // 16 plain columns: dV while there are any, then the un-rotated rest of dQ / dK
          uint32_t taddr;
          T* dst;
          float mul;
          if (cv < dv) {
            taddr = lane_base + acc_v + cv; dst = v_row + cv; mul = 1.f;
            cv += 16;
            if (v_owed > 0) --v_owed;
            if (cv >= dv) v_owed = 0;
          } else if (r < nrot) {
            v_owed = 0;
            continue;
          } else if (cq < dqk) {
            taddr = aqk + cq; dst = qk_row + cq; mul = scale;
            cq += 16;
          } else {
            break;
          }
          uint32_t a[16];
          float v[16];
          tmem_ld16(taddr, a);
          tmem_wait_ld();
          if (r == nrot && cv >= dv && cq >= dqk) { tc_fence_before(); mbar_arrive(&sh->acc_free); }   // the last load
#pragma unroll
          for (int e = 0; e < 16; ++e) v[e] = __uint_as_float(a[e]) * mul;
          if (t_in) store16<BF16>(dst, v);
        }
        trace_ev(p, 5, tn, t == 0 && it >= p.trace_it, 2 * 16 + (it & 15));
      }
      trace_ev(p, 5, tn, t == 0 && it >= p.trace_it, 3 * 16 + (it & 15));
    };

    int stage = 0, stage_par = 1;                    // parity of the "free" phase a rewrite of this stage's rows waits for
    int vslot = 0;
    bool ring_full = false;
    uint64_t pen_sig = ~0ull;                        // geometry the penalty tables in shared memory were built for
    uint32_t G = 0;                                  // stream position of the next block to prepare
    bool pend = false;                               // an item whose epilogue has not run yet
    int pend_item = 0, pend_it = 0;
    uint32_t pend_G = 0;                             // ... and the stream position before which it runs
#pragma unroll 1
    for (int it = 0, item = blockIdx.x;; ++it, item += gridDim.x) {   // one extra round flushes the last epilogue
      const bool have = item < n_items;
      const int bh = have ? item / tiles_per_head : 0;
      TilePos tp;
      tp.r0 = tp.x0 = tp.hx0 = tp.hr_first = tp.hr_last = 0;
      tp.nblk = 0;
      if (have) tp = tile_pos(p, item - bh * tiles_per_head);
      const int64_t vec_base = (int64_t)bh * p.t_h * p.Wtok;

      // -lse and delta of this thread's row of block j (dK/dV: the streamed rows are queries)
      float nl = -INFINITY, dl = 0.f;
      auto load_vec = [&](int j) {
        nl = -INFINITY;
        dl = 0.f;
        if constexpr (DKDV) {
          int band, cblk;
          block_pos(pl, j, band, cblk);
          const int row = tp.hr_first + band * pl.KR + jr, c = tp.hx0 + cblk * pl.KW + jc;
          if (row_on && c >= 0 && c < p.Wtok && j < tp.nblk && row < p.t_h) {
            nl = -__ldg(lse + vec_base + (int64_t)row * p.Wtok + c);
            dl = __ldg(delta + vec_base + (int64_t)row * p.Wtok + c);
          }
        }
      };
      if (have) {
        load_vec(0);
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
        // the score MMAs that read them have completed, and the lse / delta ring is two slots deeper than the block
        // ring: the score MMAs of block G - stages were issued after the accumulating MMAs of block G - stages - 2,
        // i.e. after the compute warps had finished reading that block's slot).  The block at stream position
        // (last block of an item + 2 + stages) is the first one they would have to wait for until that item's
        // last accumulating MMA has completed: the item's epilogue runs right before it (or at the end of a
        // later item that ends earlier, or after the last item), hidden behind that lead.
        const bool at_end = j >= tp.nblk;
        if (pend && (at_end || G >= pend_G)) {
          epilogue(pend_item, pend_it);
          pend = false;
        }
        if (at_end) break;
        const float a0 = nl, b0 = dl;
        load_vec(j + 1);                             // one block ahead: the latency hides behind this block's wait
        trace_ev(p, 4, tn, t == 0 && it >= p.trace_it, 0 * 16 + (j & 15));
        if (ring_full) wait_park(&sh->yx_free[stage], (uint32_t)stage_par, 10);
        trace_ev(p, 4, tn, t == 0 && it >= p.trace_it, 1 * 16 + (j & 15));
        if (ok) {
          if (row_on) {
            int band, cblk;
            block_pos(pl, j, band, cblk);
            write_penalty_row_v(yx_smem + stage * yx_stage, t, pen, band * pl.KR + jr, cblk * pl.KW + jc, pl.TH >> 3, pl.TW >> 3);
            if constexpr (DKDV) {
              vec_smem[vslot * 256 + t] = a0;
              vec_smem[vslot * 256 + 128 + t] = b0;
            }
          }
          fence_proxy_async_smem();
          mbar_arrive(&sh->y_ready[stage]);
          if constexpr (DKDV) mbar_arrive(&sh->vec_ready[vslot]);
        }
        trace_ev(p, 4, tn, t == 0 && it >= p.trace_it, 2 * 16 + (j & 15));
        if (++stage == pl.stages) { stage = 0; stage_par ^= 1; ring_full = true; }
        if (++vslot == vslots) vslot = 0;
      }
      if (!have) break;
      pend = true;
      pend_item = item;
      pend_it = it;
      pend_G = G - 1 + (uint32_t)(pl.stages + 2);
      if (rope_on) {                                 // fetched long before the epilogue needs it
        const int tr = tp.r0 + t / pl.TW, tx = tp.x0 + t % pl.TW;
        pend_packed = (tr < p.t_h && tx < p.Wtok) ? __ldg(p.rope.idx + (int64_t)tr * p.Wtok + tx) : -1;
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // let whatever is still in flight (TMA, MMA) land before shared memory and TMEM are released
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    if (threadIdx.x == 0) report_abort(p.status, DKDV ? 5 : 4, sh->abort_site);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kBwdTmemCols);
  }
}

}  // namespace tc
}  // namespace swa
