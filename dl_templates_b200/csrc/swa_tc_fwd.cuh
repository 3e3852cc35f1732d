// tcgen05 forward kernel: o = softmax(scale * rope(q) rope(k)^T + window mask) v, lse.
//
// Persistent: one CTA per SM walks a list of work items, one item = one 128-query tile (8 rows
// x 16 token columns) of one (batch, head); consecutive items are neighbouring tiles of the same
// head, so the K/V halo re-reads of the CTAs running at one time are served by L2.  The query
// tile and the O accumulator are double-buffered, so the loads, the RoPE rotation and the first
// MMAs of item i+1 run under the tail (last blocks, normalisation, stores) of item i.
//
// Warp roles (448 threads):
//   warp 0       TMA producer: per item the query tile, then the K and V halo blocks through a
//                `stages`-deep ring of shared-memory buffers
//   warp 1       MMA issuer (whole warp in uniform control flow, one elected lane issues):
//                S = Q K^T (+ the window mask as 32 extra contraction columns) into one of two
//                TMEM buffers, O += P V into one of two more; owns the TMEM allocation
//   warps 2-9    softmax, TWO threads per query row (TMEM lane): warps w and w+4 share a lane
//                quarter and take the lower / upper half of each block's columns, so every
//                scheduler has two softmax warps whose dependency stalls overlap; the pair
//                exchanges its block maximum through shared memory.  tcgen05.ld of the S row,
//                running max / sum, P written to shared memory as the A operand of the PV MMA,
//                lazy rescale of O, final normalisation and stores
//   warps 10-13  fused RoPE-2D: rotate the Q tile and every K block in shared memory between
//                TMA arrival and MMA issue, and write the window-mask tiles
// S for block j+1 is computed by the tensor core while the softmax warps work on block j.
// All waits are bounded; a timed-out wait raises a CTA-wide abort flag, every role runs its
// loops to the end without touching anything, TMEM is freed and the status word records it.
#pragma once

#include "swa_tc_common.cuh"

namespace swa {
namespace tc {

struct FwdBars {
  uint64_t q_full[2], q_ready[2], q_empty[2], o_full[2], o_free[2];
  uint64_t kv_full[kMaxStages], k_ready[kMaxStages], kv_empty[kMaxStages];
  uint64_t s_full[2], s_empty[2], p_full[2], p_empty[2];
  float xchg[2][2][128];  // [S buffer][column half][row]: block maxima of the two threads of a row
  float lsum[2][2][128];  // [item parity][column half][row]: partial row sums, exchanged once per item
  PenaltyTables pen;      // window-mask penalty parts of the current item's halo rows / columns
  uint32_t tmem_base;
  int abort_flag;
};

constexpr int kFwdThreads = 448;
constexpr int kFwdRopeThread0 = 320;
constexpr uint32_t kFwdTmemCols = 512;
constexpr uint32_t kTmemS = 0, kTmemO = 256;   // column offsets: S0 at 0, S1 at 128, O0 at 256, O1 behind it
constexpr float kRescaleThreshold = 8.f;       // lazy rescale when the running max grows by > 2^8

template <bool BF16>
__global__ void __launch_bounds__(kFwdThreads, 1)
fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
           const __grid_constant__ CUtensorMap tm_v, KParams p, View4 o, float* __restrict__ lse) {
  using namespace ptx;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const Plan& pl = p.pl;
  const int N = pl.N;
  const uint32_t blk_bytes = (uint32_t)N * 128u;               // one 64-wide chunk of a streamed block
  const uint32_t q_bytes = p.qch * 16384u;
  const uint32_t k_stage = blk_bytes * p.qch, v_stage = blk_bytes * p.vch;
  const int pch = (N + 63) >> 6;                                 // 64-key chunks of P
  const uint32_t kx_stage = (uint32_t)N * kXRowBytes;           // window-mask penalty rows of a streamed block
  const uint32_t o_cols = p.vch * 64u;                           // TMEM columns of one O buffer
  uint8_t* q_smem = smem;                                        // two buffers
  uint8_t* qx_smem = q_smem + 2 * q_bytes;                      // window-mask indicator rows of a query tile
  uint8_t* k_smem = qx_smem + 128 * kXRowBytes;
  uint8_t* v_smem = k_smem + pl.stages * k_stage;
  uint8_t* kx_smem = v_smem + pl.stages * v_stage;
  uint8_t* p_smem = kx_smem + pl.stages * kx_stage;
  FwdBars* bars = reinterpret_cast<FwdBars*>(p_smem + pl.pbufs * pch * 16384);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->q_full[s], 1);
      mbar_init(&bars->q_ready[s], 128);
      mbar_init(&bars->q_empty[s], 1);
      mbar_init(&bars->o_full[s], 1);
      mbar_init(&bars->o_free[s], 256);
      mbar_init(&bars->s_full[s], 1);
      mbar_init(&bars->s_empty[s], 256);
      mbar_init(&bars->p_full[s], 256);
      mbar_init(&bars->p_empty[s], 1);
    }
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->k_ready[s], 128);
      mbar_init(&bars->kv_empty[s], 1);
    }
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, kFwdTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  // `ok` is kept warp-uniform in every role.  A failed (timed-out) wait does not leave the loops:
  // warps that meet at named barriers must all run the same number of iterations; with ok == false
  // every later wait returns at once and nothing is touched any more.
  bool ok = true;
  auto wait_spin = [&](uint64_t* bar, uint32_t parity) {
    const bool r = ok && mbar_wait<0>(bar, parity, abort_flag);
    ok = __all_sync(0xffffffffu, r);
  };
  auto wait_park = [&](uint64_t* bar, uint32_t parity) {
    const bool r = ok && mbar_wait<100>(bar, parity, abort_flag);
    ok = __all_sync(0xffffffffu, r);
  };
  const int n_items = p.n_items, tiles_per_head = pl.n_tiles_x * pl.n_tiles_y;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
    }
    __syncwarp();
    uint32_t kv = 0;
    for (int it = 0, item = blockIdx.x; item < n_items; ++it, item += gridDim.x) {
      const int bh = item / tiles_per_head, bi = bh / p.H, hi = bh - bi * p.H;
      const TilePos tp = tile_pos(p, item - bh * tiles_per_head);
      const int qb = it & 1;
      if (it >= 2) wait_park(&bars->q_empty[qb], ((it >> 1) - 1) & 1);
      if (ok && elect_one()) {
        mbar_arrive_expect_tx(&bars->q_full[qb], q_bytes);
        for (int c = 0; c < p.qch; ++c)
          tma_load_5d(q_smem + qb * q_bytes + c * 16384, &tm_q, &bars->q_full[qb], c * 64, tp.x0, tp.r0, hi, bi);
      }
      __syncwarp();
      for (int j = 0; j < tp.nblk; ++j, ++kv) {
        const int s = kv % pl.stages;
        if (kv >= (uint32_t)pl.stages) wait_park(&bars->kv_empty[s], ((kv / pl.stages) - 1) & 1);
        if (ok && elect_one()) {
          mbar_arrive_expect_tx(&bars->kv_full[s], k_stage + v_stage);
          const int row = tp.hr_first + j * pl.KR;
          for (int c = 0; c < p.qch; ++c)
            tma_load_5d(k_smem + s * k_stage + c * blk_bytes, &tm_k, &bars->kv_full[s], c * 64, tp.hx0, row, hi, bi);
          for (int c = 0; c < p.vch; ++c)
            tma_load_5d(v_smem + s * v_stage + c * blk_bytes, &tm_v, &bars->kv_full[s], c * 64, tp.hx0, row, hi, bi);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t fmt = BF16 ? 1u : 0u;
    const uint32_t idesc_s = instr_desc(fmt, 128, N, 0, 0);
    const uint32_t idesc_pv = instr_desc(fmt, 128, p.vch * 64, 0, 1);
    const uint32_t q_addr = smem_u32(q_smem), k_addr = smem_u32(k_smem), v_addr = smem_u32(v_smem),
                   p_addr = smem_u32(p_smem), qx_addr = smem_u32(qx_smem), kx_addr = smem_u32(kx_smem);
    const uint32_t hi_sw = smem_desc_hi(1024, true), hi_ns = smem_desc_hi(kXSbo, false);
    uint32_t kv = 0, sc = 0, pc = 0;     // running counts of K/V blocks, S tiles, P tiles
    for (int it = 0, item = blockIdx.x; item < n_items; ++it, item += gridDim.x) {
      const int bh = item / tiles_per_head;
      const TilePos tp = tile_pos(p, item - bh * tiles_per_head);
      const int qb = it & 1, ob = it & 1;
      const uint32_t kv0 = kv, o_tm = tmem + kTmemO + ob * o_cols;
      // O += P V for block i of this item
      auto issue_pv = [&](int i) {
        const int pb = pc % pl.pbufs, s = (kv0 + i) % pl.stages;
        wait_spin(&bars->p_full[pb], (pc / pl.pbufs) & 1);
        if (i == 0 && it >= 2) wait_spin(&bars->o_free[ob], ((it >> 1) - 1) & 1);   // first write of this O buffer
        if (ok) {
          tc_fence_after();
          const uint32_t pa = p_addr + pb * pch * 16384, vb = v_addr + s * v_stage;
          if (elect_one()) {
            for (int ks = 0; ks < (N >> 4); ++ks)
              umma_ss(o_tm, smem_desc_from(pa + (ks >> 2) * 16384 + (ks & 3) * 32, 16, hi_sw),
                      smem_desc_from(vb + ks * 2048, blk_bytes, hi_sw), idesc_pv, (i > 0 || ks > 0) ? 1u : 0u);
            umma_commit(&bars->kv_empty[s]);
            umma_commit(&bars->p_empty[pb]);
            if (i == tp.nblk - 1) umma_commit(&bars->o_full[ob]);
          }
          __syncwarp();
        }
        ++pc;
      };
      wait_spin(&bars->q_ready[qb], (it >> 1) & 1);
      for (int j = 0; j < tp.nblk; ++j, ++kv, ++sc) {
        const int s = kv % pl.stages, sb = sc & 1;
        wait_spin(&bars->k_ready[s], (kv / pl.stages) & 1);
        if (sc >= 2) wait_spin(&bars->s_empty[sb], ((sc >> 1) - 1) & 1);
        if (ok) {
          tc_fence_after();
          const uint32_t qa = q_addr + qb * q_bytes, kb = k_addr + s * k_stage, kxb = kx_addr + s * kx_stage,
                         sd = tmem + kTmemS + sb * 128;
          if (elect_one()) {
            for (int c = 0; c < p.qch; ++c) {
#pragma unroll
              for (int k = 0; k < 4; ++k)
                umma_ss(sd, smem_desc_from(qa + c * 16384 + k * 32, 16, hi_sw),
                        smem_desc_from(kb + c * blk_bytes + k * 32, 16, hi_sw), idesc_s, (c | k) ? 1u : 0u);
            }
#pragma unroll
            for (int k = 0; k < 2; ++k)  // + indicator x penalty: the window mask
              umma_ss(sd, smem_desc_from(qx_addr + k * kXStepBytes, kXLbo, hi_ns),
                      smem_desc_from(kxb + k * kXStepBytes, kXLbo, hi_ns), idesc_s, 1u);
            umma_commit(&bars->s_full[sb]);
            if (j == tp.nblk - 1) umma_commit(&bars->q_empty[qb]);   // last read of this query buffer
            if (it == p.trace_it) trace_mark(p, 1, 1 + 2 * j);
          }
          __syncwarp();
        }
        if (j >= 1) issue_pv(j - 1);
      }
      issue_pv(tp.nblk - 1);
    }
  } else if (warp < 10) {
    // ------------------------------------------------------------------ softmax, two threads per query row
    const int quarter = warp & 3;                 // TMEM lane quarter this warp may touch
    const int half = (warp - 2) >> 2;             // lower / upper half of each block's columns is this thread's
    const int m = quarter * 32 + lane;
    const float none_thresh = -0.5f * p.mask_a * p.mask_b;     // a block maximum below this: every entry masked
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    const uint32_t p_base = smem_u32(p_smem) + m * 128;
    const uint32_t xchg_base = smem_u32(&bars->xchg[0][0][0]), lsum_base = smem_u32(&bars->lsum[0][0][0]);
    const int sw = m & 7;
    const float c2 = p.scale_log2;
    const bool tr = (m == 0 && half == 0);
    // This thread's nh = N/2 columns (a multiple of 8, <= 64) are held as up to eight 8-column units in
    // fixed registers: units 0-3 one 32-column load (nh >= 32); units 4-7 a second one (nh == 64), or
    // a 16-column load (units 4-5, nh & 16) and an 8-column load (unit 6, nh & 8).
    const int nh = N >> 1, col0 = half * nh;
    const int off16 = nh & ~31, off8 = nh & ~15;
    int ucol[8];                                  // first column (within the thread's half) of each unit
    uint32_t uvalid = 0;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      bool v;
      if (u < 4) { v = nh >= 32; ucol[u] = u * 8; }
      else if (nh == 64) { v = true; ucol[u] = u * 8; }
      else if (u < 6) { v = (nh & 16) != 0; ucol[u] = off16 + (u - 4) * 8; }
      else if (u == 6) { v = (nh & 8) != 0; ucol[u] = off8; }
      else { v = false; ucol[u] = 0; }
      uvalid |= (v ? 1u : 0u) << u;
    }
    uint32_t sc = 0, pc = 0;
    for (int it = 0, item = blockIdx.x; item < n_items; ++it, item += gridDim.x) {
      const int bh = item / tiles_per_head, bi = bh / p.H, hi = bh - bi * p.H;
      const TilePos tp = tile_pos(p, item - bh * tiles_per_head);
      const int ob = it & 1;
      const int qr = tp.r0 + m / pl.TW, qx = tp.x0 + m % pl.TW;
      const bool q_in = qr < p.t_h && qx < p.Wtok;
      float m_used = -INFINITY, l = 0.f;
      if (tr && it == p.trace_it) trace_mark(p, 2, 29);
      for (int j = 0; j < tp.nblk; ++j, ++sc, ++pc) {
        const int sb = sc & 1, pb = pc % pl.pbufs;
        wait_spin(&bars->s_full[sb], (sc >> 1) & 1);
        uint32_t sr[64];
        float mx = -INFINITY;
        if (ok) {
          tc_fence_after();
          if (tr && it == p.trace_it) trace_mark(p, 2, 1 + 4 * j);
          const uint32_t sbase = lane_base + kTmemS + sb * 128 + col0;
          if (nh >= 32) tmem_ld32(sbase, &sr[0]);
          if (nh == 64) {
            tmem_ld32(sbase + 32, &sr[32]);
          } else {
            if (nh & 16) tmem_ld16(sbase + off16, &sr[32]);
            if (nh & 8) tmem_ld8(sbase + off8, &sr[48]);
          }
          tmem_wait_ld();
          tc_fence_before();
          mbar_arrive(&bars->s_empty[sb]);
          float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if ((uvalid >> u) & 1u) {
#pragma unroll
              for (int i = 0; i < 8; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sr[u * 8 + i]));
            }
          mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        }
        // combine with the thread that owns the other half of this row
        sts32(xchg_base + ((sb * 2 + half) * 128 + m) * 4, mx);
        named_bar_sync(1 + quarter, 64);
        mx = fmaxf(mx, lds32(xchg_base + ((sb * 2 + (half ^ 1)) * 128 + m) * 4));
        if (mx < none_thresh) mx = -INFINITY;
        // running max with lazy rescale: keep scaling by m_used until the true max exceeds it by 2^8
        bool need = false;
        float m_new = m_used;
        if (mx > m_used) {
          if (m_used == -INFINITY) m_used = mx;        // nothing accumulated yet for this row
          else if ((mx - m_used) * c2 > kRescaleThreshold) { need = true; m_new = mx; }
        }
        const bool any_need = __any_sync(0xffffffffu, need);
        const float alpha = need ? exp2f((m_used - m_new) * c2) : 1.f;
        if (need) { m_used = m_new; l *= alpha; }
        const float mc = (m_used == -INFINITY) ? 0.f : m_used * c2;

        if (pc >= (uint32_t)pl.pbufs) wait_spin(&bars->p_empty[pb], ((pc / pl.pbufs) - 1) & 1);
        if (ok) {
          const uint32_t prow = p_base + pb * pch * 16384;
          float ls4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if ((uvalid >> u) & 1u) {
              uint32_t w[4];
#pragma unroll
              for (int h = 0; h < 4; ++h) {
                const float p0 = exp2f(fmaf(__uint_as_float(sr[u * 8 + 2 * h]), c2, -mc));
                const float p1 = exp2f(fmaf(__uint_as_float(sr[u * 8 + 2 * h + 1]), c2, -mc));
                ls4[h] += p0 + p1;
                w[h] = pack2<BF16>(p0, p1);
              }
              const int pu = (col0 + ucol[u]) >> 3;     // 16-byte unit of the P row (8 keys)
              sts128(prow + (pu >> 3) * 16384 + (((pu & 7) ^ sw) << 4), w[0], w[1], w[2], w[3]);
            }
          l += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
          fence_proxy_async_smem();
        }
        if (any_need && j > 0) {
          // O must be at rest: wait for PV of the previous block of this item, then scale this thread's share
          const uint32_t pprev = pc - 1;
          wait_spin(&bars->p_empty[pprev % pl.pbufs], (pprev / pl.pbufs) & 1);
          if (ok) {
            tc_fence_after();
            for (int c = half; c < p.vch * 4; c += 2) {
              uint32_t orow[16];
              tmem_ld16(lane_base + kTmemO + ob * o_cols + c * 16, orow);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 16; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * alpha);
              tmem_st16(lane_base + kTmemO + ob * o_cols + c * 16, orow);
            }
            tmem_wait_st();
            tc_fence_before();
          }
        }
        if (ok) mbar_arrive(&bars->p_full[pb]);
        if (tr && it == p.trace_it) trace_mark(p, 2, 4 + 4 * j);
      }
      // epilogue of the item: O / l and lse; each thread of the pair stores one contiguous half of the row
      wait_spin(&bars->o_full[ob], (it >> 1) & 1);
      sts32(lsum_base + ((ob * 2 + half) * 128 + m) * 4, l);
      named_bar_sync(1 + quarter, 64);
      l += lds32(lsum_base + ((ob * 2 + (half ^ 1)) * 128 + m) * 4);
      if (ok) {
        tc_fence_after();
        if (tr && it == p.trace_it) trace_mark(p, 2, 30);
        const float inv = 1.f / l;
        const int64_t tok = (int64_t)qr * p.Wtok + qx;
        using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
        const int ncol = p.vch * 32;                 // columns per thread: d_v / 2
        T* orow_g = (T*)o.ptr + bi * o.s0 + hi * o.s1 + tok * o.s2 + half * ncol;
        for (int c0 = 0; c0 < ncol; c0 += 32) {
          uint32_t orow[32];
          tmem_ld32(lane_base + kTmemO + ob * o_cols + half * ncol + c0, orow);
          tmem_wait_ld();
          if (c0 + 32 >= ncol) {                     // this thread has read all it needs of the O buffer
            tc_fence_before();
            mbar_arrive(&bars->o_free[ob]);
          }
          if (q_in) {
            uint4* dst = reinterpret_cast<uint4*>(orow_g + c0);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint32_t w[4];
#pragma unroll
              for (int h = 0; h < 4; ++h)
                w[h] = pack2<BF16>(__uint_as_float(orow[u * 8 + 2 * h]) * inv, __uint_as_float(orow[u * 8 + 2 * h + 1]) * inv);
              dst[u] = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
        if (q_in && half == 0) lse[(int64_t)bh * p.t_h * p.Wtok + tok] = m_used * c2 + log2f(l);
        if (tr && it == p.trace_it) trace_mark(p, 2, 31);
      }
    }
  } else {
    // ------------------------------------------------------------------ fused RoPE-2D on Q and K tiles, mask tiles
    const int t = threadIdx.x - kFwdRopeThread0;
    const bool rope_on = p.rope.idx != nullptr;
    const RopeParts qp = rope_parts(t, 128), kp = rope_parts(t, N);   // share of a Q tile / of a K block
    write_indicator_row<BF16>(qx_smem, qp.row, qp.lo, qp.hi, p);      // the same for every item
    uint32_t kv = 0;
    RopeRow rc;
    rc.pos[0] = rc.pos[1] = -1;
    for (int it = 0, item = blockIdx.x; item < n_items; ++it, item += gridDim.x) {
      const int bh = item / tiles_per_head;
      const TilePos tp = tile_pos(p, item - bh * tiles_per_head);
      const int qb = it & 1;
      const int qr = tp.r0 + qp.row / pl.TW, qx = tp.x0 + qp.row % pl.TW;
      const bool q_in = qr < p.t_h && qx < p.Wtok;
      const int kjr = kp.row / pl.KW, kx = tp.hx0 + kp.row % pl.KW;   // this thread's row inside every streamed block
      const bool kx_in = kp.active && kx >= 0 && kx < p.Wtok;
      int32_t k_idx = -1;
      rc.pos[0] = rc.pos[1] = -1;
      if (rope_on) {
        if (q_in) rope_fetch(rc, __ldg(p.rope.idx + qr * p.Wtok + qx), qp, p.rope);
        const int kr0 = tp.hr_first + kjr;
        if (kx_in && kr0 < p.t_h) k_idx = __ldg(p.rope.idx + kr0 * p.Wtok + kx);
      }
      named_bar_sync(5, 128);                        // nobody still reads the previous item's tables
      build_penalty_tables<BF16>(&bars->pen, t, p, tp);
      named_bar_sync(5, 128);                        // the tables are complete before any of these warps reads them
      wait_park(&bars->q_full[qb], (it >> 1) & 1);
      if (ok) {
        if (rope_on && q_in) rope_apply<BF16>(q_smem + qb * q_bytes, 16384, rc, qp, p.rope);
        fence_proxy_async_smem();
        mbar_arrive(&bars->q_ready[qb]);
      }
      rope_fetch(rc, k_idx, kp, p.rope);             // cos/sin of this thread's row of block 0
      for (int j = 0; j < tp.nblk; ++j, ++kv) {
        const int s = kv % pl.stages;
        const int kr = tp.hr_first + j * pl.KR + kjr;
        // index of the same row of the next block: in flight while this block is rotated
        int32_t k_idx_next = -1;
        if (rope_on && kx_in && j + 1 < tp.nblk && kr + pl.KR < p.t_h) k_idx_next = __ldg(p.rope.idx + (kr + pl.KR) * p.Wtok + kx);
        // the stage (K, V and penalty rows) is free once its refill has landed: the producer refills
        // only after every MMA of the stage's previous block has completed
        wait_park(&bars->kv_full[s], (kv / pl.stages) & 1);
        if (ok) {
          if (kp.active) write_penalty_row(kx_smem + s * kx_stage, kp.row, kp.lo, kp.hi, &bars->pen, j * pl.KR + kjr, kp.row % pl.KW, pl.TH >> 3, pl.TW >> 3);
          if (rope_on && kx_in && kr < p.t_h) rope_apply<BF16>(k_smem + s * k_stage, blk_bytes, rc, kp, p.rope);
          fence_proxy_async_smem();
          mbar_arrive(&bars->k_ready[s]);
        }
        rope_fetch(rc, k_idx_next, kp, p.rope);      // lands while this thread waits for the next block
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // let whatever is still in flight (TMA, MMA) land before shared memory and TMEM are released
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    if (threadIdx.x == 0) report_abort(p.status, 1, 0);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kFwdTmemCols);
  }
}

}  // namespace tc
}  // namespace swa
