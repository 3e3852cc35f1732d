// tcgen05 forward kernel: o = softmax(scale * rope(q) rope(k)^T + window mask) v, lse.
//
// Persistent: one CTA per SM walks a list of work items, one item = one 128-query tile
// (TH rows x TW token columns) of one (batch, head); consecutive items are neighbouring tiles of
// the same head, so the K/V halo re-reads of the CTAs running at one time are served by L2.
//
// The halo blocks of all items of a CTA form one stream G = 0, 1, 2, ...  Two groups of softmax
// warps take the blocks of even resp. odd G; each group has its own running maximum / sum and its
// own output accumulator O_g, as if the keys were split between two independent attention passes;
// the two partial results of an item are merged when it ends.  The groups therefore never wait for
// each other inside an item, and the two warps a scheduler hosts (one of each group) are in
// different phases of their block: while one waits for tensor memory or a barrier, the other one
// keeps the exp2 unit busy.
//
// Warp roles (512 threads):
//   warp 0        TMA producer: per item the query tile (double-buffered), then the K and V halo
//                 blocks through a `stages`-deep ring of shared-memory buffers
//   warp 1        MMA issuer (whole warp in uniform control flow, one elected lane issues), `nsb`
//                 score blocks ahead: S = Q K^T (+ the window mask as 32 extra contraction columns)
//                 into a ring of `nsb` score buffers, and O_g += P V with P read from TENSOR memory,
//                 where the softmax thread of a row has written it over the row of S it came from
//   warps 4-7     softmax group 0, warps 8-11 softmax group 1: ONE thread per query row (TMEM lane):
//                 row maximum, exp2, row sum, P packed to 16 bits and stored in place, lazy rescale
//                 of O_g.  A warp skips the blocks none of its 32 rows can see (P = 0 for them).
//   warps 2-3, 12-15  fused RoPE-2D (two threads per row where the thread count allows): rotate the Q tile and every K block in shared memory between
//                 TMA arrival and MMA issue, and write the window-mask tiles
//
// Code size is a first-order concern here: each role is a different instruction stream, the
// scalar roles run a few hundred instructions per block, and with 16 warps of 5 kinds per SM
// nothing stays in the small per-scheduler instruction caches unless the loops are compact.  So
// every inner loop is a real loop with a small body (no full unrolling over a row), every
// helper has one call site per role, and the RoPE table width is a template parameter.
//
// All waits are bounded; a timed-out wait raises a CTA-wide abort flag, every role runs its
// loops to the end without touching anything, TMEM is freed and the status word records it.
#pragma once

#include "swa_tc_common.cuh"

namespace swa {
namespace tc {

struct FwdShared {
  uint64_t q_full[2], q_ready[2], q_empty[2];
  uint64_t kv_full[kMaxStages], k_ready[kMaxStages], kv_empty[kMaxStages];
  uint64_t s_full[4], p_full[4], pv_done[2], o_full, o_free;
  float ml[2][2][2][128];   // [item parity][group][maximum | sum][row]: merged when an item ends
  PenaltyTables pen;        // window-mask penalty parts of the current item's halo rows / columns
  uint32_t tmem_base;
  int abort_flag;
};

constexpr int kFwdThreads = 512;
constexpr int kFwdRopeThreads = 192;     // warps 2-3 and 12-15
constexpr uint32_t kFwdTmemCols = 512;
constexpr float kRescaleThreshold = 8.f;       // lazy rescale when the running max grows by > 2^8

template <bool BF16, int NI, bool TABS>
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
  const uint32_t kx_stage = (uint32_t)N * kXRowBytes;           // window-mask penalty rows of a streamed block
  const uint32_t o_cols = p.vch * 64u;                           // TMEM columns of one O accumulator
  // score buffers: the score MMAs run `nsb` blocks ahead, so that a softmax group finds its next block
  // ready when it has finished one (2 to 4, chosen by the planner)
  const int nsb = pl.nsb;
  // score buffer b at column s_stride*b (128-column strides when they fit, else packed), O_g behind them
  const uint32_t s_stride = (N <= 128 && nsb * 128u + 2 * o_cols <= kFwdTmemCols) ? 128u : (uint32_t)N;
  const uint32_t o_base = nsb * s_stride;
  uint8_t* q_smem = smem;                                        // two buffers
  uint8_t* qx_smem = q_smem + 2 * q_bytes;                      // window-mask indicator rows of a query tile
  uint8_t* k_smem = qx_smem + 128 * kXRowBytes;
  uint8_t* v_smem = k_smem + pl.stages * k_stage;
  uint8_t* kx_smem = v_smem + pl.stages * v_stage;
  FwdShared* sh = reinterpret_cast<FwdShared*>(kx_smem + pl.stages * kx_stage);
  uint8_t* tab_smem = reinterpret_cast<uint8_t*>(sh) + ((sizeof(FwdShared) + 15) & ~size_t(15));   // cos/sin tables (TABS)
  volatile int* abort_flag = &sh->abort_flag;

  const int warp = threadIdx.x >> 5;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sh->q_full[s], 1);
      mbar_init(&sh->q_ready[s], kFwdRopeThreads);
      mbar_init(&sh->q_empty[s], 1);
      mbar_init(&sh->pv_done[s], 1);
    }
    for (int s = 0; s < 4; ++s) {
      mbar_init(&sh->s_full[s], 1);
      mbar_init(&sh->p_full[s], 128);   // per score buffer: a group may finish two blocks before the issuer looks
    }
    mbar_init(&sh->o_full, 1);
    mbar_init(&sh->o_free, 256);
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(&sh->kv_full[s], 1);
      mbar_init(&sh->k_ready[s], kFwdRopeThreads);
      mbar_init(&sh->kv_empty[s], 1);
    }
    sh->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, kFwdTmemCols);
    tmem_relinquish();
  }
  if constexpr (TABS) stage_rope_tables(tab_smem, p.rope, threadIdx.x, kFwdThreads);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;

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

  // Registers follow the work: the kernel starts with 128 per thread; the producer / issuer / RoPE
  // warpgroups (warps 0-3 and 12-15) give some back, the two softmax warpgroups take them.
  // (2 * 104 + 2 * 152) * 128 = 64 Ki.  Not done in the variant whose RoPE warps keep cos/sin rows in registers.  Each setmaxnreg is the first instruction of its branch, so that the
  // whole branch is compiled for that budget.
  if (warp >= 4 && warp < 12) {
    if constexpr (TABS || NI == 0) setmaxnreg_inc<152>();
    // ------------------------------------------------------------------ softmax, one thread per query row and group
    const int lane = threadIdx.x & 31;
    const int g = (warp - 4) >> 2;                // group: takes the blocks whose stream position has parity g
    const int quarter = warp & 3;                 // TMEM lane quarter this warp may touch
    const int m = quarter * 32 + lane;
    const float none_thresh = -0.5f * p.mask_a * p.mask_b;     // a row maximum below this: every entry masked
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    const uint32_t o_tm = lane_base + o_base + g * o_cols, o_other = lane_base + o_base + (g ^ 1) * o_cols;
    const float c2 = p.scale_log2;
    const int ng = N >> 4;                        // 16-column granules of a row
    const bool tr = (m == 0);
    const int trole = g ? 0 : 2;              // trace rows: group 0 -> 2, group 1 -> 0
    uint32_t gbase = 0;                           // stream position of the current item's block 0
    // this group's next block: stream position, its score buffer and that buffer's barrier parity
    uint32_t own_next = g, n_own = 0;
    int sbuf = g, spar = 0;
    // The merge / store of an item is deferred until this thread has worked on its first block of the
    // NEXT item: the last PV MMAs of an item complete long after a group has finished its own last block,
    // and the score MMAs of the next item's first blocks have been issued by then.
    bool pend = false, pend_even = false;
    int pend_item = 0, pend_it = 0, pend_cnt = 0, pend_cnt_other = 0;
    float pend_m = 0.f, pend_l = 0.f;
#pragma unroll 1
    for (int it = 0, item = blockIdx.x;; ++it, item += gridDim.x) {
      const bool have = item < n_items;
      TilePos tp;
      tp.r0 = tp.x0 = tp.hx0 = tp.hr_first = tp.hr_last = 0;
      tp.nblk = 0;
      if (have) tp = tile_pos(p, item % tiles_per_head);
      // rows of the grid the 32 queries of this warp can see
      const int see_lo = tp.r0 + (quarter * 32) / pl.TW - p.wr, see_hi = tp.r0 + (quarter * 32 + 31) / pl.TW + p.wr;
      float m_used = -INFINITY, l = 0.f;
      int cnt = 0;                                // blocks of this item this group has handed to the PV MMA
      if (tr && it == p.trace_it) trace_mark(p, trole, 29);
      int j = have ? (int)(own_next - gbase) : 0;
      bool first = true;
#pragma unroll 1
      while (true) {
      if (j < tp.nblk) {
        const uint32_t s_tm = lane_base + sbuf * s_stride;
        uint64_t* const p_bar = &sh->p_full[sbuf];
        wait_spin(&sh->s_full[sbuf], spar);
        sbuf += 2;                                // two positions on in the ring of nsb buffers
        if (sbuf >= nsb) { sbuf -= nsb; spar ^= 1; }
        const int blk_first = tp.hr_first + j * pl.KR, blk_last = blk_first + pl.KR - 1;
        const bool seen = !(blk_last < see_lo || blk_first > see_hi);
        if (tr && it == p.trace_it) trace_mark(p, trole, 1 + 4 * (j >> 1));
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
          if (tr && it == p.trace_it) trace_mark(p, trole, 2 + 4 * (j >> 1));
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
        if (tr && it == p.trace_it) trace_mark(p, trole, 4 + 4 * (j >> 1));
        j += 2;
        own_next += 2;
        ++n_own;
        ++cnt;
      }
      if (first) {
      first = false;
      if (pend) {
      pend = false;
      // merge the two groups' partial results of the pending item; each group stores one half of the row
      const int e_bh = pend_item / tiles_per_head, bi = e_bh / p.H, hi = e_bh - bi * p.H;
      const TilePos e_tp = tile_pos(p, pend_item - e_bh * tiles_per_head);
      const int qr = e_tp.r0 + m / pl.TW, qx = e_tp.x0 + m % pl.TW;
      const bool q_in = qr < p.t_h && qx < p.Wtok;
      const int par = pend_it & 1;
      wait_spin(&sh->o_full, pend_it & 1);
      sh->ml[par][g][0][m] = pend_m;
      sh->ml[par][g][1][m] = pend_l;
      named_bar_sync(1 + quarter, 64);
      const float m_o = sh->ml[par][g ^ 1][0][m], l_o = sh->ml[par][g ^ 1][1][m];
      if (ok) {
        tc_fence_after();
        if (tr && pend_it == p.trace_it) trace_mark(p, trole, 30);
        // Merge in an order fixed by the blocks' positions in the item (even ones first), not by which
        // group happened to get them: the result of a tile must not depend on the work that preceded it.
        const bool mine_even = pend_even;
        const float m_e = mine_even ? pend_m : m_o, m_d = mine_even ? m_o : pend_m;
        const float l_e = mine_even ? pend_l : l_o, l_d = mine_even ? l_o : pend_l;
        const int cnt_e = mine_even ? pend_cnt : pend_cnt_other, cnt_d = mine_even ? pend_cnt_other : pend_cnt;
        const float mm = fmaxf(m_e, m_d);
        const float w_e = (m_e == -INFINITY) ? 0.f : exp2f((m_e - mm) * c2);
        const float w_d = (m_d == -INFINITY) ? 0.f : exp2f((m_d - mm) * c2);
        const float lt = fmaf(l_d, w_d, l_e * w_e);
        const float inv = 1.f / lt;
        const float f_e = w_e * inv, f_d = w_d * inv;
        const int64_t tok = (int64_t)qr * p.Wtok + qx;
        using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
        const int ncol = p.vch * 32;                 // columns per thread: d_v / 2
        T* orow_g = (T*)o.ptr + bi * o.s0 + hi * o.s1 + tok * o.s2 + g * ncol;
        const uint32_t o_even = mine_even ? o_tm : o_other, o_odd = mine_even ? o_other : o_tm;
#pragma unroll 1
        for (int c0 = 0; c0 < ncol; c0 += 16) {
          uint32_t a[16], b[16];
          if (cnt_e > 0) tmem_ld16(o_even + g * ncol + c0, a);
          if (cnt_d > 0) tmem_ld16(o_odd + g * ncol + c0, b);
          tmem_wait_ld();
          if (c0 + 16 >= ncol) {                     // this thread has read all it needs of both accumulators
            tc_fence_before();
            mbar_arrive(&sh->o_free);
          }
          if (q_in) {
            uint4* dst = reinterpret_cast<uint4*>(orow_g + c0);
#pragma unroll
            for (int uu = 0; uu < 2; ++uu) {
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
        if (q_in && g == 0) lse[(int64_t)e_bh * p.t_h * p.Wtok + tok] = mm * c2 + log2f(lt);
        if (tr && pend_it == p.trace_it) trace_mark(p, trole, 31);
      }
      }
      }
      if (j >= tp.nblk) break;
      }
      if (!have) break;
      // this item's result becomes the pending one
      pend = true;
      pend_item = item;
      pend_it = it;
      pend_m = m_used;
      pend_l = l;
      pend_cnt = cnt;
      pend_cnt_other = (int)((tp.nblk + (((gbase & 1u) == (uint32_t)(g ^ 1)) ? 1 : 0)) >> 1);
      pend_even = ((gbase & 1u) == (uint32_t)g);
      gbase += tp.nblk;
    }
  } else {
    if constexpr (TABS || NI == 0) setmaxnreg_dec<104>();
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
          const int row = tp.hr_first + j * pl.KR;
#pragma unroll 1
          for (int c = 0; c < p.qch; ++c)
            tma_load_5d(k_smem + stage * k_stage + c * blk_bytes, &tm_k, &sh->kv_full[stage], c * 64, tp.hx0, row, hi, bi);
#pragma unroll 1
          for (int c = 0; c < p.vch; ++c)
            tma_load_5d(v_smem + stage * v_stage + c * blk_bytes, &tm_v, &sh->kv_full[stage], c * 64, tp.hx0, row, hi, bi);
        }
        __syncwarp();
        if (++stage == pl.stages) { stage = 0; stage_par ^= 1; ring_full = true; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // Everything this warp needs per block is kept incrementally (ring indices, barrier parities,
    // descriptor bases), and each kind of MMA group has exactly one issue site.
    const uint32_t fmt = BF16 ? 1u : 0u;
    const uint32_t idesc_s = instr_desc(fmt, 128, N, 0, 0);
    const uint32_t idesc_pv = instr_desc(fmt, 128, o_cols, 0, 1);
    const uint32_t hi_sw = smem_desc_hi(1024, true), hi_ns = smem_desc_hi(kXSbo, false);
    const uint64_t q_desc0 = smem_desc_from(smem_u32(q_smem), 16, hi_sw), k_desc0 = smem_desc_from(smem_u32(k_smem), 16, hi_sw),
                   v_desc0 = smem_desc_from(smem_u32(v_smem), blk_bytes, hi_sw),
                   qx_desc0 = smem_desc_from(smem_u32(qx_smem), kXLbo, hi_ns), kx_desc0 = smem_desc_from(smem_u32(kx_smem), kXLbo, hi_ns);
    const uint32_t k_stage16 = k_stage >> 4, v_stage16 = v_stage >> 4, kx_stage16 = kx_stage >> 4, blk16 = blk_bytes >> 4;
    const int nks = N >> 4;
    // score side: runs `nsb` blocks ahead of the PV side
    int s_it = 0, s_item = blockIdx.x, s_j = 0, s_nblk = 1, s_stage = 0, s_stage_par = 0, s_buf = 0;
    // PV side
    int p_it = 0, p_item = blockIdx.x, p_j = 0, p_nblk = 1, p_stage = 0, p_buf = 0, p_buf_par = 0, p_grp = 0;
    if (s_item < n_items) s_nblk = p_nblk = item_blocks(p, s_item, tiles_per_head);
    int lead = nsb;
    while (true) {
      if (lead > 0) {
        --lead;
      } else {
        if (p_item >= n_items) break;
        // ---- O_g += P V for the block at the PV cursor
        const bool first = p_j < 2;                       // first block of this item for group p_grp: O_g starts over
        wait_spin(&sh->p_full[p_buf], p_buf_par);
        if (first && p_it >= 1) wait_spin(&sh->o_free, (p_it - 1) & 1);   // the previous item's O_g has been read
        if (ok) {
          tc_fence_after();
          if (elect_one()) {
            const uint32_t pa = tmem + p_buf * s_stride, od = tmem + o_base + p_grp * o_cols;
            uint64_t vd = v_desc0 + (uint64_t)(p_stage * v_stage16);
            uint32_t acc = first ? 0u : 1u;
#pragma unroll 1
            for (int ks = 0; ks < nks; ++ks, vd += 128, acc = 1u) umma_ts(od, pa + ks * 8, vd, idesc_pv, acc);
            umma_commit(&sh->kv_empty[p_stage]);
            umma_commit(&sh->pv_done[p_grp]);
            if (p_j == p_nblk - 1) umma_commit(&sh->o_full);
            if (p_it == p.trace_it) trace_mark(p, 1, 2 + 2 * p_j);
          }
          __syncwarp();
        }
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
      if (s_item < n_items) {
        // ---- S = Q K^T + mask for the block at the score cursor
        const int qb = s_it & 1;
        if (s_j == 0) wait_spin(&sh->q_ready[qb], (s_it >> 1) & 1);
        wait_spin(&sh->k_ready[s_stage], s_stage_par);
        // score buffer s_buf is free: the PV MMA of the block that used it last was issued before this one
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
            if (s_j == s_nblk - 1) umma_commit(&sh->q_empty[qb]);   // last read of this query buffer
            if (s_it == p.trace_it) trace_mark(p, 1, 1 + 2 * s_j);
          }
          __syncwarp();
        }
        if (++s_stage == pl.stages) { s_stage = 0; s_stage_par ^= 1; }
        if (++s_buf == nsb) s_buf = 0;
        if (++s_j == s_nblk) {
          s_j = 0;
          ++s_it;
          s_item += gridDim.x;
          if (s_item < n_items) s_nblk = item_blocks(p, s_item, tiles_per_head);
        }
      } else {
        lead = 0;                        // nothing left to issue ahead
      }
    }
  } else {
    // ------------------------------------------------------------------ fused RoPE-2D on Q and K tiles, mask tiles
    // One loop over the "units" of an item: unit -1 is the query tile, units 0.. are the K blocks.
    const int t = warp < 4 ? (int)threadIdx.x - 64 : (int)threadIdx.x - 384 + 64;
    const bool rope_on = NI > 0 && p.rope.idx != nullptr;
    const RopeParts qp = rope_parts_n(t, 128, kFwdRopeThreads), kp = rope_parts_n(t, N, kFwdRopeThreads);   // share of a Q tile / of a K block
    write_indicator_row<BF16>(qx_smem, qp.row, qp.lo, qp.hi, p);      // the same for every item
    const int kjr = kp.row / pl.KW, kjc = kp.row % pl.KW;             // this thread's row inside every streamed block
    int stage = 0, stage_par = 0;
    RopeRow rc;                                        // register cache of cos/sin values (only without TABS)
    rc.pos[0] = rc.pos[1] = -1;
    RopeTabs tabs;
    tabs.row_addr = smem_u32(tab_smem);
    tabs.col_addr = tabs.row_addr + (uint32_t)p.rope.max_h * rope_tab_stride(p.rope.R);
#pragma unroll 1
    for (int it = 0, item = blockIdx.x; item < n_items; ++it, item += gridDim.x) {
      const int bh = item / tiles_per_head;
      const TilePos tp = tile_pos(p, item - bh * tiles_per_head);
      const int qb = it & 1;
      const int qr = tp.r0 + qp.row / pl.TW, qx = tp.x0 + qp.row % pl.TW;
      const bool q_in = qr < p.t_h && qx < p.Wtok;
      const int kx = tp.hx0 + kjc;
      const bool kx_in = kp.active && kx >= 0 && kx < p.Wtok;
      int32_t idx_cur = -1;
      if (rope_on && q_in) idx_cur = __ldg(p.rope.idx + qr * p.Wtok + qx);
      named_bar_sync(5, kFwdRopeThreads);           // nobody still reads the previous item's tables
      build_penalty_tables<BF16>(&sh->pen, t, p, tp, kFwdRopeThreads);
      named_bar_sync(5, kFwdRopeThreads);                       // the tables are complete before any of these warps reads them
      RopeParts parts = qp;
#pragma unroll 1
      for (int j = -1; j < tp.nblk; ++j) {
        const bool isq = j < 0;
        // cos/sin of this thread's row of this unit: in flight while the unit's tile arrives
        if constexpr (!TABS) {
          if (rope_on) rope_fetch_t<NI>(rc, idx_cur, parts, p.rope);
        }
        // index of this thread's row of the next unit (always a K block)
        const int kr_next = tp.hr_first + (j + 1) * pl.KR + kjr;
        int32_t idx_next = -1;
        if (rope_on && kx_in && j + 1 < tp.nblk && kr_next < p.t_h) idx_next = __ldg(p.rope.idx + kr_next * p.Wtok + kx);
        // the stage (K, V and penalty rows) is free once its refill has landed: the producer refills
        // only after every MMA of the stage's previous block has completed
        wait_park(isq ? &sh->q_full[qb] : &sh->kv_full[stage], isq ? (uint32_t)((it >> 1) & 1) : (uint32_t)stage_par);
        if (t == 0 && it == p.trace_it) trace_mark(p, 3, 3 + 2 * j);
        if (ok) {
          if (!isq && kp.active)
            write_penalty_row(kx_smem + stage * kx_stage, kp.row, kp.lo, kp.hi, &sh->pen, j * pl.KR + kjr, kjc, pl.TH >> 3, pl.TW >> 3);
          if (rope_on) {  // a row outside the grid carries index -1: both halves un-rotated
            uint8_t* const tile = isq ? q_smem + qb * q_bytes : k_smem + stage * k_stage;
            if constexpr (TABS) rope_apply_s<BF16, NI>(tile, isq ? 16384u : blk_bytes, idx_cur, parts, p.rope, tabs);
            else rope_apply_t<BF16, NI>(tile, isq ? 16384u : blk_bytes, rc, parts, p.rope);
          }
          fence_proxy_async_smem();
          mbar_arrive(isq ? &sh->q_ready[qb] : &sh->k_ready[stage]);
        }
        if (t == 0 && it == p.trace_it) trace_mark(p, 3, 4 + 2 * j);
        if (!isq && ++stage == pl.stages) { stage = 0; stage_par ^= 1; }
        idx_cur = idx_next;
        parts = kp;
      }
    }
  }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // let whatever is still in flight (TMA, MMA) land before shared memory and TMEM are released
#pragma unroll 1
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
