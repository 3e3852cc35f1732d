// tcgen05 backward kernels.  One template covers both passes; they differ in which side is resident:
//
//   dQ    (DKDV = false)  resident X = (Q, dO) of 128 queries, streamed Y = (K, V) halo blocks:
//                          S = Q K^T, dP = dO V^T, P = exp2(c S - lse), dS = P o (dP - delta),
//                          dQ += dS K
//   dK/dV (DKDV = true)   resident X = (K, V) of 128 keys, streamed Y = (Q, dO) halo blocks with the
//                          queries' lse / delta:  S^T = K Q^T, dP^T = V dO^T, P^T, dS^T likewise,
//                          dV += P^T dO, dK += dS^T Q
//
// The tile-window relation is symmetric, so halo, window mask (32 extra contraction columns of the
// score MMA) and RoPE handling are the same for both.  RoPE-2D is fused: q and k tiles are rotated in
// shared memory before the MMAs, dQ / dK are rotated back in the epilogue registers.
//
// Persistent: one CTA per SM walks the work items (resident tiles); the resident tile is
// double-buffered where shared memory allows, so loading and rotating the next tile overlaps the
// current one.  The streamed blocks of all items form one stream G = 0, 1, ...; two groups of
// compute warps (one thread per resident row each) take the even resp. odd blocks, each with its own
// (S, dP) buffer pair in tensor memory.  A thread turns its row of S / dP into P / dS 16 columns at
// a time and stores them, packed to 16 bits, over the columns it has read; the accumulating MMAs
// read them from there as their A operand (no shared-memory round trip).
//
// Warp roles (512 threads): warp 0 TMA producer; warp 1 MMA issuer; warps 4-7 / 8-11 compute
// groups 0 / 1; warps 2-3 and 12-15 RoPE, window-mask tiles and lse / delta staging.
// Every inner loop is a real loop with a small body and the RoPE width is a template parameter: the
// kernel is instruction-fetch bound in its scalar roles otherwise.
// All waits are bounded; a timed-out wait raises a CTA-wide abort flag, every role runs its
// loops to the end without touching anything, TMEM is freed and the status word records it.
#pragma once

#include "swa_tc_common.cuh"

namespace swa {
namespace tc {

constexpr int kBwdThreads = 512;
constexpr int kBwdRopeThreads = 192;
constexpr uint32_t kBwdTmemCols = 512;

struct BwdShared {
  uint64_t x_full[2], x_ready[2], x_empty[2];
  uint64_t y_full[kMaxStages], y_ready[kMaxStages], y_empty[kMaxStages];
  uint64_t sd_full[2], ds_full[2], acc_full, acc_free;
  PenaltyTables pen;
  uint32_t tmem_base;
  int abort_flag;
  int abort_site;   // which wait gave up first (debugging aid, reported in the status word)
};

// Rotate back (transposed rotation) one group of pairs held in registers: x0' = x0 c + x1 s, x1' = x1 c - x0 s.
template <int NP>
__device__ __forceinline__ void inv_rotate_pairs(float* x0, float* x1, const float2* cs) {
#pragma unroll
  for (int e = 0; e < NP; ++e) {
    const float a = x0[e], b = x1[e];
    x0[e] = a * cs[e].x + b * cs[e].y;
    x1[e] = b * cs[e].x - a * cs[e].y;
  }
}

template <bool BF16>
__device__ __forceinline__ void store16(void* dst, const float* v) {
  uint4* d = reinterpret_cast<uint4*>(dst);
  d[0] = make_uint4(pack2<BF16>(v[0], v[1]), pack2<BF16>(v[2], v[3]), pack2<BF16>(v[4], v[5]), pack2<BF16>(v[6], v[7]));
  d[1] = make_uint4(pack2<BF16>(v[8], v[9]), pack2<BF16>(v[10], v[11]), pack2<BF16>(v[12], v[13]), pack2<BF16>(v[14], v[15]));
}

template <bool BF16, bool DKDV, int NI, bool TABS>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_kernel(const __grid_constant__ CUtensorMap tm_xqk, const __grid_constant__ CUtensorMap tm_xv,
            const __grid_constant__ CUtensorMap tm_yqk, const __grid_constant__ CUtensorMap tm_yv, KParams p,
            const float* __restrict__ lse, const float* __restrict__ delta, View4 out_qk, View4 out_v) {
  using namespace ptx;
  constexpr int R = 8 * NI;
  constexpr int Rd = NI > 0 ? R : 1;   // divisor that stays legal when there is no rotation
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const Plan& pl = p.pl;
  const int N = pl.N, nxb = pl.nxb;
  constexpr int nsb = 2;                                         // (S, dP) buffer pairs; the planner sizes N so that two fit
  const uint32_t blk_bytes = (uint32_t)N * 128u;               // one 64-wide chunk of a streamed block
  const uint32_t xqk_bytes = p.qch * 16384u, xv_bytes = p.vch * 16384u, x_bytes = xqk_bytes + xv_bytes;
  const uint32_t yqk_stage = blk_bytes * p.qch, yv_stage = blk_bytes * p.vch;
  const uint32_t yx_stage = (uint32_t)N * kXRowBytes;
  uint8_t* x_smem = smem;                                        // nxb buffers of (qk chunks, v chunks)
  uint8_t* xx_smem = x_smem + nxb * x_bytes;                    // window-mask indicator rows of a resident tile
  uint8_t* yqk_smem = xx_smem + 128 * kXRowBytes;
  uint8_t* yv_smem = yqk_smem + pl.stages * yqk_stage;
  uint8_t* yx_smem = yv_smem + pl.stages * yv_stage;
  float* vec_smem = reinterpret_cast<float*>(yx_smem + pl.stages * yx_stage);   // [stage][-lse | delta][128]
  BwdShared* sh = reinterpret_cast<BwdShared*>(reinterpret_cast<uint8_t*>(vec_smem) + pl.stages * 1024);
  uint8_t* tab_smem = reinterpret_cast<uint8_t*>(sh) + ((sizeof(BwdShared) + 15) & ~size_t(15));   // cos/sin tables (TABS)
  volatile int* abort_flag = &sh->abort_flag;
  // tensor memory: buffer pair b = (S at 2N b, dP at 2N b + N), accumulators behind the pairs
  const uint32_t acc_qk = nsb * 2 * N, acc_v = acc_qk + p.qch * 64;

  const int warp = threadIdx.x >> 5;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sh->x_full[s], 1);
      mbar_init(&sh->x_ready[s], kBwdRopeThreads);
      mbar_init(&sh->x_empty[s], 1);
      mbar_init(&sh->sd_full[s], 1);
      mbar_init(&sh->ds_full[s], 128);
    }
    mbar_init(&sh->acc_full, 1);
    mbar_init(&sh->acc_free, 256);
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(&sh->y_full[s], 1);
      mbar_init(&sh->y_ready[s], kBwdRopeThreads);
      mbar_init(&sh->y_empty[s], 1);
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

  bool ok = true;   // warp-uniform; see the forward kernel
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

  // Registers follow the work: the kernel starts with 128 per thread; the producer / issuer / RoPE
  // warpgroups (warps 0-3 and 12-15) give some back, the two compute warpgroups take them.
  // (2 * 104 + 2 * 152) * 128 = 64 Ki.  Not done in the variant whose RoPE warps keep cos/sin rows in registers.  Each setmaxnreg is the first instruction of its branch, so that the
  // whole branch is compiled for that budget.
  if (warp >= 4 && warp < 12) {
    if constexpr (TABS || NI == 0) setmaxnreg_inc<152>();
    // ------------------------------------------------------------------ P / dS, one thread per resident row and group
    const int lane = threadIdx.x & 31;
    const int g = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int m = quarter * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    const float c2 = p.scale_log2;
    const int ng = N >> 4;
    uint32_t gbase = 0, own_next = g;
    // this group's next block: buffer pair (group g owns pair g, every block flips its parity), stage of
    // the ring and its parity
    const int buf = g;
    int buf_par = 0;
    int stage = g % pl.stages, stage_par = (g / pl.stages) & 1;
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    // (cos, sin) of NP consecutive pairs starting at pair `first` of table row `pos` (row or column table):
    // from the staged tables in shared memory when there are any, else from global memory; identity for pos < 0
    const uint32_t tab_row_addr = smem_u32(tab_smem), tab_col_addr = tab_row_addr + (uint32_t)p.rope.max_h * rope_tab_stride(Rd);
    auto load_pairs = [&](float2* cs, bool col, int pos, int first) {
      constexpr int NP = R >= 16 ? 16 : 8;
      if (pos < 0) {
#pragma unroll
        for (int e = 0; e < NP; ++e) cs[e] = make_float2(1.f, 0.f);
      } else if constexpr (TABS) {
        const uint32_t a = (col ? tab_col_addr : tab_row_addr) + (uint32_t)pos * rope_tab_stride(Rd) + first * 8;
#pragma unroll
        for (int e = 0; e < NP; e += 2) {
          const uint4 u = lds128(a + e * 8);
          cs[e] = make_float2(__uint_as_float(u.x), __uint_as_float(u.y));
          cs[e + 1] = make_float2(__uint_as_float(u.z), __uint_as_float(u.w));
        }
      } else {
        const float2* trow = reinterpret_cast<const float2*>((col ? p.rope.col_cs : p.rope.row_cs) + (int64_t)pos * Rd * 2) + first;
#pragma unroll
        for (int e = 0; e < NP; ++e) cs[e] = __ldg(trow + e);
      }
    };
    // Without RoPE the epilogue of an item is deferred until this thread has worked on its first block of
    // the NEXT item: the last accumulating MMAs of an item complete long after a group has finished its
    // own last block, and the score MMAs of the next item's first blocks have been issued by then.  (With
    // RoPE the rotating warps set the pace and holding back the first accumulating MMA of the next item,
    // which frees a stage of the ring, costs more than the tail; measured.)
    constexpr bool kDefer = NI == 0;
    bool pend = false;
    int pend_item = 0, pend_it = 0;
#pragma unroll 1
    for (int it = 0, item = blockIdx.x;; ++it, item += gridDim.x) {
      const bool have = item < n_items;
      TilePos tp;
      tp.r0 = tp.x0 = tp.hx0 = tp.hr_first = tp.hr_last = 0;
      tp.nblk = 0;
      const int bh = have ? item / tiles_per_head : 0;
      if (have) tp = tile_pos(p, item - bh * tiles_per_head);
      const int see_lo = tp.r0 + (quarter * 32) / pl.TW - p.wr, see_hi = tp.r0 + (quarter * 32 + 31) / pl.TW + p.wr;
      float my_nlse = -INFINITY, my_delta = 0.f;     // dQ: -lse and delta of this thread's query
      if (!DKDV && have) {
        const int tr = tp.r0 + m / pl.TW, tx = tp.x0 + m % pl.TW;
        if (tr < p.t_h && tx < p.Wtok) {
          const int64_t at = (int64_t)bh * p.t_h * p.Wtok + (int64_t)tr * p.Wtok + tx;
          my_nlse = -__ldg(lse + at);
          my_delta = __ldg(delta + at);
        }
      }
      int j = have ? (int)(own_next - gbase) : 0;
      bool first = true;
#pragma unroll 1
      while (true) {
      if (j < tp.nblk) {
        const uint32_t s_tm = lane_base + buf * 2 * N, d_tm = s_tm + N;
        uint64_t* const ds_bar = &sh->ds_full[buf];
        wait_spin(&sh->sd_full[buf], buf_par, 7);
        if (m == 0 && g == 0 && it == p.trace_it) trace_mark(p, 2, 1 + 2 * (j >> 1));
        const float* vec = vec_smem + stage * 256;
        if (DKDV) wait_spin(&sh->y_ready[stage], stage_par, 8);   // -lse / delta of the block's queries are staged
        // advance by two positions in the rings
        buf_par ^= 1;
        stage += 2;
        if (stage >= pl.stages) { stage -= pl.stages; stage_par ^= 1; }
        const int blk_first = tp.hr_first + j * pl.KR, blk_last = blk_first + pl.KR - 1;
        const bool seen = !(blk_last < see_lo || blk_first > see_hi);
        if (ok) {
        tc_fence_after();
        uint32_t sa[16], sb[16], da[16], db[16];
        if (!seen) {
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
        if (m == 0 && g == 0 && it == p.trace_it) trace_mark(p, 2, 2 + 2 * (j >> 1));
        j += 2;
        own_next += 2;
      }
      const bool at_end = j >= tp.nblk;
      if (kDefer ? first : at_end) {
      first = false;
      if (!kDefer && have) {                       // the item that has just ended
        pend = true;
        pend_item = item;
        pend_it = it;
      }
      if (pend) {
      pend = false;
      // ---- the pending item: this group stores its half of the accumulator row(s)
      const int e_bh = pend_item / tiles_per_head, bi = e_bh / p.H, hi = e_bh - bi * p.H;
      const TilePos e_tp = tile_pos(p, pend_item - e_bh * tiles_per_head);
      const int tr = e_tp.r0 + m / pl.TW, tx = e_tp.x0 + m % pl.TW;
      const bool t_in = tr < p.t_h && tx < p.Wtok;
      const int64_t tok = (int64_t)tr * p.Wtok + tx;
      // dQ / dK: columns [g W, g W + W), W = 32 qch; the partner of a rotated dim lies in the same half
      // Control flow below is warp-uniform (the tensor-memory loads are warp-collective): whether a
      // granule is rotated depends only on its dims; a thread whose token is outside the grid or has a
      // negative index half rotates by the identity.
      const bool rope_on = NI > 0 && p.rope.idx != nullptr;
      int irow = -1, icol = -1;
      if (rope_on && t_in) decode_idx(__ldg(p.rope.idx + tok), p.rope.max_h, p.rope.max_w, irow, icol);
      const int W = 32 * p.qch, base = g * W;
      // cos/sin of the first rotated pairs of this thread, fetched before the wait (served by L2)
      float2 cs[16];
      int pre_d0 = -1;                                // first dim of the granule(s) the prefetched pairs belong to
      if constexpr (NI > 0) {
        if (rope_on && base < 4 * R && ((base / Rd) & 1) == 0) {
          pre_d0 = base;
          const int seg = base / Rd;
          load_pairs(cs, seg >= 2, seg >= 2 ? icol : irow, base - seg * R);
        }
      }
      if (m == 0 && g == 0 && pend_it == p.trace_it) trace_mark(p, 2, 29);
      wait_spin(&sh->acc_full, pend_it & 1, 9);
      if (ok) {
        tc_fence_after();
        if (m == 0 && g == 0 && pend_it == p.trace_it) trace_mark(p, 2, 30);
        T* qk_row = (T*)out_qk.ptr + bi * out_qk.s0 + hi * out_qk.s1 + tok * out_qk.s2;
        const uint32_t aqk = lane_base + acc_qk;
        const float scale = p.sm_scale;
#pragma unroll 1
        for (int d0 = base; d0 < base + W; d0 += 16) {
          const bool roped = NI > 0 && rope_on && d0 < 4 * R;   // warp-uniform
          if (roped && R >= 16 && ((d0 / Rd) & 1) == 1) continue;        // stored together with its partner granule
          uint32_t ra[16], rb[16];
          float va[16], vb[16];
          tmem_ld16(aqk + d0, ra);
          if (roped && R >= 16) tmem_ld16(aqk + d0 + R, rb);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 16; ++e) va[e] = __uint_as_float(ra[e]) * scale;
          if constexpr (NI > 0) {
            if (roped) {
              if (d0 != pre_d0) {                                         // pairs that were not prefetched
                const int seg = d0 / Rd;
                load_pairs(cs, seg >= 2, seg >= 2 ? icol : irow, d0 - seg * R);
              }
              if constexpr (R >= 16) {
#pragma unroll
                for (int e = 0; e < 16; ++e) vb[e] = __uint_as_float(rb[e]) * scale;
                inv_rotate_pairs<16>(va, vb, cs);
                if (t_in) store16<BF16>(qk_row + d0 + R, vb);
              } else {
                inv_rotate_pairs<8>(va, va + 8, cs);
              }
            }
          }
          if (t_in) store16<BF16>(qk_row + d0, va);
        }
        if constexpr (DKDV) {
          T* v_row = (T*)out_v.ptr + bi * out_v.s0 + hi * out_v.s1 + tok * out_v.s2;
          const uint32_t av = lane_base + acc_v;
          const int Wv = 32 * p.vch;
#pragma unroll 1
          for (int d0 = g * Wv; d0 < g * Wv + Wv; d0 += 16) {
            uint32_t ra[16];
            float va[16];
            tmem_ld16(av + d0, ra);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 16; ++e) va[e] = __uint_as_float(ra[e]);
            if (t_in) store16<BF16>(v_row + d0, va);
          }
        }
        tc_fence_before();
        mbar_arrive(&sh->acc_free);
        if (m == 0 && g == 0 && pend_it == p.trace_it) trace_mark(p, 2, 31);
      }
      }
      }
      if (at_end) break;
      }
      if (!have) break;
      if (kDefer) {                                // this item's accumulators are stored during the next item
        pend = true;
        pend_item = item;
        pend_it = it;
      }
      gbase += tp.nblk;
    }
  } else {
    if constexpr (TABS || NI == 0) setmaxnreg_dec<104>();
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
        if (ring_full) wait_park(&sh->y_empty[stage], stage_par, 2);
        if (ok && elect_one()) {
          mbar_arrive_expect_tx(&sh->y_full[stage], yqk_stage + yv_stage);
          const int row = tp.hr_first + j * pl.KR;
#pragma unroll 1
          for (int c = 0; c < p.qch; ++c)
            tma_load_5d(yqk_smem + stage * yqk_stage + c * blk_bytes, &tm_yqk, &sh->y_full[stage], c * 64, tp.hx0, row, hi, bi);
#pragma unroll 1
          for (int c = 0; c < p.vch; ++c)
            tma_load_5d(yv_smem + stage * yv_stage + c * blk_bytes, &tm_yv, &sh->y_full[stage], c * 64, tp.hx0, row, hi, bi);
        }
        __syncwarp();
        if (++stage == pl.stages) { stage = 0; stage_par ^= 1; ring_full = true; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t fmt = BF16 ? 1u : 0u;
    const uint32_t idesc_s = instr_desc(fmt, 128, N, 0, 0);                 // S / dP: both operands K-major
    const uint32_t idesc_qk = instr_desc(fmt, 128, p.qch * 64, 0, 1);       // dQ / dK: B = streamed qk tile, MN-major
    const uint32_t idesc_v = instr_desc(fmt, 128, p.vch * 64, 0, 1);        // dV: B = streamed dO tile, MN-major
    const uint32_t hi_sw = smem_desc_hi(1024, true), hi_ns = smem_desc_hi(kXSbo, false);
    const uint64_t x_desc0 = smem_desc_from(smem_u32(x_smem), 16, hi_sw),
                   yqk_desc0 = smem_desc_from(smem_u32(yqk_smem), 16, hi_sw), yv_desc0 = smem_desc_from(smem_u32(yv_smem), 16, hi_sw),
                   yqk_mn0 = smem_desc_from(smem_u32(yqk_smem), blk_bytes, hi_sw), yv_mn0 = smem_desc_from(smem_u32(yv_smem), blk_bytes, hi_sw),
                   xx_desc0 = smem_desc_from(smem_u32(xx_smem), kXLbo, hi_ns), yx_desc0 = smem_desc_from(smem_u32(yx_smem), kXLbo, hi_ns);
    const uint32_t yqk16 = yqk_stage >> 4, yv16 = yv_stage >> 4, yx16 = yx_stage >> 4, blk16 = blk_bytes >> 4, x16 = x_bytes >> 4;
    const int nks = N >> 4;
    // score side (S, dP), `nsb` blocks ahead of the accumulating side
    int s_it = 0, s_item = blockIdx.x, s_j = 0, s_nblk = 1, s_stage = 0, s_stage_par = 0, s_buf = 0, s_xb = 0, s_xb_par = 0;
    // accumulating side
    int a_it = 0, a_item = blockIdx.x, a_j = 0, a_nblk = 1, a_stage = 0, a_buf = 0, a_buf_par = 0;
    if (s_item < n_items) s_nblk = a_nblk = item_blocks(p, s_item, tiles_per_head);
    int lead = nsb;
#pragma unroll 1
    while (true) {
      if (lead > 0) {
        --lead;
      } else {
        if (a_item >= n_items) break;
        // ---- accumulate the block at the accumulating cursor: A operands come from tensor memory
        wait_spin(&sh->ds_full[a_buf], a_buf_par, 3);
        if (a_j == 0 && a_it >= 1) wait_spin(&sh->acc_free, (a_it - 1) & 1, 4);   // the previous item's accumulators have been read
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
            umma_commit(&sh->y_empty[a_stage]);
            if (a_j == a_nblk - 1) umma_commit(&sh->acc_full);
            if (a_it == p.trace_it) trace_mark(p, 1, 2 + 2 * a_j);
          }
          __syncwarp();
        }
        if (++a_stage == pl.stages) a_stage = 0;
        if (++a_buf == nsb) { a_buf = 0; a_buf_par ^= 1; }
        if (++a_j == a_nblk) {
          a_j = 0;
          ++a_it;
          a_item += gridDim.x;
          if (a_item < n_items) a_nblk = item_blocks(p, a_item, tiles_per_head);
        }
      }
      if (s_item < n_items) {
        // ---- S (+ mask) and dP for the block at the score cursor
        if (s_j == 0) wait_spin(&sh->x_ready[s_xb], s_xb_par, 5);
        wait_spin(&sh->y_ready[s_stage], s_stage_par, 6);
        // buffer pair s_buf is free: the accumulating MMAs of the block that used it last were issued before
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
            if (s_j == s_nblk - 1) umma_commit(&sh->x_empty[s_xb]);   // last read of this resident buffer
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
          if (++s_xb == nxb) { s_xb = 0; s_xb_par ^= 1; }
          if (s_item < n_items) s_nblk = item_blocks(p, s_item, tiles_per_head);
        }
      } else {
        lead = 0;
      }
    }
  } else {
    // ------------------------------------------------------------------ RoPE on the qk tiles, mask tiles, lse / delta staging
    // One loop over the "units" of an item: unit -1 is the resident tile, units 0.. are the streamed blocks.
    const int t = warp < 4 ? (int)threadIdx.x - 64 : (int)threadIdx.x - 384 + 64;
    const bool rope_on = NI > 0 && p.rope.idx != nullptr;
    const RopeParts xp = rope_parts_n(t, 128, kBwdRopeThreads), yp = rope_parts_n(t, N, kBwdRopeThreads);
    write_indicator_row<BF16>(xx_smem, xp.row, xp.lo, xp.hi, p);      // the same for every item
    const int yjr = yp.row / pl.KW, yjc = yp.row % pl.KW;             // this thread's row inside every streamed block
    const int vjr = t / pl.KW, vjc = t % pl.KW;                       // the row whose lse / delta this thread stages
    int stage = 0, stage_par = 0, xb = 0, xb_par = 0;
    RopeRow rc;                                        // register cache of cos/sin values (only without TABS)
    rc.pos[0] = rc.pos[1] = -1;
    RopeTabs tabs;
    tabs.row_addr = smem_u32(tab_smem);
    tabs.col_addr = tabs.row_addr + (uint32_t)p.rope.max_h * rope_tab_stride(p.rope.R);
    float nlse_cur = -INFINITY, delta_cur = 0.f;       // lse / delta of this thread's row of the current unit
#pragma unroll 1
    for (int it = 0, item = blockIdx.x; item < n_items; ++it, item += gridDim.x) {
      const int bh = item / tiles_per_head;
      const TilePos tp = tile_pos(p, item - bh * tiles_per_head);
      const int64_t vec_base = (int64_t)bh * p.t_h * p.Wtok;
      const int xr = tp.r0 + xp.row / pl.TW, xc = tp.x0 + xp.row % pl.TW;
      const bool x_in = xr < p.t_h && xc < p.Wtok;
      const int yc = tp.hx0 + yjc;
      const bool yc_in = yp.active && yc >= 0 && yc < p.Wtok;
      const int vc = tp.hx0 + vjc;
      const bool vc_in = t < N && vc >= 0 && vc < p.Wtok;
      int32_t idx_cur = -1;
      if (rope_on && x_in) idx_cur = __ldg(p.rope.idx + xr * p.Wtok + xc);
      named_bar_sync(5, kBwdRopeThreads);           // nobody still reads the previous item's tables
      build_penalty_tables<BF16>(&sh->pen, t, p, tp, kBwdRopeThreads);
      named_bar_sync(5, kBwdRopeThreads);
      RopeParts parts = xp;
#pragma unroll 1
      for (int j = -1; j < tp.nblk; ++j) {
        const bool isx = j < 0;
        if constexpr (!TABS) {
          if (rope_on) rope_fetch_t<NI>(rc, idx_cur, parts, p.rope);
        }
        const int yr_next = tp.hr_first + (j + 1) * pl.KR + yjr;
        int32_t idx_next = -1;
        if (rope_on && yc_in && j + 1 < tp.nblk && yr_next < p.t_h) idx_next = __ldg(p.rope.idx + yr_next * p.Wtok + yc);
        // -lse and delta of the NEXT block's queries (thread t stages both values of block row t): loaded one
        // unit ahead, so the latency is hidden behind this unit's work
        float nlse_next = -INFINITY, delta_next = 0.f;
        if constexpr (DKDV) {
          const int vr = tp.hr_first + (j + 1) * pl.KR + vjr;
          if (j + 1 < tp.nblk && vc_in && vr < p.t_h) {
            nlse_next = -__ldg(lse + vec_base + (int64_t)vr * p.Wtok + vc);
            delta_next = __ldg(delta + vec_base + (int64_t)vr * p.Wtok + vc);
          }
        }
        // a stage (tiles, penalty rows, lse / delta slots) is free once its refill has landed: the producer
        // refills only after every MMA of the stage's previous block has completed, which in turn is
        // after the compute warps finished reading that block's lse / delta
        wait_park(isx ? &sh->x_full[xb] : &sh->y_full[stage], isx ? (uint32_t)xb_par : (uint32_t)stage_par, 10);
        if (t == 0 && it == p.trace_it) trace_mark(p, 3, 3 + 2 * j);
        if (ok) {
          if (!isx && yp.active)
            write_penalty_row(yx_smem + stage * yx_stage, yp.row, yp.lo, yp.hi, &sh->pen, j * pl.KR + yjr, yjc, pl.TH >> 3, pl.TW >> 3);
          if (rope_on) {
            uint8_t* const tile = isx ? x_smem + xb * x_bytes : yqk_smem + stage * yqk_stage;
            if constexpr (TABS) rope_apply_s<BF16, NI>(tile, isx ? 16384u : blk_bytes, idx_cur, parts, p.rope, tabs);
            else rope_apply_t<BF16, NI>(tile, isx ? 16384u : blk_bytes, rc, parts, p.rope);
          }
          if constexpr (DKDV) {
            if (!isx && t < N) {
              vec_smem[stage * 256 + t] = nlse_cur;
              vec_smem[stage * 256 + 128 + t] = delta_cur;
            }
          }
          fence_proxy_async_smem();
          mbar_arrive(isx ? &sh->x_ready[xb] : &sh->y_ready[stage]);
        }
        if (t == 0 && it == p.trace_it) trace_mark(p, 3, 4 + 2 * j);
        if (isx) {
          if (++xb == nxb) { xb = 0; xb_par ^= 1; }
        } else if (++stage == pl.stages) {
          stage = 0;
          stage_par ^= 1;
        }
        idx_cur = idx_next;
        nlse_cur = nlse_next;
        delta_cur = delta_next;
        parts = yp;
      }
    }
  }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // let whatever is still in flight (TMA, MMA) land before shared memory and TMEM are released
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    if (threadIdx.x == 0) report_abort(p.status, DKDV ? 3 : 2, sh->abort_site);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kBwdTmemCols);
  }
}

}  // namespace tc
}  // namespace swa
