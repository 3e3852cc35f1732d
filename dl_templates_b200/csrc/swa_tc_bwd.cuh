// tcgen05 backward kernels.  One template serves both launches:
//
//   DKDV = false  (dQ kernel)    resident tile X = (Q, dO) of 128 queries,
//                                streamed blocks Y = (K, V) of the halo keys
//   DKDV = true   (dK/dV kernel) resident tile X = (K, V) of 128 keys,
//                                streamed blocks Y = (Q, dO) of the halo queries
//
// Per streamed block (N <= 128 tokens), with T = the resident token (one TMEM lane):
//   S  = Xqk Yqk^T  (+ the window mask as 32 extra contraction columns)
//   dP = Xv  Yv^T
//   P  = exp2(scale*log2e * S - lse[query])      (exactly 0 outside the window)
//   dS = P * (dP - delta[query])
//   acc_qk += dS Yqk        (dQ resp. dK, before the sm_scale factor)
//   acc_v  += P  Yv         (dV; dK/dV kernel only)
// lse/delta belong to the query: the row's own scalar in the dQ kernel, one value per
// streamed column (staged in shared memory) in the dK/dV kernel.  P is recomputed
// from the saved logsumexp, nothing is accumulated with atomics, and RoPE-2D is
// fused: q/k tiles are rotated in shared memory before the MMAs and the dQ / dK rows
// are rotated back in registers before they are stored.
//
// Warp roles (448 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner (both
// keep the whole warp in uniform control flow and let one elected lane issue),
// warps 2-9 compute: TWO threads per resident token -- warps w and w+4 share a TMEM
// lane quarter and take the lower / upper half of each block's columns -- then the
// epilogue; warps 10-13 RoPE rotation of the tiles (two threads per row of a streamed block:
// row-angle and column-angle pairs), the window-mask tiles and staging of lse/delta.  S and dP are double-buffered in TMEM so the tensor core works on
// block j+1 while the compute warps work on j.
// TMEM columns: S[2] at 0/64, dP[2] at 128/192, acc_qk at 256, acc_v at 384.
#pragma once

#include <type_traits>

#include "swa_tc_common.cuh"

namespace swa {
namespace tc {

struct BwdBars {
  uint64_t x_full, x_ready, acc_done;
  uint64_t y_full[kMaxStages], y_ready[kMaxStages], y_empty[kMaxStages];
  uint64_t sd_full[2], sd_empty[2], op_full[2], op_empty[2];
  PenaltyTables pen;  // window-mask penalty parts of this CTA's halo rows / columns
  uint32_t tmem_base;
  int abort_flag;
};

constexpr int kBwdThreads = 448;
constexpr int kBwdRopeThread0 = 320;
constexpr uint32_t kBwdTmemCols = 512;
constexpr uint32_t kTmS = 0, kTmDP = 128, kTmAccQK = 256, kTmAccV = 384;

// cos/sin pairs needed to rotate back W consecutive dims (starting at dim BASE) of a dQ/dK row: pair e of
// the piece is dims (BASE+e, BASE+e+R).  Fetched before the final wait so that the table latency (L2)
// is hidden.  For the supported n_rdim (8, 16, 32) and piece widths both elements of a pair fall into
// the same piece.
template <int W>
struct EpiRope {
  float2 cs[W / 2];
};

template <int R, int BASE, int W>
__device__ __forceinline__ void epi_fetch_n(EpiRope<W>& c, int irow, int icol, const RopeDev& rp) {
  int n = 0;
#pragma unroll
  for (int e = 0; e < W; ++e) {
    const int d = BASE + e;
    if (d < 4 * R && ((d / R) & 1) == 0 && e + R < W) {
      const int seg = d / R;
      const int pos = seg >= 2 ? icol : irow;
      c.cs[n] = pos >= 0 ? __ldg(reinterpret_cast<const float2*>((seg >= 2 ? rp.col_cs : rp.row_cs) +
                                                                 ((int64_t)pos * R + (d - seg * R)) * 2))
                         : make_float2(1.f, 0.f);
      ++n;
    }
  }
}

template <int BASE, int W>
__device__ __forceinline__ void epi_fetch(EpiRope<W>& c, bool rot, int irow, int icol, const RopeDev& rp) {
  if (!rot) return;
#ifdef SWA_ROPE_ONLY_R
  epi_fetch_n<SWA_ROPE_ONLY_R, BASE, W>(c, irow, icol, rp);
#else
  switch (rp.R) {
    case 8: epi_fetch_n<8, BASE, W>(c, irow, icol, rp); break;
    case 16: epi_fetch_n<16, BASE, W>(c, irow, icol, rp); break;
    case 32: epi_fetch_n<32, BASE, W>(c, irow, icol, rp); break;
    default: break;
  }
#endif
}

// Rotate back (transposed rotation) the piece held in registers with the prefetched pairs.
template <int R, int BASE, int W>
__device__ __forceinline__ void inv_rotate_piece(float (&v)[W], const EpiRope<W>& c) {
  int n = 0;
#pragma unroll
  for (int e = 0; e < W; ++e) {
    const int d = BASE + e;
    if (d < 4 * R && ((d / R) & 1) == 0 && e + R < W) {
      const float2 cs = c.cs[n];
      ++n;
      const float x0 = v[e], x1 = v[(e + R) % W];
      v[e] = x0 * cs.x + x1 * cs.y;
      v[(e + R) % W] = x1 * cs.x - x0 * cs.y;
    }
  }
}

// Load W accumulator columns (starting at column BASE) of this thread's TMEM lane, scale,
// optionally rotate back, store W 16-bit elements at dst_row + BASE.
template <bool BF16, int BASE, int W>
__device__ __forceinline__ void store_acc_piece(uint32_t taddr, float scale, bool rot, const EpiRope<W>& c, int R,
                                                void* dst_row, bool in_grid) {
  using namespace ptx;
  uint32_t raw[W];
#pragma unroll
  for (int k = 0; k < W / 16; ++k) tmem_ld16(taddr + BASE + k * 16, &raw[k * 16]);
  tmem_wait_ld();
  float v[W];
#pragma unroll
  for (int e = 0; e < W; ++e) v[e] = __uint_as_float(raw[e]) * scale;
  if (rot) {
#ifdef SWA_ROPE_ONLY_R
    inv_rotate_piece<SWA_ROPE_ONLY_R, BASE, W>(v, c);
#else
    switch (R) {
      case 8: inv_rotate_piece<8, BASE, W>(v, c); break;
      case 16: inv_rotate_piece<16, BASE, W>(v, c); break;
      case 32: inv_rotate_piece<32, BASE, W>(v, c); break;
      default: break;
    }
#endif
  }
  if (in_grid) {
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(dst_row) + BASE * 2);
#pragma unroll
    for (int u = 0; u < W / 8; ++u)
      dst[u] = make_uint4(pack2<BF16>(v[u * 8], v[u * 8 + 1]), pack2<BF16>(v[u * 8 + 2], v[u * 8 + 3]),
                          pack2<BF16>(v[u * 8 + 4], v[u * 8 + 5]), pack2<BF16>(v[u * 8 + 6], v[u * 8 + 7]));
  }
}

template <bool BF16, bool DKDV>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_kernel(const __grid_constant__ CUtensorMap tm_xqk, const __grid_constant__ CUtensorMap tm_xv,
           const __grid_constant__ CUtensorMap tm_yqk, const __grid_constant__ CUtensorMap tm_yv, KParams p,
           const float* __restrict__ lse, const float* __restrict__ delta, View4 out_qk, View4 out_v) {
  using namespace ptx;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const Plan& pl = p.pl;
  const int N = pl.N;
  const uint32_t blk_bytes = (uint32_t)N * 128u;
  const uint32_t yqk_stage = blk_bytes * p.qch, yv_stage = blk_bytes * p.vch;
  constexpr int kOps = DKDV ? 2 : 1;                       // 16-bit operand tiles written per block: dS (and P)
  const int pch = (N + 63) >> 6;                           // 64-column chunks of such a tile
  const int nsb = N <= 64 ? 2 : 1;                         // S / dP buffers in TMEM
  const uint32_t yx_stage = (uint32_t)N * kXRowBytes;      // window-mask penalty rows of a streamed block
  uint8_t* xqk_smem = smem;
  uint8_t* xv_smem = xqk_smem + p.qch * 16384;
  uint8_t* xx_smem = xv_smem + p.vch * 16384;              // window-mask indicator rows of the resident tile
  uint8_t* yqk_smem = xx_smem + 128 * kXRowBytes;
  uint8_t* yv_smem = yqk_smem + pl.stages * yqk_stage;
  uint8_t* yx_smem = yv_smem + pl.stages * yv_stage;
  uint8_t* op_smem = yx_smem + pl.stages * yx_stage;       // [pbufs][kOps][pch][128 x 64] : dS then P
  float* vec_smem = reinterpret_cast<float*>(op_smem + pl.pbufs * kOps * pch * 16384);  // [stages][2][128]: lse, delta
  BwdBars* bars = reinterpret_cast<BwdBars*>(reinterpret_cast<uint8_t*>(vec_smem) + kMaxStages * 2 * 128 * 4);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int bh = blockIdx.y, bi = bh / p.H, hi = bh - bi * p.H;
  const TilePos tp = tile_pos(p, blockIdx.x);
  const int64_t vec_base = (int64_t)bh * p.t_h * p.Wtok;
  if (threadIdx.x == 64) trace_mark(p, 0, 31);

  if (threadIdx.x == 0) {
    mbar_init(&bars->x_full, 1);
    mbar_init(&bars->x_ready, 256);
    mbar_init(&bars->acc_done, 1);
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(&bars->y_full[s], 1);
      mbar_init(&bars->y_ready[s], 128);
      mbar_init(&bars->y_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->sd_full[s], 1);
      mbar_init(&bars->sd_empty[s], 256);
      mbar_init(&bars->op_full[s], 256);
      mbar_init(&bars->op_empty[s], 1);
    }
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, kBwdTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  // `ok` is kept warp-uniform in every role: a failed (timed-out) wait is agreed on by the warp.
  bool ok = true;
  auto wait_spin = [&](uint64_t* bar, uint32_t parity) {
    const bool r = ok && mbar_wait<0>(bar, parity, abort_flag);
    ok = __all_sync(0xffffffffu, r);
  };
  auto wait_park = [&](uint64_t* bar, uint32_t parity) {
    const bool r = ok && mbar_wait<100>(bar, parity, abort_flag);
    ok = __all_sync(0xffffffffu, r);
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (whole warp, one lane issues)
    if (elect_one()) {
      prefetch_tmap(&tm_xqk);
      prefetch_tmap(&tm_xv);
      prefetch_tmap(&tm_yqk);
      prefetch_tmap(&tm_yv);
      mbar_arrive_expect_tx(&bars->x_full, (p.qch + p.vch) * 16384);
      for (int c = 0; c < p.qch; ++c) tma_load_5d(xqk_smem + c * 16384, &tm_xqk, &bars->x_full, c * 64, tp.x0, tp.r0, hi, bi);
      for (int c = 0; c < p.vch; ++c) tma_load_5d(xv_smem + c * 16384, &tm_xv, &bars->x_full, c * 64, tp.x0, tp.r0, hi, bi);
    }
    __syncwarp();
    for (int j = 0; j < tp.nblk; ++j) {
      const int s = j % pl.stages;
      if (j >= pl.stages) wait_park(&bars->y_empty[s], ((j / pl.stages) - 1) & 1);
      if (!ok) break;
      if (elect_one()) {
        mbar_arrive_expect_tx(&bars->y_full[s], yqk_stage + yv_stage);
        const int row = tp.hr_first + j * pl.KR;
        for (int c = 0; c < p.qch; ++c)
          tma_load_5d(yqk_smem + s * yqk_stage + c * blk_bytes, &tm_yqk, &bars->y_full[s], c * 64, tp.hx0, row, hi, bi);
        for (int c = 0; c < p.vch; ++c)
          tma_load_5d(yv_smem + s * yv_stage + c * blk_bytes, &tm_yv, &bars->y_full[s], c * 64, tp.hx0, row, hi, bi);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (whole warp, one lane issues)
    const uint32_t fmt = BF16 ? 1u : 0u;
    const uint32_t idesc_s = instr_desc(fmt, 128, N, 0, 0);
    const uint32_t idesc_aqk = instr_desc(fmt, 128, p.qch * 64, 0, 1);
    const uint32_t idesc_av = instr_desc(fmt, 128, p.vch * 64, 0, 1);
    const uint32_t xqk = smem_u32(xqk_smem), xv = smem_u32(xv_smem), yqk = smem_u32(yqk_smem), yv = smem_u32(yv_smem),
                   ops = smem_u32(op_smem), xx = smem_u32(xx_smem), yx = smem_u32(yx_smem);
    const uint32_t hi_sw = smem_desc_hi(1024, true), hi_ns = smem_desc_hi(kXSbo, false);
    wait_spin(&bars->x_ready, 0);
    auto issue_acc = [&](int i) {
      const int pb = i % pl.pbufs, s = i % pl.stages;
      wait_spin(&bars->op_full[pb], (i / pl.pbufs) & 1);
      if (!ok) return;
      tc_fence_after();
      const uint32_t ds_addr = ops + (pb * kOps) * pch * 16384, yqk_s = yqk + s * yqk_stage, yv_s = yv + s * yv_stage;
      if (elect_one()) {
        for (int ks = 0; ks < (N >> 4); ++ks)
          umma_ss(tmem + kTmAccQK, smem_desc_from(ds_addr + (ks >> 2) * 16384 + (ks & 3) * 32, 16, hi_sw),
                  smem_desc_from(yqk_s + ks * 2048, blk_bytes, hi_sw), idesc_aqk, (i > 0 || ks > 0) ? 1u : 0u);
        if constexpr (DKDV) {
          for (int ks = 0; ks < (N >> 4); ++ks)
            umma_ss(tmem + kTmAccV, smem_desc_from(ds_addr + (pch + (ks >> 2)) * 16384 + (ks & 3) * 32, 16, hi_sw),
                    smem_desc_from(yv_s + ks * 2048, blk_bytes, hi_sw), idesc_av, (i > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&bars->y_empty[s]);
        umma_commit(&bars->op_empty[pb]);
        if (i == tp.nblk - 1) umma_commit(&bars->acc_done);
        trace_mark(p, 1, 2 * i + 1);
      }
      __syncwarp();
    };
    for (int j = 0; ok && j < tp.nblk; ++j) {
      const int s = j % pl.stages, sb = j % nsb;
      wait_spin(&bars->y_ready[s], (j / pl.stages) & 1);
      if (j >= nsb) wait_spin(&bars->sd_empty[sb], ((j / nsb) - 1) & 1);
      if (!ok) break;
      tc_fence_after();
      const uint32_t yqk_s = yqk + s * yqk_stage, yv_s = yv + s * yv_stage, yx_s = yx + s * yx_stage;
      if (elect_one()) {
        for (int c = 0; c < p.qch; ++c) {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_ss(tmem + kTmS + sb * 64, smem_desc_from(xqk + c * 16384 + k * 32, 16, hi_sw),
                    smem_desc_from(yqk_s + c * blk_bytes + k * 32, 16, hi_sw), idesc_s, (c | k) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < 2; ++k)  // + indicator x penalty: the window mask
          umma_ss(tmem + kTmS + sb * 64, smem_desc_from(xx + k * kXStepBytes, kXLbo, hi_ns),
                  smem_desc_from(yx_s + k * kXStepBytes, kXLbo, hi_ns), idesc_s, 1u);
        for (int c = 0; c < p.vch; ++c) {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_ss(tmem + kTmDP + sb * 64, smem_desc_from(xv + c * 16384 + k * 32, 16, hi_sw),
                    smem_desc_from(yv_s + c * blk_bytes + k * 32, 16, hi_sw), idesc_s, (c | k) ? 1u : 0u);
        }
        umma_commit(&bars->sd_full[sb]);
        trace_mark(p, 1, 2 * j);
      }
      __syncwarp();
      if (j >= 1) issue_acc(j - 1);
    }
    if (ok) issue_acc(tp.nblk - 1);
  } else if (warp < 10) {
    // ------------------------------------------------------------------ P / dS, two threads per resident token
    const int quarter = warp & 3;                 // TMEM lane quarter this warp may touch
    const int half = (warp - 2) >> 2;             // lower / upper half of each block's columns
    const int m = quarter * 32 + lane;
    const int tr = tp.r0 + m / pl.TW, tx = tp.x0 + m % pl.TW;
    const bool t_in = tr < p.t_h && tx < p.Wtok;
    const int64_t tok = (int64_t)tr * p.Wtok + tx;
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    const float c2 = p.scale_log2;
    const int nh = N >> 1;                        // columns per thread, a multiple of 8, <= 64
    const int col0 = half * nh;
    const int sw = m & 7;
    float my_lse = INFINITY, my_delta = 0.f;
    if (!DKDV && t_in) {
      my_lse = lse[vec_base + tok];
      my_delta = delta[vec_base + tok];
    }
    const uint32_t op_base = smem_u32(op_smem) + m * 128;
    const uint32_t vec_addr = smem_u32(vec_smem);
    // Prologue: these warps have nothing to do until the first S / dP tiles exist, so they rotate the
    // resident q/k tile (thread (m, half) takes the row-angle or the column-angle pairs of row m) while
    // the RoPE warps already work on the first streamed blocks.
    {
      const bool rope_on = p.rope.idx != nullptr;
      RopeParts xp;
      xp.row = m; xp.lo = xp.hi = half; xp.active = true;
      RopeRow rc;
      rc.pos[0] = rc.pos[1] = -1;
      if (rope_on && t_in) rope_fetch(rc, __ldg(p.rope.idx + tok), xp, p.rope);
      wait_spin(&bars->x_full, 0);
      if (ok) {
        if (rope_on && t_in) rope_apply<BF16>(xqk_smem, 16384, rc, xp, p.rope);
        fence_proxy_async_smem();
        mbar_arrive(&bars->x_ready);
      }
    }
    for (int j = 0; j < tp.nblk && ok; ++j) {
      const int sb = j % nsb, pb = j % pl.pbufs, s = j % pl.stages;
      wait_spin(&bars->sd_full[sb], (j / nsb) & 1);
      if (DKDV) wait_spin(&bars->y_ready[s], (j / pl.stages) & 1);   // lse/delta of the block are staged
      if (j >= pl.pbufs) wait_spin(&bars->op_empty[pb], ((j / pl.pbufs) - 1) & 1);
      if (!ok) break;
      tc_fence_after();
      if (m == 0 && half == 0) trace_mark(p, 2, 2 * j);
      const uint32_t ds_row = op_base + (pb * kOps) * pch * 16384;
      const uint32_t lse_s = vec_addr + (s * 256) * 4, dl_s = lse_s + 128 * 4;
      // columns [col0 + off, col0 + off + CNT) of the block
      auto process = [&](int off, auto cnt_tag) {
        constexpr int CNT = decltype(cnt_tag)::value;
        uint32_t sr[CNT], dr[CNT];
        if constexpr (CNT == 16) {
          tmem_ld16(lane_base + kTmS + sb * 64 + col0 + off, sr);
          tmem_ld16(lane_base + kTmDP + sb * 64 + col0 + off, dr);
        } else {
          tmem_ld8(lane_base + kTmS + sb * 64 + col0 + off, sr);
          tmem_ld8(lane_base + kTmDP + sb * 64 + col0 + off, dr);
        }
        float lq[CNT], dq_[CNT];
        if constexpr (DKDV) {
#pragma unroll
          for (int e = 0; e < CNT; e += 4) {
            const uint4 a = lds128(lse_s + (col0 + off + e) * 4), b = lds128(dl_s + (col0 + off + e) * 4);
            lq[e] = __uint_as_float(a.x); lq[e + 1] = __uint_as_float(a.y);
            lq[e + 2] = __uint_as_float(a.z); lq[e + 3] = __uint_as_float(a.w);
            dq_[e] = __uint_as_float(b.x); dq_[e + 1] = __uint_as_float(b.y);
            dq_[e + 2] = __uint_as_float(b.z); dq_[e + 3] = __uint_as_float(b.w);
          }
        }
        tmem_wait_ld();
#pragma unroll
        for (int u = 0; u < CNT / 8; ++u) {
          uint32_t wds[4], wp[4];
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            float pv[2], dsv[2];
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              const int e = u * 8 + 2 * h + t;
              const float l_ = DKDV ? lq[e] : my_lse;
              const float d_ = DKDV ? dq_[e] : my_delta;
              // pairs outside the window carry a large negative score from the MMA: exp2 gives exactly 0
              const float pe = exp2f(fmaf(__uint_as_float(sr[e]), c2, -l_));
              pv[t] = pe;
              dsv[t] = pe * (__uint_as_float(dr[e]) - d_);
            }
            wds[h] = pack2<BF16>(dsv[0], dsv[1]);
            wp[h] = pack2<BF16>(pv[0], pv[1]);
          }
          const int unit = ((col0 + off) >> 3) + u;
          const uint32_t a = ds_row + (unit >> 3) * 16384 + (((unit & 7) ^ sw) << 4);
          sts128(a, wds[0], wds[1], wds[2], wds[3]);
          if constexpr (DKDV) sts128(a + pch * 16384, wp[0], wp[1], wp[2], wp[3]);
        }
      };
      for (int off = 0; off + 16 <= nh; off += 16) process(off, std::integral_constant<int, 16>{});
      if (nh & 8) process(nh - 8, std::integral_constant<int, 8>{});
      tc_fence_before();
      mbar_arrive(&bars->sd_empty[sb]);
      fence_proxy_async_smem();
      mbar_arrive(&bars->op_full[pb]);
      if (m == 0 && half == 0) trace_mark(p, 2, 2 * j + 1);
    }
    // epilogue: the two threads of a row each store half of the accumulator row(s): with one 64-column chunk
    // each takes 32 columns, with two chunks each takes one chunk.  The cos/sin pairs for rotating dQ / dK
    // back are fetched before the final wait.
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    const bool rot = p.rope.idx != nullptr && t_in;
    int irow = -1, icol = -1;
    if (rot) decode_idx(__ldg(p.rope.idx + tok), p.rope.max_h, p.rope.max_w, irow, icol);
    EpiRope<32> c32;
    EpiRope<64> c64;
    if (p.qch == 1) {
      if (half == 0) epi_fetch<0, 32>(c32, rot, irow, icol, p.rope); else epi_fetch<32, 32>(c32, rot, irow, icol, p.rope);
    } else {
      if (half == 0) epi_fetch<0, 64>(c64, rot, irow, icol, p.rope); else epi_fetch<64, 64>(c64, rot, irow, icol, p.rope);
    }
    wait_spin(&bars->acc_done, 0);
    if (ok) {
      tc_fence_after();
      if (m == 0 && half == 0) trace_mark(p, 2, 30);
      T* qk_row = (T*)out_qk.ptr + bi * out_qk.s0 + hi * out_qk.s1 + tok * out_qk.s2;
      const uint32_t aqk = lane_base + kTmAccQK;
      if (p.qch == 1) {
        if (half == 0) store_acc_piece<BF16, 0, 32>(aqk, p.sm_scale, rot, c32, p.rope.R, qk_row, t_in);
        else store_acc_piece<BF16, 32, 32>(aqk, p.sm_scale, rot, c32, p.rope.R, qk_row, t_in);
      } else {
        if (half == 0) store_acc_piece<BF16, 0, 64>(aqk, p.sm_scale, rot, c64, p.rope.R, qk_row, t_in);
        else store_acc_piece<BF16, 64, 64>(aqk, p.sm_scale, rot, c64, p.rope.R, qk_row, t_in);
      }
      if constexpr (DKDV) {
        T* v_row = (T*)out_v.ptr + bi * out_v.s0 + hi * out_v.s1 + tok * out_v.s2;
        const uint32_t av = lane_base + kTmAccV;
        if (p.vch == 1) {
          if (half == 0) store_acc_piece<BF16, 0, 32>(av, 1.f, false, c32, 0, v_row, t_in);
          else store_acc_piece<BF16, 32, 32>(av, 1.f, false, c32, 0, v_row, t_in);
        } else {
          if (half == 0) store_acc_piece<BF16, 0, 64>(av, 1.f, false, c64, 0, v_row, t_in);
          else store_acc_piece<BF16, 64, 64>(av, 1.f, false, c64, 0, v_row, t_in);
        }
      }
      tc_fence_before();
      if (m == 0 && half == 0) trace_mark(p, 2, 31);
    }
  } else {
    // ------------------------------------------------------------------ RoPE on the q/k tiles, mask tiles, lse/delta staging
    const int t = threadIdx.x - kBwdRopeThread0;
    const bool rope_on = p.rope.idx != nullptr;
    const RopeParts ip = rope_parts(t, 128), yp = rope_parts(t, N);   // share of the indicator tile / of a streamed block
    const int yjr = yp.row / pl.KW, yx_ = tp.hx0 + yp.row % pl.KW;    // this thread's row inside every streamed block
    const bool yx_in = yp.active && yx_ >= 0 && yx_ < p.Wtok;
    int32_t y_idx = -1;
    RopeRow rc;
    rc.pos[0] = rc.pos[1] = -1;
    if (rope_on) {
      const int yr0 = tp.hr_first + yjr;
      if (yx_in && yr0 < p.t_h) y_idx = __ldg(p.rope.idx + yr0 * p.Wtok + yx_);
    }
    write_indicator_row<BF16>(xx_smem, ip.row, ip.lo, ip.hi, p);
    build_penalty_tables<BF16>(&bars->pen, t, p, tp);
    named_bar_sync(5, 128);                          // the tables are complete before any of these warps reads them
    {
      rope_fetch(rc, y_idx, yp, p.rope);             // cos/sin of this thread's row of block 0
      for (int j = 0; j < tp.nblk; ++j) {
        const int s = j % pl.stages;
        const int yr = tp.hr_first + j * pl.KR + yjr;
        const bool in = yx_in && yr < p.t_h;
        int32_t y_idx_next = -1;
        if (rope_on && yx_in && j + 1 < tp.nblk && yr + pl.KR < p.t_h) y_idx_next = __ldg(p.rope.idx + (yr + pl.KR) * p.Wtok + yx_);
        // lse and delta of the block's queries: thread t stages both values of block row t
        float lse_v = INFINITY, delta_v = 0.f;
        if constexpr (DKDV) {
          if (t < N) {
            const int vr = tp.hr_first + j * pl.KR + t / pl.KW, vx = tp.hx0 + t % pl.KW;
            if (vr < p.t_h && vx >= 0 && vx < p.Wtok) {
              lse_v = __ldg(lse + vec_base + (int64_t)vr * p.Wtok + vx);
              delta_v = __ldg(delta + vec_base + (int64_t)vr * p.Wtok + vx);
            }
          }
        }
        // the stage (tiles, penalty rows, lse/delta slots) is free once its refill has landed: the
        // producer refills only after every MMA of the stage's previous block has completed, which in
        // turn is after the compute warps finished reading that block's lse/delta
        wait_park(&bars->y_full[s], (j / pl.stages) & 1);
        if (!ok) break;
        if (t == 0) trace_mark(p, 3, 2 * j);
        if (yp.active) {
          write_penalty_row(yx_smem + s * yx_stage, yp.row, yp.lo, yp.hi, &bars->pen, j * pl.KR + yjr, yp.row % pl.KW, pl.TH >> 3, pl.TW >> 3);
          if (rope_on && in) rope_apply<BF16>(yqk_smem + s * yqk_stage, blk_bytes, rc, yp, p.rope);
        }
        if constexpr (DKDV) {
          if (t < N) {
            vec_smem[s * 256 + t] = lse_v;
            vec_smem[s * 256 + 128 + t] = delta_v;
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(&bars->y_ready[s]);
        if (t == 0) trace_mark(p, 3, 2 * j + 1);
        rope_fetch(rc, y_idx_next, yp, p.rope);    // lands while this thread waits for the next block
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    if (threadIdx.x == 0) report_abort(p.status, DKDV ? 3 : 2, 0);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kBwdTmemCols);
  }
}

}  // namespace tc
}  // namespace swa
