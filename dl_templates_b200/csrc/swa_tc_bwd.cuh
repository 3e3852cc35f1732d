// tcgen05 backward kernels.  One template serves both launches:
//
//   DKDV = false  (dQ kernel)    resident tile X = (Q, dO) of 128 queries,
//                                streamed blocks Y = (K, V) of the halo keys
//   DKDV = true   (dK/dV kernel) resident tile X = (K, V) of 128 keys,
//                                streamed blocks Y = (Q, dO) of the halo queries
//
// Per streamed block (N <= 64 tokens), with T = the resident token (one TMEM lane):
//   S  = Xqk Yqk^T          (scores, transposed in the dK/dV kernel)
//   dP = Xv  Yv^T
//   P  = exp2(scale*log2e * S - lse[query])  under the window mask
//   dS = P * (dP - delta[query])
//   acc_qk += dS Yqk        (dQ resp. dK, before the sm_scale factor)
//   acc_v  += P  Yv         (dV; dK/dV kernel only)
// lse/delta belong to the query: the row's own scalar in the dQ kernel, one value per
// streamed column (staged in shared memory) in the dK/dV kernel.  P is recomputed
// from the saved logsumexp, nothing is accumulated with atomics, and RoPE-2D is
// fused: q/k tiles are rotated in shared memory before the MMAs and the dQ / dK rows
// are rotated back in registers before they are stored.
//
// Warp roles (320 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner,
// warps 2-5 one thread per resident token (P/dS computation, epilogue), warps 6-9
// RoPE rotation of the tiles and staging of lse/delta.  S and dP are double-buffered
// in TMEM so the tensor core works on block j+1 while the compute warps work on j.
// TMEM columns: S[2] at 0/64, dP[2] at 128/192, acc_qk at 256, acc_v at 384.
#pragma once

#include "swa_tc_common.cuh"

namespace swa {
namespace tc {

struct BwdBars {
  uint64_t x_full, x_ready, acc_done;
  uint64_t y_full[kMaxStages], y_ready[kMaxStages], y_empty[kMaxStages];
  uint64_t sd_full[2], sd_empty[2], op_full[2], op_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

constexpr int kBwdThreads = 320;
constexpr uint32_t kBwdTmemCols = 512;
constexpr uint32_t kTmS = 0, kTmDP = 128, kTmAccQK = 256, kTmAccV = 384;

// Rotate back (transpose rotation) the 64 dims [CH*64, CH*64+64) of a dQ/dK row held in registers.
template <int R, int CH>
__device__ __forceinline__ void inv_rotate64(float (&v)[64], int irow, int icol, const RopeDev& rp) {
#pragma unroll
  for (int e = 0; e < 64; ++e) {
    const int d = CH * 64 + e;
    if (d < 4 * R && ((d / R) & 1) == 0) {
      const int seg = d / R;
      const int pos = seg >= 2 ? icol : irow;
      if (pos >= 0) {
        const float2 cs =
            __ldg(reinterpret_cast<const float2*>((seg >= 2 ? rp.col_cs : rp.row_cs) + ((int64_t)pos * R + (d - seg * R)) * 2));
        const float x0 = v[e], x1 = v[(e + R) & 63];
        v[e] = x0 * cs.x + x1 * cs.y;
        v[(e + R) & 63] = x1 * cs.x - x0 * cs.y;
      }
    }
  }
}

template <int CH>
__device__ __forceinline__ void inv_rotate64_any(float (&v)[64], int irow, int icol, const RopeDev& rp) {
  switch (rp.R) {
    case 8: inv_rotate64<8, CH>(v, irow, icol, rp); break;
    case 16: inv_rotate64<16, CH>(v, irow, icol, rp); break;
    case 32: inv_rotate64<32, CH>(v, irow, icol, rp); break;
    default: break;
  }
}

// Load 64 accumulator columns of this thread's TMEM lane, scale, optionally rotate back, store 128 bytes.
template <bool BF16, int CH>
__device__ __forceinline__ void store_acc_chunk(uint32_t taddr, float scale, bool rot, int irow, int icol,
                                                const RopeDev& rp, void* dst_row, bool in_grid) {
  using namespace ptx;
  uint32_t raw[64];
#pragma unroll
  for (int c = 0; c < 4; ++c) tmem_ld16(taddr + CH * 64 + c * 16, &raw[c * 16]);
  tmem_wait_ld();
  float v[64];
#pragma unroll
  for (int e = 0; e < 64; ++e) v[e] = __uint_as_float(raw[e]) * scale;
  if (rot) inv_rotate64_any<CH>(v, irow, icol, rp);
  if (in_grid) {
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(dst_row) + CH * 128);
#pragma unroll
    for (int u = 0; u < 8; ++u)
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
  uint8_t* xqk_smem = smem;
  uint8_t* xv_smem = xqk_smem + p.qch * 16384;
  uint8_t* yqk_smem = xv_smem + p.vch * 16384;
  uint8_t* yv_smem = yqk_smem + pl.stages * yqk_stage;
  uint8_t* op_smem = yv_smem + pl.stages * yv_stage;       // [pbufs][kOps][128 x 64] : dS then P
  float* vec_smem = reinterpret_cast<float*>(op_smem + pl.pbufs * kOps * 16384);  // [stages][2][64]: lse, delta
  BwdBars* bars = reinterpret_cast<BwdBars*>(reinterpret_cast<uint8_t*>(vec_smem) + kMaxStages * 2 * 64 * 4);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y, bi = bh / p.H, hi = bh - bi * p.H;
  const TilePos tp = tile_pos(p, blockIdx.x);
  const int64_t vec_base = (int64_t)bh * p.t_h * p.Wtok;

  if (threadIdx.x == 0) {
    mbar_init(&bars->x_full, 1);
    mbar_init(&bars->x_ready, 128);
    mbar_init(&bars->acc_done, 1);
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(&bars->y_full[s], 1);
      mbar_init(&bars->y_ready[s], 128);
      mbar_init(&bars->y_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->sd_full[s], 1);
      mbar_init(&bars->sd_empty[s], 128);
      mbar_init(&bars->op_full[s], 128);
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

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&tm_xqk);
      prefetch_tmap(&tm_xv);
      prefetch_tmap(&tm_yqk);
      prefetch_tmap(&tm_yv);
      mbar_arrive_expect_tx(&bars->x_full, (p.qch + p.vch) * 16384);
      for (int c = 0; c < p.qch; ++c) tma_load_5d(xqk_smem + c * 16384, &tm_xqk, &bars->x_full, c * 64, tp.x0, tp.r0, hi, bi);
      for (int c = 0; c < p.vch; ++c) tma_load_5d(xv_smem + c * 16384, &tm_xv, &bars->x_full, c * 64, tp.x0, tp.r0, hi, bi);
      for (int j = 0; j < tp.nblk; ++j) {
        const int s = j % pl.stages;
        if (j >= pl.stages && !mbar_wait(&bars->y_empty[s], ((j / pl.stages) - 1) & 1, abort_flag)) break;
        mbar_arrive_expect_tx(&bars->y_full[s], yqk_stage + yv_stage);
        const int row = tp.hr_first + j * pl.KR;
        for (int c = 0; c < p.qch; ++c)
          tma_load_5d(yqk_smem + s * yqk_stage + c * blk_bytes, &tm_yqk, &bars->y_full[s], c * 64, tp.hx0, row, hi, bi);
        for (int c = 0; c < p.vch; ++c)
          tma_load_5d(yv_smem + s * yv_stage + c * blk_bytes, &tm_yv, &bars->y_full[s], c * 64, tp.hx0, row, hi, bi);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t fmt = BF16 ? 1u : 0u;
      const uint32_t idesc_s = instr_desc(fmt, 128, N, 0, 0);
      const uint32_t idesc_aqk = instr_desc(fmt, 128, p.qch * 64, 0, 1);
      const uint32_t idesc_av = instr_desc(fmt, 128, p.vch * 64, 0, 1);
      const uint32_t xqk = smem_u32(xqk_smem), xv = smem_u32(xv_smem), yqk = smem_u32(yqk_smem), yv = smem_u32(yv_smem),
                     ops = smem_u32(op_smem);
      bool ok = mbar_wait(&bars->x_ready, 0, abort_flag);
      auto issue_acc = [&](int i) -> bool {
        const int pb = i % pl.pbufs, s = i % pl.stages;
        if (!mbar_wait(&bars->op_full[pb], (i / pl.pbufs) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t ds_addr = ops + (pb * kOps) * 16384;
        for (int ks = 0; ks < (N >> 4); ++ks) {
          const uint64_t a = smem_desc(ds_addr + ks * 32, 16, 1024);
          const uint64_t b = smem_desc(yqk + s * yqk_stage + ks * 2048, blk_bytes, 1024);
          umma_ss(tmem + kTmAccQK, a, b, idesc_aqk, (i > 0 || ks > 0) ? 1u : 0u);
        }
        if constexpr (DKDV) {
          for (int ks = 0; ks < (N >> 4); ++ks) {
            const uint64_t a = smem_desc(ds_addr + 16384 + ks * 32, 16, 1024);
            const uint64_t b = smem_desc(yv + s * yv_stage + ks * 2048, blk_bytes, 1024);
            umma_ss(tmem + kTmAccV, a, b, idesc_av, (i > 0 || ks > 0) ? 1u : 0u);
          }
        }
        umma_commit(&bars->y_empty[s]);
        umma_commit(&bars->op_empty[pb]);
        return true;
      };
      for (int j = 0; ok && j < tp.nblk; ++j) {
        const int s = j % pl.stages, sb = j & 1;
        if (!mbar_wait(&bars->y_ready[s], (j / pl.stages) & 1, abort_flag)) { ok = false; break; }
        if (j >= 2 && !mbar_wait(&bars->sd_empty[sb], ((j >> 1) - 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        for (int c = 0; c < p.qch; ++c)
          for (int k = 0; k < 4; ++k)
            umma_ss(tmem + kTmS + sb * 64, smem_desc(xqk + c * 16384 + k * 32, 16, 1024),
                    smem_desc(yqk + s * yqk_stage + c * blk_bytes + k * 32, 16, 1024), idesc_s, (c | k) ? 1u : 0u);
        for (int c = 0; c < p.vch; ++c)
          for (int k = 0; k < 4; ++k)
            umma_ss(tmem + kTmDP + sb * 64, smem_desc(xv + c * 16384 + k * 32, 16, 1024),
                    smem_desc(yv + s * yv_stage + c * blk_bytes + k * 32, 16, 1024), idesc_s, (c | k) ? 1u : 0u);
        umma_commit(&bars->sd_full[sb]);
        if (j >= 1 && !issue_acc(j - 1)) { ok = false; break; }
      }
      if (ok && issue_acc(tp.nblk - 1)) umma_commit(&bars->acc_done);
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ P / dS, one thread per resident token
    const int quarter = warp & 3;
    const int m = quarter * 32 + lane;
    const int tr = tp.r0 + m / pl.TW, tx = tp.x0 + m % pl.TW;
    const bool t_in = tr < p.t_h && tx < p.Wtok;
    const int64_t tok = (int64_t)tr * p.Wtok + tx;
    const uint64_t colmask = column_mask(p, tp.hx0, tx, t_in);
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    const float c2 = p.scale_log2;
    float my_lse = INFINITY, my_delta = 0.f;
    if (!DKDV && t_in) {
      my_lse = lse[vec_base + tok];
      my_delta = delta[vec_base + tok];
    }
    bool ok = true;
    for (int j = 0; j < tp.nblk; ++j) {
      const int sb = j & 1, pb = j % pl.pbufs, s = j % pl.stages;
      if (!mbar_wait(&bars->sd_full[sb], (j >> 1) & 1, abort_flag)) { ok = false; break; }
      if (DKDV && !mbar_wait(&bars->y_ready[s], (j / pl.stages) & 1, abort_flag)) { ok = false; break; }  // lse/delta staged
      tc_fence_after();
      uint32_t vm[4];
      block_mask(vm, p, colmask, tp.hr_first + j * pl.KR, tr, tp.hr_last);
      if (j >= pl.pbufs && !mbar_wait(&bars->op_empty[pb], ((j / pl.pbufs) - 1) & 1, abort_flag)) { ok = false; break; }
      uint8_t* ds_tile = op_smem + (pb * kOps) * 16384;
      const float* lse_s = vec_smem + s * 128;
      const float* dl_s = lse_s + 64;
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (c * 16 < N) {
          uint32_t sr[16], dr[16];
          tmem_ld16(lane_base + kTmS + sb * 64 + c * 16, sr);
          tmem_ld16(lane_base + kTmDP + sb * 64 + c * 16, dr);
          tmem_wait_ld();
          uint32_t wds[8], wp[8];
#pragma unroll
          for (int h = 0; h < 8; ++h) {
            float pv[2], dsv[2];
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              const int e = c * 16 + 2 * h + t;
              const bool valid = (vm[e >> 5] >> (e & 31)) & 1u;
              const float l_ = DKDV ? lse_s[e] : my_lse;
              const float d_ = DKDV ? dl_s[e] : my_delta;
              const float pe = valid ? exp2f(fmaf(__uint_as_float(sr[2 * h + t]), c2, -l_)) : 0.f;
              pv[t] = pe;
              dsv[t] = pe * (__uint_as_float(dr[2 * h + t]) - d_);
            }
            wds[h] = pack2<BF16>(dsv[0], dsv[1]);
            wp[h] = pack2<BF16>(pv[0], pv[1]);
          }
          *reinterpret_cast<uint4*>(swz(ds_tile, m, 2 * c)) = make_uint4(wds[0], wds[1], wds[2], wds[3]);
          *reinterpret_cast<uint4*>(swz(ds_tile, m, 2 * c + 1)) = make_uint4(wds[4], wds[5], wds[6], wds[7]);
          if constexpr (DKDV) {
            *reinterpret_cast<uint4*>(swz(ds_tile + 16384, m, 2 * c)) = make_uint4(wp[0], wp[1], wp[2], wp[3]);
            *reinterpret_cast<uint4*>(swz(ds_tile + 16384, m, 2 * c + 1)) = make_uint4(wp[4], wp[5], wp[6], wp[7]);
          }
        }
      tc_fence_before();
      mbar_arrive(&bars->sd_empty[sb]);
      fence_proxy_async_smem();
      mbar_arrive(&bars->op_full[pb]);
    }
    // epilogue
    if (ok && mbar_wait(&bars->acc_done, 0, abort_flag)) {
      tc_fence_after();
      using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
      const bool rot = p.rope.idx != nullptr;
      int irow = -1, icol = -1;
      if (rot && t_in) decode_idx(p.rope.idx[tok], p.rope.max_h, p.rope.max_w, irow, icol);
      T* qk_row = (T*)out_qk.ptr + bi * out_qk.s0 + hi * out_qk.s1 + tok * out_qk.s2;
      store_acc_chunk<BF16, 0>(lane_base + kTmAccQK, p.sm_scale, rot && t_in, irow, icol, p.rope, qk_row, t_in);
      if (p.qch > 1) store_acc_chunk<BF16, 1>(lane_base + kTmAccQK, p.sm_scale, rot && t_in, irow, icol, p.rope, qk_row, t_in);
      if constexpr (DKDV) {
        T* v_row = (T*)out_v.ptr + bi * out_v.s0 + hi * out_v.s1 + tok * out_v.s2;
        store_acc_chunk<BF16, 0>(lane_base + kTmAccV, 1.f, false, -1, -1, p.rope, v_row, t_in);
        if (p.vch > 1) store_acc_chunk<BF16, 1>(lane_base + kTmAccV, 1.f, false, -1, -1, p.rope, v_row, t_in);
      }
      tc_fence_before();
    }
  } else {
    // ------------------------------------------------------------------ RoPE on the q/k tiles, lse/delta staging
    const int t = threadIdx.x - 192;
    const bool rope_on = p.rope.idx != nullptr;
    if (mbar_wait(&bars->x_full, 0, abort_flag)) {
      if (rope_on) {
        const int r = tp.r0 + t / pl.TW, x = tp.x0 + t % pl.TW;
        if (r < p.t_h && x < p.Wtok) rotate_row_smem<BF16>(xqk_smem, 16384, t, r * p.Wtok + x, p.rope);
        fence_proxy_async_smem();
      }
      mbar_arrive(&bars->x_ready);
      for (int j = 0; j < tp.nblk; ++j) {
        const int s = j % pl.stages;
        // the stage's lse/delta slots are free once the previous user of the stage has been consumed,
        // which the producer already waited for before refilling it; wait for the refill itself
        if (!mbar_wait(&bars->y_full[s], (j / pl.stages) & 1, abort_flag)) break;
        if (t < N) {
          const int r = tp.hr_first + j * pl.KR + t / pl.KW, x = tp.hx0 + t % pl.KW;
          const bool in = r < p.t_h && x >= 0 && x < p.Wtok;
          if (rope_on && in) rotate_row_smem<BF16>(yqk_smem + s * yqk_stage, blk_bytes, t, r * p.Wtok + x, p.rope);
          if constexpr (DKDV) {
            vec_smem[s * 128 + t] = in ? lse[vec_base + (int64_t)r * p.Wtok + x] : INFINITY;
            vec_smem[s * 128 + 64 + t] = in ? delta[vec_base + (int64_t)r * p.Wtok + x] : 0.f;
          }
        }
        if (rope_on) fence_proxy_async_smem();
        mbar_arrive(&bars->y_ready[s]);
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
