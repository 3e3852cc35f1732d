// tcgen05 forward kernel: o = softmax(scale * rope(q) rope(k)^T + window mask) v, lse.
//
// One CTA per 128-query tile (TH rows x TW token columns) of one (batch, head).
// Warp roles (320 threads):
//   warp 0      TMA producer: the query tile once, then the K and V halo blocks
//               through a `stages`-deep ring of shared-memory buffers
//   warp 1      MMA issuer (one thread): S = Q K^T into one of two TMEM buffers,
//               O += P V into a third; owns the TMEM allocation
//   warps 2-5   softmax, one thread per query row (TMEM lane): tcgen05.ld of the S
//               row, window mask, running max / sum, P written to shared memory as the
//               A operand of the PV MMA, lazy rescale of O, final normalisation
//   warps 6-9   fused RoPE-2D: rotate the Q tile and every K block in shared memory
//               between TMA arrival and MMA issue (pass-through when RoPE is off)
// S for block j+1 is computed by the tensor core while the softmax warps work on
// block j.  All waits are bounded; a timed-out wait raises a CTA-wide abort flag,
// every role leaves its loop, TMEM is freed and the status word records the event.
#pragma once

#include "swa_tc_common.cuh"

namespace swa {
namespace tc {

struct FwdBars {
  uint64_t q_full, q_ready, o_done;
  uint64_t kv_full[kMaxStages], k_ready[kMaxStages], kv_empty[kMaxStages];
  uint64_t s_full[2], s_empty[2], p_full[2], p_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

constexpr int kFwdThreads = 320;
constexpr uint32_t kFwdTmemCols = 512;
constexpr uint32_t kTmemS = 0, kTmemO = 256;   // column offsets: S0 at 0, S1 at 128, O at 256
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
  const uint32_t k_stage = blk_bytes * p.qch, v_stage = blk_bytes * p.vch;
  const int pch = (N + 63) >> 6;                                 // 64-key chunks of P
  uint8_t* q_smem = smem;
  uint8_t* k_smem = q_smem + p.qch * 16384;
  uint8_t* v_smem = k_smem + pl.stages * k_stage;
  uint8_t* p_smem = v_smem + pl.stages * v_stage;
  FwdBars* bars = reinterpret_cast<FwdBars*>(p_smem + pl.pbufs * pch * 16384);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y, bi = bh / p.H, hi = bh - bi * p.H;
  const TilePos tp = tile_pos(p, blockIdx.x);

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    mbar_init(&bars->q_ready, 128);
    mbar_init(&bars->o_done, 1);
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->k_ready[s], 128);
      mbar_init(&bars->kv_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->s_full[s], 1);
      mbar_init(&bars->s_empty[s], 128);
      mbar_init(&bars->p_full[s], 128);
      mbar_init(&bars->p_empty[s], 1);
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

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      mbar_arrive_expect_tx(&bars->q_full, p.qch * 16384);
      for (int c = 0; c < p.qch; ++c) tma_load_5d(q_smem + c * 16384, &tm_q, &bars->q_full, c * 64, tp.x0, tp.r0, hi, bi);
      for (int j = 0; j < tp.nblk; ++j) {
        const int s = j % pl.stages;
        if (j >= pl.stages && !mbar_wait(&bars->kv_empty[s], ((j / pl.stages) - 1) & 1, abort_flag)) break;
        mbar_arrive_expect_tx(&bars->kv_full[s], k_stage + v_stage);
        const int row = tp.hr_first + j * pl.KR;
        for (int c = 0; c < p.qch; ++c)
          tma_load_5d(k_smem + s * k_stage + c * blk_bytes, &tm_k, &bars->kv_full[s], c * 64, tp.hx0, row, hi, bi);
        for (int c = 0; c < p.vch; ++c)
          tma_load_5d(v_smem + s * v_stage + c * blk_bytes, &tm_v, &bars->kv_full[s], c * 64, tp.hx0, row, hi, bi);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t fmt = BF16 ? 1u : 0u;
      const uint32_t idesc_s = instr_desc(fmt, 128, N, 0, 0);
      const uint32_t idesc_pv = instr_desc(fmt, 128, p.vch * 64, 0, 1);
      const uint32_t q_addr = smem_u32(q_smem), k_addr = smem_u32(k_smem), v_addr = smem_u32(v_smem),
                     p_addr = smem_u32(p_smem);
      bool ok = mbar_wait(&bars->q_ready, 0, abort_flag);
      auto issue_pv = [&](int i) -> bool {
        const int pb = i % pl.pbufs, s = i % pl.stages;
        if (!mbar_wait(&bars->p_full[pb], (i / pl.pbufs) & 1, abort_flag)) return false;
        tc_fence_after();
        for (int ks = 0; ks < (N >> 4); ++ks) {
          const uint64_t a = smem_desc(p_addr + pb * pch * 16384 + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024);
          const uint64_t b = smem_desc(v_addr + s * v_stage + ks * 2048, blk_bytes, 1024);
          umma_ss(tmem + kTmemO, a, b, idesc_pv, (i > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&bars->kv_empty[s]);
        umma_commit(&bars->p_empty[pb]);
        return true;
      };
      for (int j = 0; ok && j < tp.nblk; ++j) {
        const int s = j % pl.stages, sb = j & 1;
        if (!mbar_wait(&bars->k_ready[s], (j / pl.stages) & 1, abort_flag)) { ok = false; break; }
        if (j >= 2 && !mbar_wait(&bars->s_empty[sb], ((j >> 1) - 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        for (int c = 0; c < p.qch; ++c)
          for (int k = 0; k < 4; ++k) {
            const uint64_t a = smem_desc(q_addr + c * 16384 + k * 32, 16, 1024);
            const uint64_t b = smem_desc(k_addr + s * k_stage + c * blk_bytes + k * 32, 16, 1024);
            umma_ss(tmem + kTmemS + sb * 128, a, b, idesc_s, (c | k) ? 1u : 0u);
          }
        umma_commit(&bars->s_full[sb]);
        if (j >= 1 && !issue_pv(j - 1)) { ok = false; break; }
      }
      if (ok && issue_pv(tp.nblk - 1)) umma_commit(&bars->o_done);
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ softmax, one thread per query row
    const int quarter = warp & 3;
    const int m = quarter * 32 + lane;
    const int qr = tp.r0 + m / pl.TW, qx = tp.x0 + m % pl.TW;
    const bool q_in = qr < p.t_h && qx < p.Wtok;
    const uint64_t colmask = column_mask(p, tp.hx0, qx, q_in);
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    const float c2 = p.scale_log2;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < tp.nblk; ++j) {
      const int sb = j & 1, pb = j % pl.pbufs;
      if (!mbar_wait(&bars->s_full[sb], (j >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      uint32_t sr[128];
#pragma unroll
      for (int c = 0; c < 8; ++c)
        if (c * 16 < N) tmem_ld16(lane_base + kTmemS + sb * 128 + c * 16, &sr[c * 16]);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(&bars->s_empty[sb]);

      uint32_t vm[4];
      block_mask(vm, p, colmask, tp.hr_first + j * pl.KR, qr, tp.hr_last);
      float mx = -INFINITY;
#pragma unroll
      for (int e = 0; e < 128; ++e)
        if (e < N) {
          float v = __uint_as_float(sr[e]);
          v = ((vm[e >> 5] >> (e & 31)) & 1u) ? v : -INFINITY;
          sr[e] = __float_as_uint(v);
          mx = fmaxf(mx, v);
        }
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

      if (j >= pl.pbufs && !mbar_wait(&bars->p_empty[pb], ((j / pl.pbufs) - 1) & 1, abort_flag)) { ok = false; break; }
      uint8_t* prow = p_smem + pb * pch * 16384;
      float lsum = 0.f;
#pragma unroll
      for (int u = 0; u < 16; ++u)
        if (u * 8 < N) {
          uint32_t w[4];
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            const float p0 = exp2f(fmaf(__uint_as_float(sr[u * 8 + 2 * h]), c2, -mc));
            const float p1 = exp2f(fmaf(__uint_as_float(sr[u * 8 + 2 * h + 1]), c2, -mc));
            lsum += p0 + p1;
            w[h] = pack2<BF16>(p0, p1);
          }
          *reinterpret_cast<uint4*>(swz(prow + (u >> 3) * 16384, m, u & 7)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      l += lsum;
      fence_proxy_async_smem();
      if (any_need && j > 0) {
        // O must be at rest: wait for PV of block j-1, then scale this thread's row
        const int pprev = (j - 1) % pl.pbufs;
        if (!mbar_wait(&bars->p_empty[pprev], ((j - 1) / pl.pbufs) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        for (int c = 0; c < p.vch * 4; ++c) {
          uint32_t orow[16];
          tmem_ld16(lane_base + kTmemO + c * 16, orow);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * alpha);
          tmem_st16(lane_base + kTmemO + c * 16, orow);
        }
        tmem_wait_st();
        tc_fence_before();
      }
      mbar_arrive(&bars->p_full[pb]);
    }
    // epilogue: O / l and lse
    if (ok && mbar_wait(&bars->o_done, 0, abort_flag)) {
      tc_fence_after();
      const float inv = 1.f / l;
      const int64_t tok = (int64_t)qr * p.Wtok + qx;
      using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
      T* orow_g = (T*)o.ptr + bi * o.s0 + hi * o.s1 + tok * o.s2;
      for (int c = 0; c < p.vch * 4; ++c) {
        uint32_t orow[16];
        tmem_ld16(lane_base + kTmemO + c * 16, orow);
        tmem_wait_ld();
        if (q_in) {
          uint32_t w[8];
#pragma unroll
          for (int h = 0; h < 8; ++h)
            w[h] = pack2<BF16>(__uint_as_float(orow[2 * h]) * inv, __uint_as_float(orow[2 * h + 1]) * inv);
          uint4* dst = reinterpret_cast<uint4*>(orow_g + c * 16);
          dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
          dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
        }
      }
      if (q_in) lse[(int64_t)bh * p.t_h * p.Wtok + tok] = m_used * c2 + log2f(l);
      tc_fence_before();
    }
  } else {
    // ------------------------------------------------------------------ fused RoPE-2D on Q and K tiles
    const int t = threadIdx.x - 192;
    const bool rope_on = p.rope.idx != nullptr;
    if (mbar_wait(&bars->q_full, 0, abort_flag)) {
      if (rope_on) {
        const int qr = tp.r0 + t / pl.TW, qx = tp.x0 + t % pl.TW;
        if (qr < p.t_h && qx < p.Wtok) rotate_row_smem<BF16>(q_smem, 16384, t, qr * p.Wtok + qx, p.rope);
        fence_proxy_async_smem();
      }
      mbar_arrive(&bars->q_ready);
      for (int j = 0; j < tp.nblk; ++j) {
        const int s = j % pl.stages;
        if (!mbar_wait(&bars->kv_full[s], (j / pl.stages) & 1, abort_flag)) break;
        if (rope_on) {
          if (t < N) {
            const int kr = tp.hr_first + j * pl.KR + t / pl.KW, kx = tp.hx0 + t % pl.KW;
            if (kr < p.t_h && kx >= 0 && kx < p.Wtok)
              rotate_row_smem<BF16>(k_smem + s * k_stage, blk_bytes, t, kr * p.Wtok + kx, p.rope);
          }
          fence_proxy_async_smem();
        }
        mbar_arrive(&bars->k_ready[s]);
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
