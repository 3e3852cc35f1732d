// CUDA-core (SIMT) kernels: fp32-accumulate windowed attention forward, dQ and
// dK/dV for every dtype, head dim (<= 256), tile size and stride pattern.  They are
// the fp32 path (a 1e-4 tolerance is out of reach of a single-pass tensor-core
// format) and the path for shapes the tcgen05 kernels do not cover.
//
// One warp owns one token.  Lane l holds head dims l, l+32, l+64, ...; a dot
// product is a per-lane partial sum followed by a 5-step butterfly.  Nothing is
// accumulated with atomics, so results are bitwise reproducible.
#pragma once

#include "common.cuh"

namespace swa {

constexpr int kMaxT = 8;  // head dim <= 32 * kMaxT

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Element `d` of a q/k row after the RoPE-2D rotation (sign=+1) or its inverse
// (sign=-1).  Pair (i, i+R) of the row segment and pair (2R+i, 3R+i) of the column
// segment; dims >= 4R and halves with a negative index pass through.
template <typename T>
__device__ __forceinline__ float load_rot(const T* row, int64_t s3, int d, const RopeDev& rp, int irow, int icol,
                                          float sign) {
  float x = to_f(row[d * s3]);
  if (rp.idx == nullptr || d >= 4 * rp.R) return x;
  int seg = d / rp.R, i = d - seg * rp.R;
  int pos = seg >= 2 ? icol : irow;
  if (pos < 0) return x;
  const float* t = (seg >= 2 ? rp.col_cs : rp.row_cs) + ((int64_t)pos * rp.R + i) * 2;
  float c = t[0], s = t[1] * sign;
  if ((seg & 1) == 0) {
    float x1 = to_f(row[(d + rp.R) * s3]);
    return x * c - x1 * s;
  }
  float x0 = to_f(row[(d - rp.R) * s3]);
  return x0 * s + x * c;
}

// Inverse-rotate a gradient row held across the warp (vals[t] = dim lane+32t) and
// store it.  The partner element lives in another lane, so the row goes through
// a per-warp shared buffer.
template <typename T>
__device__ __forceinline__ void store_row_inv_rot(T* dst, int64_t s3, const float* vals, int d, int lane,
                                                  const RopeDev& rp, int irow, int icol, float* buf) {
#pragma unroll
  for (int t = 0; t < kMaxT; ++t)
    if (lane + 32 * t < d) buf[lane + 32 * t] = vals[t];
  __syncwarp();
#pragma unroll
  for (int t = 0; t < kMaxT; ++t) {
    int dd = lane + 32 * t;
    if (dd < d) dst[dd * s3] = from_f<T>(load_rot<float>(buf, 1, dd, rp, irow, icol, -1.f));
  }
  __syncwarp();
}

struct TokenPos {
  int r, c, s;
};

__device__ __forceinline__ TokenPos token_pos(int n, const Geom& g) {
  int tile = n / g.b;
  TokenPos p;
  p.s = n - tile * g.b;
  p.r = tile / g.tw;
  p.c = tile - p.r * g.tw;
  return p;
}

// ---------------------------------------------------------------------------------------------
// Forward.  grid = (ceil(N / warps), B*H), block = 32 * warps.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) simt_fwd_kernel(Geom g, RopeDev rp, View4 q, View4 k, View4 v, View4 o,
                                                       float* __restrict__ lse) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int N = g.th * g.tw * g.b;
  const int n = blockIdx.x * (blockDim.x >> 5) + warp;
  if (n >= N) return;
  const int bh = blockIdx.y, bi = bh / g.H, hi = bh - bi * g.H;
  const T* qrow = (const T*)q.ptr + bi * q.s0 + hi * q.s1 + (int64_t)n * q.s2;
  const T* kb = (const T*)k.ptr + bi * k.s0 + hi * k.s1;
  const T* vb = (const T*)v.ptr + bi * v.s0 + hi * v.s1;
  const TokenPos qp = token_pos(n, g);

  int irow = -1, icol = -1;
  if (rp.idx) decode_idx(rp.idx[n], rp.max_h, rp.max_w, irow, icol);
  float qreg[kMaxT], acc[kMaxT];
#pragma unroll
  for (int t = 0; t < kMaxT; ++t) {
    int d = lane + 32 * t;
    qreg[t] = d < g.dqk ? load_rot(qrow, q.s3, d, rp, irow, icol, 1.f) * g.scale_log2 : 0.f;
    acc[t] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const int r0 = max(0, qp.r - g.wr), r1 = min(g.th - 1, qp.r + g.wr);
  const int c0 = max(0, qp.c - g.wc), c1 = min(g.tw - 1, qp.c + g.wc);
  for (int kr = r0; kr <= r1; ++kr)
    for (int kc = c0; kc <= c1; ++kc)
      for (int ks = 0; ks < g.b; ++ks) {
        const int kn = (kr * g.tw + kc) * g.b + ks;
        const T* krow = kb + (int64_t)kn * k.s2;
        int kir = -1, kic = -1;
        if (rp.idx) decode_idx(rp.idx[kn], rp.max_h, rp.max_w, kir, kic);
        float part = 0.f;
#pragma unroll
        for (int t = 0; t < kMaxT; ++t) {
          int d = lane + 32 * t;
          if (d < g.dqk) part += qreg[t] * load_rot(krow, k.s3, d, rp, kir, kic, 1.f);
        }
        const float s = warp_sum(part);
        const float mn = fmaxf(m, s);
        const float alpha = exp2f(m - mn), p = exp2f(s - mn);
        l = l * alpha + p;
        m = mn;
        const T* vrow = vb + (int64_t)kn * v.s2;
#pragma unroll
        for (int t = 0; t < kMaxT; ++t) {
          int d = lane + 32 * t;
          if (d < g.dv) acc[t] = acc[t] * alpha + p * to_f(vrow[d * v.s3]);
        }
      }
  T* orow = (T*)o.ptr + bi * o.s0 + hi * o.s1 + (int64_t)n * o.s2;
  const float inv = 1.f / l;
#pragma unroll
  for (int t = 0; t < kMaxT; ++t) {
    int d = lane + 32 * t;
    if (d < g.dv) orow[d * o.s3] = from_f<T>(acc[t] * inv);
  }
  if (lane == 0) lse[(int64_t)bh * N + n] = m + log2f(l);
}

// ---------------------------------------------------------------------------------------------
// dQ.  One warp per query; p is recomputed from lse.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) simt_dq_kernel(Geom g, RopeDev rp, View4 q, View4 k, View4 v, View4 d_o,
                                                      const float* __restrict__ lse,
                                                      const float* __restrict__ delta, View4 dq) {
  __shared__ float rot_buf[8][32 * kMaxT];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int N = g.th * g.tw * g.b;
  const int n = blockIdx.x * (blockDim.x >> 5) + warp;
  if (n >= N) return;
  const int bh = blockIdx.y, bi = bh / g.H, hi = bh - bi * g.H;
  const T* qrow = (const T*)q.ptr + bi * q.s0 + hi * q.s1 + (int64_t)n * q.s2;
  const T* dorow = (const T*)d_o.ptr + bi * d_o.s0 + hi * d_o.s1 + (int64_t)n * d_o.s2;
  const T* kb = (const T*)k.ptr + bi * k.s0 + hi * k.s1;
  const T* vb = (const T*)v.ptr + bi * v.s0 + hi * v.s1;
  const TokenPos qp = token_pos(n, g);
  int irow = -1, icol = -1;
  if (rp.idx) decode_idx(rp.idx[n], rp.max_h, rp.max_w, irow, icol);
  float qreg[kMaxT], doreg[kMaxT], acc[kMaxT];
#pragma unroll
  for (int t = 0; t < kMaxT; ++t) {
    int d = lane + 32 * t;
    qreg[t] = d < g.dqk ? load_rot(qrow, q.s3, d, rp, irow, icol, 1.f) * g.scale_log2 : 0.f;
    doreg[t] = d < g.dv ? to_f(dorow[d * d_o.s3]) : 0.f;
    acc[t] = 0.f;
  }
  const float my_lse = lse[(int64_t)bh * N + n], my_delta = delta[(int64_t)bh * N + n];
  const int r0 = max(0, qp.r - g.wr), r1 = min(g.th - 1, qp.r + g.wr);
  const int c0 = max(0, qp.c - g.wc), c1 = min(g.tw - 1, qp.c + g.wc);
  for (int kr = r0; kr <= r1; ++kr)
    for (int kc = c0; kc <= c1; ++kc)
      for (int ks = 0; ks < g.b; ++ks) {
        const int kn = (kr * g.tw + kc) * g.b + ks;
        const T* krow = kb + (int64_t)kn * k.s2;
        const T* vrow = vb + (int64_t)kn * v.s2;
        int kir = -1, kic = -1;
        if (rp.idx) decode_idx(rp.idx[kn], rp.max_h, rp.max_w, kir, kic);
        float kreg[kMaxT];
        float ps = 0.f, pd = 0.f;
#pragma unroll
        for (int t = 0; t < kMaxT; ++t) {
          int d = lane + 32 * t;
          kreg[t] = d < g.dqk ? load_rot(krow, k.s3, d, rp, kir, kic, 1.f) : 0.f;
          ps += qreg[t] * kreg[t];
          if (d < g.dv) pd += doreg[t] * to_f(vrow[d * v.s3]);
        }
        const float s = warp_sum(ps), dp = warp_sum(pd);
        const float p = exp2f(s - my_lse);
        const float ds = p * (dp - my_delta);
#pragma unroll
        for (int t = 0; t < kMaxT; ++t) acc[t] += ds * kreg[t];
      }
#pragma unroll
  for (int t = 0; t < kMaxT; ++t) acc[t] *= g.sm_scale;
  T* dqrow = (T*)dq.ptr + bi * dq.s0 + hi * dq.s1 + (int64_t)n * dq.s2;
  store_row_inv_rot(dqrow, dq.s3, acc, g.dqk, lane, rp, irow, icol, rot_buf[warp]);
}

// ---------------------------------------------------------------------------------------------
// dK / dV.  One warp per key; the tile window relation is symmetric, so the
// queries that see a key are the tokens of the tiles within the key's own window.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) simt_dkdv_kernel(Geom g, RopeDev rp, View4 q, View4 k, View4 v, View4 d_o,
                                                        const float* __restrict__ lse,
                                                        const float* __restrict__ delta, View4 dk, View4 dv) {
  __shared__ float rot_buf[8][32 * kMaxT];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int N = g.th * g.tw * g.b;
  const int n = blockIdx.x * (blockDim.x >> 5) + warp;
  if (n >= N) return;
  const int bh = blockIdx.y, bi = bh / g.H, hi = bh - bi * g.H;
  const T* krow = (const T*)k.ptr + bi * k.s0 + hi * k.s1 + (int64_t)n * k.s2;
  const T* vrow = (const T*)v.ptr + bi * v.s0 + hi * v.s1 + (int64_t)n * v.s2;
  const T* qb = (const T*)q.ptr + bi * q.s0 + hi * q.s1;
  const T* dob = (const T*)d_o.ptr + bi * d_o.s0 + hi * d_o.s1;
  const TokenPos kp = token_pos(n, g);
  int irow = -1, icol = -1;
  if (rp.idx) decode_idx(rp.idx[n], rp.max_h, rp.max_w, irow, icol);
  float kreg[kMaxT], vreg[kMaxT], dkacc[kMaxT], dvacc[kMaxT];
#pragma unroll
  for (int t = 0; t < kMaxT; ++t) {
    int d = lane + 32 * t;
    kreg[t] = d < g.dqk ? load_rot(krow, k.s3, d, rp, irow, icol, 1.f) * g.scale_log2 : 0.f;
    vreg[t] = d < g.dv ? to_f(vrow[d * v.s3]) : 0.f;
    dkacc[t] = 0.f;
    dvacc[t] = 0.f;
  }
  const int r0 = max(0, kp.r - g.wr), r1 = min(g.th - 1, kp.r + g.wr);
  const int c0 = max(0, kp.c - g.wc), c1 = min(g.tw - 1, kp.c + g.wc);
  for (int qr = r0; qr <= r1; ++qr)
    for (int qc = c0; qc <= c1; ++qc)
      for (int qs = 0; qs < g.b; ++qs) {
        const int qn = (qr * g.tw + qc) * g.b + qs;
        const T* qrow = qb + (int64_t)qn * q.s2;
        const T* dorow = dob + (int64_t)qn * d_o.s2;
        int qir = -1, qic = -1;
        if (rp.idx) decode_idx(rp.idx[qn], rp.max_h, rp.max_w, qir, qic);
        float qreg[kMaxT], doreg[kMaxT];
        float ps = 0.f, pd = 0.f;
#pragma unroll
        for (int t = 0; t < kMaxT; ++t) {
          int d = lane + 32 * t;
          qreg[t] = d < g.dqk ? load_rot(qrow, q.s3, d, rp, qir, qic, 1.f) : 0.f;
          doreg[t] = d < g.dv ? to_f(dorow[d * d_o.s3]) : 0.f;
          ps += qreg[t] * kreg[t];
          pd += doreg[t] * vreg[t];
        }
        const float s = warp_sum(ps), dp = warp_sum(pd);
        const float p = exp2f(s - lse[(int64_t)bh * N + qn]);
        const float ds = p * (dp - delta[(int64_t)bh * N + qn]);
#pragma unroll
        for (int t = 0; t < kMaxT; ++t) {
          dvacc[t] += p * doreg[t];
          dkacc[t] += ds * qreg[t];
        }
      }
#pragma unroll
  for (int t = 0; t < kMaxT; ++t) dkacc[t] *= g.sm_scale;
  T* dvrow = (T*)dv.ptr + bi * dv.s0 + hi * dv.s1 + (int64_t)n * dv.s2;
#pragma unroll
  for (int t = 0; t < kMaxT; ++t) {
    int d = lane + 32 * t;
    if (d < g.dv) dvrow[d * dv.s3] = from_f<T>(dvacc[t]);
  }
  T* dkrow = (T*)dk.ptr + bi * dk.s0 + hi * dk.s1 + (int64_t)n * dk.s2;
  store_row_inv_rot(dkrow, dk.s3, dkacc, g.dqk, lane, rp, irow, icol, rot_buf[warp]);
}

}  // namespace swa
