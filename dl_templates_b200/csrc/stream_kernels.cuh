// HBM-bound streaming kernels: the softmax-delta preprocess (delta = rowsum(o*do))
// and the stand-alone in-place RoPE-2D.  Both move each byte once with 16-byte
// accesses when the layout allows, and fall back to element accesses otherwise.
#pragma once

#include "common.cuh"

namespace swa {

// ---- delta ------------------------------------------------------------------------------------
// Vector path (16-bit types, d_v % 8 == 0, unit last stride, 16-byte aligned rows):
// a group of d_v/8 consecutive threads owns one token, each thread reads 8 elements
// of o and of do, the group reduces with shuffles.  Groups never straddle a warp
// because d_v/8 is a power of two <= 32 on this path.
template <typename T>
__global__ void __launch_bounds__(256) delta_vec_kernel(View4 o, View4 d_o, float* __restrict__ delta, int H,
                                                        int64_t N, int dv, int64_t total_rows) {
  const int tpr = dv >> 3;  // threads per row
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t row = gid / tpr;
  const int part = (int)(gid - row * tpr);
  float acc = 0.f;
  if (row < total_rows) {
    const int64_t bh = row / N, n = row - bh * N;
    const int64_t bi = bh / H, hi = bh - bi * H;
    const uint4 a = *reinterpret_cast<const uint4*>((const T*)o.ptr + bi * o.s0 + hi * o.s1 + n * o.s2 + part * 8);
    const uint4 b =
        *reinterpret_cast<const uint4*>((const T*)d_o.ptr + bi * d_o.s0 + hi * d_o.s1 + n * d_o.s2 + part * 8);
    const T* pa = reinterpret_cast<const T*>(&a);
    const T* pb = reinterpret_cast<const T*>(&b);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += to_f(pa[i]) * to_f(pb[i]);
  }
  for (int off = tpr >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (row < total_rows && part == 0) delta[row] = acc;
}

// Same for fully contiguous o and do: no per-thread index decomposition of the loads.  Head-major memory
// ([B,H,N,d_v] row-major) writes delta[row]; TOKEN_MAJOR memory ([B,N,H,d_v] row-major, the layout next to an
// output projection) is walked in memory order and row (b, n, h) writes delta[(b*H + h)*N + n].
template <typename T, bool TOKEN_MAJOR = false>
__global__ void __launch_bounds__(256) delta_flat_kernel(const T* __restrict__ o, const T* __restrict__ d_o,
                                                         float* __restrict__ delta, int dv, int64_t total_rows,
                                                         int H = 1, int64_t N = 1) {
  const int tpr = dv >> 3;  // threads per row
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t row = gid / tpr;
  float acc = 0.f;
  if (row < total_rows) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(o) + gid);
    const uint4 b = __ldg(reinterpret_cast<const uint4*>(d_o) + gid);
    const T* pa = reinterpret_cast<const T*>(&a);
    const T* pb = reinterpret_cast<const T*>(&b);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += to_f(pa[i]) * to_f(pb[i]);
  }
  for (int off = tpr >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (row < total_rows && (gid - row * tpr) == 0) {
    if (TOKEN_MAJOR) {
      if (total_rows < (int64_t(1) << 31)) {   // 32-bit index arithmetic: two 64-bit divisions per row are not free here
        const uint32_t r = (uint32_t)row, uh = (uint32_t)H, un = (uint32_t)N;
        const uint32_t bn = r / uh, h = r - bn * uh, b = bn / un, n = bn - b * un;
        delta[((int64_t)b * H + h) * N + n] = acc;
      } else {
        const int64_t bn = row / H, h = row - bn * H;
        const int64_t b = bn / N, n = bn - b * N;
        delta[(b * H + h) * N + n] = acc;
      }
    } else {
      delta[row] = acc;
    }
  }
}

// Element path: one warp per token, any dtype / stride / head dim.
template <typename T>
__global__ void __launch_bounds__(256) delta_generic_kernel(View4 o, View4 d_o, float* __restrict__ delta, int H,
                                                            int64_t N, int dv, int64_t total_rows) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= total_rows) return;
  const int64_t bh = row / N, n = row - bh * N;
  const int64_t bi = bh / H, hi = bh - bi * H;
  const T* po = (const T*)o.ptr + bi * o.s0 + hi * o.s1 + n * o.s2;
  const T* pd = (const T*)d_o.ptr + bi * d_o.s0 + hi * d_o.s1 + n * d_o.s2;
  float acc = 0.f;
  for (int d = lane; d < dv; d += 32) acc += to_f(po[d * o.s3]) * to_f(pd[d * d_o.s3]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) delta[row] = acc;
}

// ---- stand-alone RoPE-2D, in place -----------------------------------------------------------
// x [batch, N, C] with element strides (xs0, xs1, xs2).  One thread rotates VEC
// consecutive pairs (i .. i+VEC) of one half (row or column) of one token of one
// batch entry; tokens whose half has a negative index are skipped without
// touching memory.  blockIdx.y is the batch entry.
template <typename T, int VEC>
__global__ void __launch_bounds__(256) rope2d_kernel(T* __restrict__ x, int64_t batch, int64_t N, int64_t xs0,
                                                     int64_t xs1, int64_t xs2, RopeDev rp, float sign) {
  const int per_tok = 2 * (rp.R / VEC);  // work items per token: halves x chunks
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t tok = gid / per_tok;
  const int item = (int)(gid - tok * per_tok);
  const int64_t bi = blockIdx.y;
  if (tok >= N || bi >= batch) return;
  int irow, icol;
  decode_idx(rp.idx[tok], rp.max_h, rp.max_w, irow, icol);
  const int half = item / (rp.R / VEC);  // 0 row, 1 col
  const int i0 = (item - half * (rp.R / VEC)) * VEC;
  const int pos = half ? icol : irow;
  if (pos < 0) return;
  const float* tab = (half ? rp.col_cs : rp.row_cs) + ((int64_t)pos * rp.R + i0) * 2;
  T* p0 = x + bi * xs0 + tok * xs1 + (int64_t)(2 * half * rp.R + i0) * xs2;
  T* p1 = p0 + (int64_t)rp.R * xs2;
  if constexpr (VEC == 1) {
    const float c = tab[0], s = tab[1] * sign;
    const float a = to_f(*p0), b = to_f(*p1);
    *p0 = from_f<T>(a * c - b * s);
    *p1 = from_f<T>(a * s + b * c);
  } else {
    // VEC * sizeof(T) == 16 bytes, unit element stride, 16-byte aligned (checked on the host)
    uint4 va = *reinterpret_cast<const uint4*>(p0), vb = *reinterpret_cast<const uint4*>(p1);
    T* ea = reinterpret_cast<T*>(&va);
    T* eb = reinterpret_cast<T*>(&vb);
    float cs[2 * VEC];
#pragma unroll
    for (int j = 0; j < 2 * VEC; j += 4) *reinterpret_cast<float4*>(cs + j) = *reinterpret_cast<const float4*>(tab + j);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float c = cs[2 * j], s = cs[2 * j + 1] * sign;
      const float a = to_f(ea[j]), b = to_f(eb[j]);
      ea[j] = from_f<T>(a * c - b * s);
      eb[j] = from_f<T>(a * s + b * c);
    }
    *reinterpret_cast<uint4*>(p0) = va;
    *reinterpret_cast<uint4*>(p1) = vb;
  }
}

// Out-of-place form for 16-bit types: y = rope(x), x untouched.  One thread per 16-byte unit of a token row
// (8 elements): units outside the rotated dims, or of a half whose index is negative, are copied; a rotated unit
// reads its partner unit (R elements away, same row, so the same DRAM sectors another thread reads) and writes
// its own half of the pair.  Needs R % 8 == 0, C % 8 == 0, unit last strides and 16-byte aligned rows.
template <typename T>
__global__ void __launch_bounds__(256) rope2d_copy_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows,
                                                          int64_t N, int C, int64_t xs0, int64_t xs1, int64_t ys0,
                                                          int64_t ys1, RopeDev rp, float sign) {
  const int upr = C >> 3;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t row = gid / upr;
  if (row >= rows) return;
  const int u = (int)(gid - row * upr);
  const int64_t bi = row / N, tok = row - bi * N;
  const T* src = x + bi * xs0 + tok * xs1 + u * 8;
  uint4 own = *reinterpret_cast<const uint4*>(src);
  const int e0 = u * 8;
  if (e0 < 4 * rp.R) {
    const int seg = e0 / rp.R, half = seg >> 1, second = seg & 1, i0 = e0 - seg * rp.R;
    int irow, icol;
    decode_idx(rp.idx[tok], rp.max_h, rp.max_w, irow, icol);
    const int pos = half ? icol : irow;
    if (pos >= 0) {
      const uint4 oth = *reinterpret_cast<const uint4*>(second ? src - rp.R : src + rp.R);
      const float* tab = (half ? rp.col_cs : rp.row_cs) + ((int64_t)pos * rp.R + i0) * 2;
      float cs[16];
#pragma unroll
      for (int j = 0; j < 16; j += 4) *reinterpret_cast<float4*>(cs + j) = *reinterpret_cast<const float4*>(tab + j);
      T* eo = reinterpret_cast<T*>(&own);
      const T* ep = reinterpret_cast<const T*>(&oth);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float c = cs[2 * j], sn = cs[2 * j + 1] * sign;
        const float a = second ? to_f(ep[j]) : to_f(eo[j]), b = second ? to_f(eo[j]) : to_f(ep[j]);
        eo[j] = from_f<T>(second ? a * sn + b * c : a * c - b * sn);
      }
    }
  }
  *reinterpret_cast<uint4*>(y + bi * ys0 + tok * ys1 + u * 8) = own;
}

// One-pass clone + rotate for a strided [B, H, N, C] 16-bit tensor (both tensors described by four element
// strides, so packed projection outputs need no flattening copy).  One thread per "slot" of a token row: a slot of
// the rotated dims is a 16-byte unit together with its partner unit R elements further (both halves of eight
// pairs: two 16-byte loads, one set of cos/sin values, two 16-byte stores, nothing read twice); a slot of the dims
// beyond 4R is two consecutive units that are copied.  grid = (slots of one (batch, head) slice / 256, B * H).
template <typename T>
__global__ void __launch_bounds__(256) rope2d_copy4_kernel(View4 x, View4 y, int H, int N, int C, RopeDev rp, float sign) {
  const uint32_t rot_slots = (uint32_t)rp.R >> 2;                       // 4R / 8 units, two per slot
  const uint32_t spr = rot_slots + ((((uint32_t)C >> 3) - 2 * rot_slots + 1) >> 1);   // slots per row
  const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t tok = gid / spr;
  if (tok >= (uint32_t)N) return;
  const uint32_t sl = gid - tok * spr;
  const uint32_t bh = blockIdx.y;
  const int64_t b = bh / (uint32_t)H, h = bh - (uint32_t)b * (uint32_t)H;
  const T* src = (const T*)x.ptr + b * x.s0 + h * x.s1 + (int64_t)tok * x.s2;
  T* dst = (T*)y.ptr + b * y.s0 + h * y.s1 + (int64_t)tok * y.s2;
  if (sl < rot_slots) {
    const uint32_t per_half = (uint32_t)rp.R >> 3;                      // slots of the row-angle half
    const uint32_t half = sl / per_half, i0 = (sl - half * per_half) * 8;
    const uint32_t e0 = half * 2 * rp.R + i0, e1 = e0 + rp.R;
    uint4 va = *reinterpret_cast<const uint4*>(src + e0), vb = *reinterpret_cast<const uint4*>(src + e1);
    int irow, icol;
    decode_idx(__ldg(rp.idx + tok), rp.max_h, rp.max_w, irow, icol);
    const int pos = half ? icol : irow;
    if (pos >= 0) {
      const float4* tab = reinterpret_cast<const float4*>((half ? rp.col_cs : rp.row_cs) + ((int64_t)pos * rp.R + i0) * 2);
      T* ea = reinterpret_cast<T*>(&va);
      T* eb = reinterpret_cast<T*>(&vb);
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        const float4 cs = __ldg(tab + (j >> 1));                        // (cos, sin) of pairs j and j + 1
        const float a0 = to_f(ea[j]), b0 = to_f(eb[j]), a1 = to_f(ea[j + 1]), b1 = to_f(eb[j + 1]);
        const float s0 = cs.y * sign, s1 = cs.w * sign;
        ea[j] = from_f<T>(a0 * cs.x - b0 * s0);
        eb[j] = from_f<T>(a0 * s0 + b0 * cs.x);
        ea[j + 1] = from_f<T>(a1 * cs.z - b1 * s1);
        eb[j + 1] = from_f<T>(a1 * s1 + b1 * cs.z);
      }
    }
    *reinterpret_cast<uint4*>(dst + e0) = va;
    *reinterpret_cast<uint4*>(dst + e1) = vb;
  } else {
    const uint32_t e0 = 4 * rp.R + (sl - rot_slots) * 16;
    *reinterpret_cast<uint4*>(dst + e0) = *reinterpret_cast<const uint4*>(src + e0);
    if (e0 + 8 < (uint32_t)C) *reinterpret_cast<uint4*>(dst + e0 + 8) = *reinterpret_cast<const uint4*>(src + e0 + 8);
  }
}

// Element path of the same operation for any dtype and any strides; x == y (in place) is allowed.  One thread
// per (token row, rotated pair): it reads both elements of its pair and writes both, and copies its share of the
// dims beyond 4 * n_rdim when the operation is out of place.
template <typename T>
__global__ void __launch_bounds__(256) rope2d_generic4_kernel(View4 x, View4 y, int64_t rows, int H, int64_t N, int C,
                                                              RopeDev rp, float sign) {
  const int ppr = 2 * rp.R;   // pairs per row
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t row = gid / ppr;
  if (row >= rows) return;
  const int pi = (int)(gid - row * ppr);
  const int64_t bh = row / N, tok = row - bh * N;
  const int64_t b = bh / H, h = bh - b * H;
  const T* src = (const T*)x.ptr + b * x.s0 + h * x.s1 + tok * x.s2;
  T* dst = (T*)y.ptr + b * y.s0 + h * y.s1 + tok * y.s2;
  const int half = pi / rp.R, i = pi - half * rp.R;
  const int d0 = 2 * half * rp.R + i, d1 = d0 + rp.R;
  int irow, icol;
  decode_idx(rp.idx[tok], rp.max_h, rp.max_w, irow, icol);
  const int pos = half ? icol : irow;
  float a = to_f(src[d0 * x.s3]), bb = to_f(src[d1 * x.s3]);
  if (pos >= 0) {
    const float* tab = (half ? rp.col_cs : rp.row_cs) + ((int64_t)pos * rp.R + i) * 2;
    const float c = tab[0], sn = tab[1] * sign;
    const float ra = a * c - bb * sn, rb = a * sn + bb * c;
    a = ra;
    bb = rb;
  }
  dst[d0 * y.s3] = from_f<T>(a);
  dst[d1 * y.s3] = from_f<T>(bb);
  if (src != dst || x.s3 != y.s3)
    for (int d = 4 * rp.R + pi; d < C; d += ppr) dst[d * y.s3] = src[d * x.s3];
}

}  // namespace swa
