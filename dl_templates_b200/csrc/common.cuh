// Shared device/host helpers for the 2D sliding-window attention kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/swa2d.h"

namespace swa {

constexpr float kLog2e = 1.4426950408889634f;

// ---- element <-> float ---------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- strided [B,H,N,d] view ----------------------------------------------------------------
struct View4 {
  void* ptr;
  int64_t s0, s1, s2, s3;
};

inline View4 make_view(const swa_tensor_t* t) {
  return View4{t->ptr, t->stride[0], t->stride[1], t->stride[2], t->stride[3]};
}

// ---- fused RoPE-2D parameters (idx == nullptr: none) ---------------------------------------
struct RopeDev {
  const int32_t* idx;
  const float* row_cs;
  const float* col_cs;
  int R, max_h, max_w;
};

inline RopeDev make_rope(const swa_rope_t* r) {
  if (r == nullptr || r->idx == nullptr) return RopeDev{nullptr, nullptr, nullptr, 0, 0, 0};
  return RopeDev{r->idx, r->row_cs, r->col_cs, r->n_rdim, r->max_h, r->max_w};
}

// Packed index -> (row, col) as sign-extended 16-bit halves; a negative half
// disables that half's rotation.  Positions are clamped to the table length so a
// bad index can never read outside the table.
__device__ __forceinline__ void decode_idx(int32_t packed, int max_h, int max_w, int& row, int& col) {
  row = packed >> 16;
  col = (int)(int16_t)(packed & 0xFFFF);
  row = row >= max_h ? max_h - 1 : row;
  col = col >= max_w ? max_w - 1 : col;
}

// Geometry handed to every attention kernel.
struct Geom {
  int B, H, b, th, tw, wr, wc, dqk, dv;
  float scale_log2;  // sm_scale * log2(e)
  float sm_scale;
};

inline Geom make_geom(const swa_geom_t* g) {
  Geom r;
  r.B = g->B; r.H = g->H; r.b = g->b_size; r.th = g->t_height; r.tw = g->t_width;
  r.wr = g->row_size; r.wc = g->col_size; r.dqk = g->d_qk; r.dv = g->d_v;
  r.sm_scale = g->sm_scale; r.scale_log2 = g->sm_scale * kLog2e;
  return r;
}

}  // namespace swa
