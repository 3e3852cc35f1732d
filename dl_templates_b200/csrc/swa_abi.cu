// C ABI (include/swa2d.h): argument validation, kernel-family selection, launches.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "stream_kernels.cuh"
#include "swa_simt.cuh"
#include "swa_tc.cuh"

namespace {

thread_local char g_err[512] = "";
std::atomic<int64_t> g_launches{0};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

enum : int {
  E_NULL = -1, E_DTYPE = -2, E_SHAPE = -3, E_ROPE = -4, E_IMPL = -5, E_LAUNCH = -6, E_STRIDE = -7
};

int check_geom(const swa_geom_t* g) {
  if (!g) return fail(E_NULL, "geometry is NULL");
  if (g->dtype < SWA_F32 || g->dtype > SWA_BF16) return fail(E_DTYPE, "unknown dtype %d", g->dtype);
  if (g->B <= 0 || g->H <= 0 || g->b_size <= 0 || g->t_height <= 0 || g->t_width <= 0)
    return fail(E_SHAPE, "B, H, b_size, t_height, t_width must be positive");
  if (g->row_size < 0 || g->col_size < 0) return fail(E_SHAPE, "window half-sizes must be >= 0");
  if (g->d_qk <= 0 || g->d_v <= 0 || g->d_qk > 32 * swa::kMaxT || g->d_v > 32 * swa::kMaxT)
    return fail(E_SHAPE, "head dims must be in [1, %d]", 32 * swa::kMaxT);
  if ((int64_t)g->t_height * g->t_width * g->b_size > (int64_t)INT32_MAX)
    return fail(E_SHAPE, "too many tokens per head");
  if ((int64_t)g->B * g->H > 65535) return fail(E_SHAPE, "B*H exceeds 65535");
  if (g->impl < SWA_IMPL_AUTO || g->impl > SWA_IMPL_TC) return fail(E_IMPL, "unknown impl %d", g->impl);
  return 0;
}

int check_rope(const swa_geom_t* g, const swa_rope_t* r) {
  if (!r || !r->idx) return 0;
  if (!r->row_cs || !r->col_cs) return fail(E_ROPE, "rope tables are NULL");
  if (r->n_rdim <= 0 || 4 * r->n_rdim > g->d_qk)
    return fail(E_ROPE, "4*n_rdim (%d) must be in [4, d_qk=%d]", 4 * r->n_rdim, g->d_qk);
  if (r->max_h <= 0 || r->max_w <= 0) return fail(E_ROPE, "rope table lengths must be positive");
  return 0;
}

int check_tensor(const swa_tensor_t* t, const char* name) {
  if (!t || !t->ptr) return fail(E_NULL, "%s is NULL", name);
  return 0;
}

int launch_ok(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(E_LAUNCH, "%s launch failed: %s", what, cudaGetErrorString(e));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return 0;
}

// Runs `body` with T bound to the element type of the call.
#define SWA_DISPATCH_DTYPE(dtype, ...)                                  \
  do {                                                                  \
    switch (dtype) {                                                    \
      case SWA_F32: { using T = float; __VA_ARGS__; break; }            \
      case SWA_F16: { using T = __half; __VA_ARGS__; break; }           \
      default: { using T = __nv_bfloat16; __VA_ARGS__; break; }         \
    }                                                                   \
  } while (0)

// Resolve AUTO / reject TC requests the tensor-core kernels cannot serve.
int resolve_impl(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* const* tensors, int n_tensors,
                 int which, bool prerotated = false) {
  const char* why = swa::tc::unsupported_reason(g, rope, tensors, n_tensors, which, prerotated);
  if (g->impl == SWA_IMPL_SIMT) return SWA_IMPL_SIMT;
  if (why == nullptr) return SWA_IMPL_TC;
  if (g->impl == SWA_IMPL_TC) return fail(E_IMPL, "tensor-core path unavailable: %s", why);
  return SWA_IMPL_SIMT;
}

}  // namespace

extern "C" {

int swa_version(void) { return 2; }
void swa_refresh_env(void) { swa::tc::refresh_env(); }
const char* swa_last_error(void) { return g_err; }
int64_t swa_launch_count(void) { return g_launches.load(); }

int swa_select_impl(const swa_geom_t* g, const swa_rope_t* rope, int32_t which) {
  if (int e = check_geom(g)) return e;
  if (int e = check_rope(g, rope)) return e;
  return resolve_impl(g, rope, nullptr, 0, which);
}

int swa_describe_plan(const swa_geom_t* g, const swa_rope_t* rope, int32_t which, int32_t* out) {
  if (int e = check_geom(g)) return e;
  if (int e = check_rope(g, rope)) return e;
  if (!out || which < 0 || which > 5) return fail(E_NULL, "swa_describe_plan: out is NULL or `which` not in 0..5");
  if (which >= 3 && !(rope && rope->idx)) return fail(E_ROPE, "swa_describe_plan: kernels 3..5 are the RoPE hand-off entries");
  if (swa::tc::unsupported_reason(g, rope, nullptr, 0, which % 3, which >= 3) != nullptr || !swa::tc::describe_plan(g, rope, which, out))
    return fail(E_SHAPE, "the tensor-core kernels do not take this shape");
  return 0;
}

int swa_fwd(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q, const swa_tensor_t* k,
            const swa_tensor_t* v, const swa_tensor_t* o, float* lse, int32_t* status, void* stream) {
  if (int e = check_geom(g)) return e;
  if (int e = check_rope(g, rope)) return e;
  if (int e = check_tensor(q, "q")) return e;
  if (int e = check_tensor(k, "k")) return e;
  if (int e = check_tensor(v, "v")) return e;
  if (int e = check_tensor(o, "o")) return e;
  if (!lse) return fail(E_NULL, "lse is NULL");
  const swa_tensor_t* ts[] = {q, k, v, o};
  const int impl = resolve_impl(g, rope, ts, 4, 0);
  if (impl < 0) return impl;
  cudaStream_t st = (cudaStream_t)stream;
  if (impl == SWA_IMPL_TC) {
    int e = swa::tc::launch_fwd(g, rope, q, k, v, o, lse, status, st);
    if (e) return fail(E_LAUNCH, "tcgen05 forward: %s", swa::tc::last_error());
    return launch_ok("tcgen05 forward");
  }
  const swa::Geom gg = swa::make_geom(g);
  const swa::RopeDev rp = swa::make_rope(rope);
  const int N = g->t_height * g->t_width * g->b_size;
  dim3 grid((N + 7) / 8, g->B * g->H), block(256);
  SWA_DISPATCH_DTYPE(g->dtype, swa::simt_fwd_kernel<T><<<grid, block, 0, st>>>(
                                   gg, rp, swa::make_view(q), swa::make_view(k), swa::make_view(v),
                                   swa::make_view(o), lse));
  return launch_ok("simt forward");
}

int swa_bwd_delta(const swa_geom_t* g, const swa_tensor_t* o, const swa_tensor_t* d_o, float* delta, void* stream) {
  if (int e = check_geom(g)) return e;
  if (int e = check_tensor(o, "o")) return e;
  if (int e = check_tensor(d_o, "do")) return e;
  if (!delta) return fail(E_NULL, "delta is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t N = (int64_t)g->t_height * g->t_width * g->b_size;
  const int64_t rows = N * g->B * g->H;
  const int dv = g->d_v;
  const int esz = g->dtype == SWA_F32 ? 4 : 2;
  auto vec_ok = [&](const swa_tensor_t* t) {
    return t->stride[3] == 1 && ((uintptr_t)t->ptr % 16) == 0 && (t->stride[0] * esz) % 16 == 0 &&
           (t->stride[1] * esz) % 16 == 0 && (t->stride[2] * esz) % 16 == 0;
  };
  const bool pow2 = (dv & (dv - 1)) == 0;
  if (esz == 2 && pow2 && dv >= 8 && dv <= 256 && vec_ok(o) && vec_ok(d_o)) {
    const int64_t threads = rows * (dv / 8);
    const unsigned blocks = (unsigned)((threads + 255) / 256);
    auto flat = [&](const swa_tensor_t* t) {
      return t->stride[2] == dv && t->stride[1] == N * dv && (g->B == 1 || t->stride[0] == (int64_t)g->H * N * dv);
    };
    if (flat(o) && flat(d_o)) {
      if (g->dtype == SWA_F16)
        swa::delta_flat_kernel<__half><<<blocks, 256, 0, st>>>((const __half*)o->ptr, (const __half*)d_o->ptr, delta, dv, rows);
      else
        swa::delta_flat_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)o->ptr,
                                                                      (const __nv_bfloat16*)d_o->ptr, delta, dv, rows);
      return launch_ok("delta");
    }
    auto token_major = [&](const swa_tensor_t* t) {   // [B,N,H,d_v] row-major seen as [B,H,N,d_v]
      return t->stride[1] == dv && t->stride[2] == (int64_t)g->H * dv && (g->B == 1 || t->stride[0] == (int64_t)g->H * N * dv);
    };
    if (token_major(o) && token_major(d_o)) {
      if (g->dtype == SWA_F16)
        swa::delta_flat_kernel<__half, true><<<blocks, 256, 0, st>>>((const __half*)o->ptr, (const __half*)d_o->ptr, delta, dv,
                                                                     rows, g->H, N);
      else
        swa::delta_flat_kernel<__nv_bfloat16, true><<<blocks, 256, 0, st>>>(
            (const __nv_bfloat16*)o->ptr, (const __nv_bfloat16*)d_o->ptr, delta, dv, rows, g->H, N);
      return launch_ok("delta");
    }
    if (g->dtype == SWA_F16)
      swa::delta_vec_kernel<__half><<<blocks, 256, 0, st>>>(swa::make_view(o), swa::make_view(d_o), delta, g->H, N,
                                                            dv, rows);
    else
      swa::delta_vec_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(swa::make_view(o), swa::make_view(d_o), delta,
                                                                   g->H, N, dv, rows);
    return launch_ok("delta");
  }
  const unsigned blocks = (unsigned)((rows + 7) / 8);
  SWA_DISPATCH_DTYPE(g->dtype, swa::delta_generic_kernel<T><<<blocks, 256, 0, st>>>(
                                   swa::make_view(o), swa::make_view(d_o), delta, g->H, N, dv, rows));
  return launch_ok("delta");
}

int swa_bwd_dq(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q, const swa_tensor_t* k,
               const swa_tensor_t* v, const swa_tensor_t* d_o, const float* lse, const float* delta,
               const swa_tensor_t* dq, int32_t* status, void* stream) {
  if (int e = check_geom(g)) return e;
  if (int e = check_rope(g, rope)) return e;
  if (int e = check_tensor(q, "q")) return e;
  if (int e = check_tensor(k, "k")) return e;
  if (int e = check_tensor(v, "v")) return e;
  if (int e = check_tensor(d_o, "do")) return e;
  if (int e = check_tensor(dq, "dq")) return e;
  if (!lse || !delta) return fail(E_NULL, "lse/delta is NULL");
  const swa_tensor_t* ts[] = {q, k, v, d_o, dq};
  const int impl = resolve_impl(g, rope, ts, 5, 1);
  if (impl < 0) return impl;
  cudaStream_t st = (cudaStream_t)stream;
  if (impl == SWA_IMPL_TC) {
    int e = swa::tc::launch_dq(g, rope, q, k, v, d_o, lse, delta, dq, status, st);
    if (e) return fail(E_LAUNCH, "tcgen05 dq: %s", swa::tc::last_error());
    return launch_ok("tcgen05 dq");
  }
  const swa::Geom gg = swa::make_geom(g);
  const swa::RopeDev rp = swa::make_rope(rope);
  const int N = g->t_height * g->t_width * g->b_size;
  dim3 grid((N + 7) / 8, g->B * g->H), block(256);
  SWA_DISPATCH_DTYPE(g->dtype, swa::simt_dq_kernel<T><<<grid, block, 0, st>>>(
                                   gg, rp, swa::make_view(q), swa::make_view(k), swa::make_view(v),
                                   swa::make_view(d_o), lse, delta, swa::make_view(dq)));
  return launch_ok("simt dq");
}

int swa_bwd_dkdv(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q, const swa_tensor_t* k,
                 const swa_tensor_t* v, const swa_tensor_t* d_o, const float* lse, const float* delta,
                 const swa_tensor_t* dk, const swa_tensor_t* dv, int32_t* status, void* stream) {
  if (int e = check_geom(g)) return e;
  if (int e = check_rope(g, rope)) return e;
  if (int e = check_tensor(q, "q")) return e;
  if (int e = check_tensor(k, "k")) return e;
  if (int e = check_tensor(v, "v")) return e;
  if (int e = check_tensor(d_o, "do")) return e;
  if (int e = check_tensor(dk, "dk")) return e;
  if (int e = check_tensor(dv, "dv")) return e;
  if (!lse || !delta) return fail(E_NULL, "lse/delta is NULL");
  const swa_tensor_t* ts[] = {q, k, v, d_o, dk, dv};
  const int impl = resolve_impl(g, rope, ts, 6, 2);
  if (impl < 0) return impl;
  cudaStream_t st = (cudaStream_t)stream;
  if (impl == SWA_IMPL_TC) {
    int e = swa::tc::launch_dkdv(g, rope, q, k, v, d_o, lse, delta, dk, dv, status, st);
    if (e) return fail(E_LAUNCH, "tcgen05 dkdv: %s", swa::tc::last_error());
    return launch_ok("tcgen05 dkdv");
  }
  const swa::Geom gg = swa::make_geom(g);
  const swa::RopeDev rp = swa::make_rope(rope);
  const int N = g->t_height * g->t_width * g->b_size;
  dim3 grid((N + 7) / 8, g->B * g->H), block(256);
  SWA_DISPATCH_DTYPE(g->dtype, swa::simt_dkdv_kernel<T><<<grid, block, 0, st>>>(
                                   gg, rp, swa::make_view(q), swa::make_view(k), swa::make_view(v),
                                   swa::make_view(d_o), lse, delta, swa::make_view(dk), swa::make_view(dv)));
  return launch_ok("simt dkdv");
}

// ---- rotation handed on between the kernels ---------------------------------------------------
namespace {

// y = rope(x) (inverse: the transposed rotation) for a strided [B, H, N, C] tensor; x == y rotates in place.
int launch_rope4(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* x, const swa_tensor_t* y, bool inverse,
                 cudaStream_t st) {
  const swa::RopeDev rp = swa::make_rope(rope);
  const int64_t N = (int64_t)g->t_height * g->t_width * g->b_size;
  const int64_t rows = N * g->B * g->H;
  const int C = g->d_qk;
  const float sign = inverse ? -1.f : 1.f;
  auto rows16 = [](const swa_tensor_t* t) {
    return t->stride[3] == 1 && ((uintptr_t)t->ptr % 16) == 0 && t->stride[0] % 8 == 0 && t->stride[1] % 8 == 0 &&
           t->stride[2] % 8 == 0;
  };
  const bool vec = g->dtype != SWA_F32 && x->ptr != y->ptr && rp.R % 8 == 0 && C % 8 == 0 && rows16(x) && rows16(y) &&
                   ((uintptr_t)rp.row_cs % 16) == 0 && ((uintptr_t)rp.col_cs % 16) == 0;
  if (vec) {
    const int64_t slots = rp.R / 4 + ((C / 8 - rp.R / 2) + 1) / 2;   // per token row (see the kernel)
    dim3 grid((unsigned)((N * slots + 255) / 256), (unsigned)(g->B * g->H));
    if (g->dtype == SWA_F16)
      swa::rope2d_copy4_kernel<__half><<<grid, 256, 0, st>>>(swa::make_view(x), swa::make_view(y), g->H, (int)N, C, rp, sign);
    else
      swa::rope2d_copy4_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(swa::make_view(x), swa::make_view(y), g->H, (int)N, C, rp, sign);
  } else {
    const int64_t threads = rows * 2 * rp.R;
    const unsigned blocks = (unsigned)((threads + 255) / 256);
    SWA_DISPATCH_DTYPE(g->dtype, swa::rope2d_generic4_kernel<T><<<blocks, 256, 0, st>>>(swa::make_view(x), swa::make_view(y),
                                                                                      rows, g->H, N, C, rp, sign));
  }
  return launch_ok("rope2d (4-D)");
}

int require_rope(const swa_rope_t* rope, const char* who) {
  if (!rope || !rope->idx) return fail(E_ROPE, "%s needs a RoPE description (idx and tables); without RoPE use the plain entry point", who);
  return 0;
}

}  // namespace

int swa_fwd_rot(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q, const swa_tensor_t* k,
                const swa_tensor_t* v, const swa_tensor_t* o, float* lse, const swa_tensor_t* q_rot,
                const swa_tensor_t* k_rot, int32_t* status, void* stream) {
  if (int e = check_geom(g)) return e;
  if (int e = require_rope(rope, "swa_fwd_rot")) return e;
  if (int e = check_rope(g, rope)) return e;
  if (int e = check_tensor(q, "q")) return e;
  if (int e = check_tensor(k, "k")) return e;
  if (int e = check_tensor(v, "v")) return e;
  if (int e = check_tensor(o, "o")) return e;
  if (int e = check_tensor(q_rot, "q_rot")) return e;
  if (int e = check_tensor(k_rot, "k_rot")) return e;
  if (!lse) return fail(E_NULL, "lse is NULL");
  if (q_rot->ptr == q->ptr || k_rot->ptr == k->ptr) return fail(E_SHAPE, "q_rot / k_rot must not alias q / k");
  const swa_tensor_t* ts[] = {q, k, v, o, q_rot, k_rot};
  const int impl = resolve_impl(g, rope, ts, 6, 0, true);
  if (impl < 0) return impl;
  cudaStream_t st = (cudaStream_t)stream;
  // every q and k row is rotated exactly once, by a streaming pass; the attention kernels read the rotated rows
  if (int e = launch_rope4(g, rope, q, q_rot, false, st)) return e;
  if (int e = launch_rope4(g, rope, k, k_rot, false, st)) return e;
  if (impl == SWA_IMPL_TC) {
    int e = swa::tc::launch_fwd2(g, q_rot, k_rot, v, o, lse, status, st);
    if (e) return fail(E_LAUNCH, "tcgen05 forward: %s", swa::tc::last_error());
    return launch_ok("tcgen05 forward (rotation handed on)");
  }
  const swa::Geom gg = swa::make_geom(g);
  const swa::RopeDev none = swa::make_rope(nullptr);
  const int N = g->t_height * g->t_width * g->b_size;
  dim3 grid((N + 7) / 8, g->B * g->H), block(256);
  SWA_DISPATCH_DTYPE(g->dtype, swa::simt_fwd_kernel<T><<<grid, block, 0, st>>>(
                                   gg, none, swa::make_view(q_rot), swa::make_view(k_rot), swa::make_view(v),
                                   swa::make_view(o), lse));
  return launch_ok("simt forward");
}

int swa_bwd_dq_rot(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q_rot, const swa_tensor_t* k_rot,
                   const swa_tensor_t* v, const swa_tensor_t* d_o, const float* lse, const float* delta,
                   const swa_tensor_t* dq, int32_t* status, void* stream) {
  if (int e = check_geom(g)) return e;
  if (int e = require_rope(rope, "swa_bwd_dq_rot")) return e;
  if (int e = check_rope(g, rope)) return e;
  if (int e = check_tensor(q_rot, "q_rot")) return e;
  if (int e = check_tensor(k_rot, "k_rot")) return e;
  if (int e = check_tensor(v, "v")) return e;
  if (int e = check_tensor(d_o, "do")) return e;
  if (int e = check_tensor(dq, "dq")) return e;
  if (!lse || !delta) return fail(E_NULL, "lse/delta is NULL");
  const swa_tensor_t* ts[] = {q_rot, k_rot, v, d_o, dq};
  const int impl = resolve_impl(g, rope, ts, 5, 1, true);
  if (impl < 0) return impl;
  cudaStream_t st = (cudaStream_t)stream;
  if (impl == SWA_IMPL_TC) {
    int e = swa::tc::launch_dq(g, rope, q_rot, k_rot, v, d_o, lse, delta, dq, status, st, true);
    if (e) return fail(E_LAUNCH, "tcgen05 dq: %s", swa::tc::last_error());
    return launch_ok("tcgen05 dq (inputs rotated)");
  }
  const swa::Geom gg = swa::make_geom(g);
  const swa::RopeDev none = swa::make_rope(nullptr);
  const int N = g->t_height * g->t_width * g->b_size;
  dim3 grid((N + 7) / 8, g->B * g->H), block(256);
  SWA_DISPATCH_DTYPE(g->dtype, swa::simt_dq_kernel<T><<<grid, block, 0, st>>>(
                                   gg, none, swa::make_view(q_rot), swa::make_view(k_rot), swa::make_view(v),
                                   swa::make_view(d_o), lse, delta, swa::make_view(dq)));
  if (int e = launch_ok("simt dq")) return e;
  return launch_rope4(g, rope, dq, dq, true, st);
}

int swa_bwd_dkdv_rot(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q_rot, const swa_tensor_t* k_rot,
                     const swa_tensor_t* v, const swa_tensor_t* d_o, const float* lse, const float* delta,
                     const swa_tensor_t* dk, const swa_tensor_t* dv, int32_t* status, void* stream) {
  if (int e = check_geom(g)) return e;
  if (int e = require_rope(rope, "swa_bwd_dkdv_rot")) return e;
  if (int e = check_rope(g, rope)) return e;
  if (int e = check_tensor(q_rot, "q_rot")) return e;
  if (int e = check_tensor(k_rot, "k_rot")) return e;
  if (int e = check_tensor(v, "v")) return e;
  if (int e = check_tensor(d_o, "do")) return e;
  if (int e = check_tensor(dk, "dk")) return e;
  if (int e = check_tensor(dv, "dv")) return e;
  if (!lse || !delta) return fail(E_NULL, "lse/delta is NULL");
  const swa_tensor_t* ts[] = {q_rot, k_rot, v, d_o, dk, dv};
  const int impl = resolve_impl(g, rope, ts, 6, 2, true);
  if (impl < 0) return impl;
  cudaStream_t st = (cudaStream_t)stream;
  if (impl == SWA_IMPL_TC) {
    int e = swa::tc::launch_dkdv(g, rope, q_rot, k_rot, v, d_o, lse, delta, dk, dv, status, st, true);
    if (e) return fail(E_LAUNCH, "tcgen05 dkdv: %s", swa::tc::last_error());
    return launch_ok("tcgen05 dkdv (inputs rotated)");
  }
  const swa::Geom gg = swa::make_geom(g);
  const swa::RopeDev none = swa::make_rope(nullptr);
  const int N = g->t_height * g->t_width * g->b_size;
  dim3 grid((N + 7) / 8, g->B * g->H), block(256);
  SWA_DISPATCH_DTYPE(g->dtype, swa::simt_dkdv_kernel<T><<<grid, block, 0, st>>>(
                                   gg, none, swa::make_view(q_rot), swa::make_view(k_rot), swa::make_view(v),
                                   swa::make_view(d_o), lse, delta, swa::make_view(dk), swa::make_view(dv)));
  if (int e = launch_ok("simt dkdv")) return e;
  return launch_rope4(g, rope, dk, dk, true, st);
}

// ---- backward without allocation ------------------------------------------------------------
// Scratch for the softmax delta of swa_bwd_noalloc.  In host code this name is only a handle of
// the symbol, not a device address: the address is looked up once per device below.
static __device__ __align__(256) float g_noalloc_delta[SWA_NOALLOC_MAX_ROWS];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mu;
float* g_noalloc_ptr[kMaxDevices] = {};

// Device address of g_noalloc_delta on the current device (set-up on first use, no allocation).
int noalloc_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(E_LAUNCH, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(E_SHAPE, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_delta);
    if (e != cudaSuccess || p == nullptr)
      return fail(E_LAUNCH, "cudaGetSymbolAddress(delta scratch) on device %d: %s", dev, cudaGetErrorString(e));
    g_noalloc_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}
}  // namespace

int swa_bwd_noalloc(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q, const swa_tensor_t* k,
                    const swa_tensor_t* v, const swa_tensor_t* o, const swa_tensor_t* d_o, const float* lse,
                    const swa_tensor_t* dq, const swa_tensor_t* dk, const swa_tensor_t* dv, int32_t* status,
                    void* stream) {
  if (int e = check_geom(g)) return e;
  const int64_t rows = (int64_t)g->B * g->H * g->t_height * g->t_width * g->b_size;
  if (rows > (int64_t)SWA_NOALLOC_MAX_ROWS)
    return fail(E_SHAPE, "swa_bwd_noalloc: B*H*N = %lld exceeds the built-in scratch of %d rows; use swa_bwd_delta/"
                "swa_bwd_dq/swa_bwd_dkdv with a caller-provided delta buffer", (long long)rows, SWA_NOALLOC_MAX_ROWS);
  // every rejection the three launches below could raise is raised here, before the first of them
  if (int e = check_rope(g, rope)) return e;
  if (int e = check_tensor(q, "q")) return e;
  if (int e = check_tensor(k, "k")) return e;
  if (int e = check_tensor(v, "v")) return e;
  if (int e = check_tensor(o, "o")) return e;
  if (int e = check_tensor(d_o, "do")) return e;
  if (int e = check_tensor(dq, "dq")) return e;
  if (int e = check_tensor(dk, "dk")) return e;
  if (int e = check_tensor(dv, "dv")) return e;
  if (!lse) return fail(E_NULL, "lse is NULL");
  {
    const swa_tensor_t* t1[] = {q, k, v, d_o, dq};
    const swa_tensor_t* t2[] = {q, k, v, d_o, dk, dv};
    if (int e = resolve_impl(g, rope, t1, 5, 1); e < 0) return e;
    if (int e = resolve_impl(g, rope, t2, 6, 2); e < 0) return e;
  }
  float* delta = nullptr;
  if (int e = noalloc_scratch(&delta)) return e;
  if (int e = swa_bwd_delta(g, o, d_o, delta, stream)) return e;
  if (int e = swa_bwd_dq(g, rope, q, k, v, d_o, lse, delta, dq, status, stream)) return e;
  return swa_bwd_dkdv(g, rope, q, k, v, d_o, lse, delta, dk, dv, status, stream);
}

int rope2d_apply(int32_t dtype, void* x, int64_t batch, int64_t n_tokens, int32_t n_dim, const int64_t* xs,
                 const swa_rope_t* rope, int32_t inverse, void* stream) {
  if (dtype < SWA_F32 || dtype > SWA_BF16) return fail(E_DTYPE, "unknown dtype %d", dtype);
  if (!x || !xs) return fail(E_NULL, "x / strides are NULL");
  if (!rope || !rope->idx || !rope->row_cs || !rope->col_cs) return fail(E_ROPE, "rope index / tables are NULL");
  if (rope->n_rdim <= 0 || 4 * rope->n_rdim > n_dim)
    return fail(E_ROPE, "4*n_rdim (%d) must be in [4, n_dim=%d]", 4 * rope->n_rdim, n_dim);
  if (rope->max_h <= 0 || rope->max_w <= 0) return fail(E_ROPE, "rope table lengths must be positive");
  if (batch <= 0 || n_tokens <= 0) return fail(E_SHAPE, "batch and n_tokens must be positive");
  if (batch > 65535) return fail(E_SHAPE, "batch exceeds 65535");
  cudaStream_t st = (cudaStream_t)stream;
  const swa::RopeDev rp = swa::make_rope(rope);
  const float sign = inverse ? -1.f : 1.f;
  const int esz = dtype == SWA_F32 ? 4 : 2;
  const int vec = 16 / esz;
  const bool vec_ok = xs[2] == 1 && rp.R % vec == 0 && ((uintptr_t)x % 16) == 0 && (xs[0] * esz) % 16 == 0 &&
                      (xs[1] * esz) % 16 == 0 && ((uintptr_t)rp.row_cs % 16) == 0 && ((uintptr_t)rp.col_cs % 16) == 0;
  const int per_tok = 2 * (vec_ok ? rp.R / vec : rp.R);
  const int64_t items = n_tokens * per_tok;
  dim3 grid((unsigned)((items + 255) / 256), (unsigned)batch), block(256);
  if (vec_ok) {
    if (dtype == SWA_F32)
      swa::rope2d_kernel<float, 4><<<grid, block, 0, st>>>((float*)x, batch, n_tokens, xs[0], xs[1], xs[2], rp, sign);
    else if (dtype == SWA_F16)
      swa::rope2d_kernel<__half, 8><<<grid, block, 0, st>>>((__half*)x, batch, n_tokens, xs[0], xs[1], xs[2], rp, sign);
    else
      swa::rope2d_kernel<__nv_bfloat16, 8><<<grid, block, 0, st>>>((__nv_bfloat16*)x, batch, n_tokens, xs[0], xs[1],
                                                                   xs[2], rp, sign);
  } else {
    SWA_DISPATCH_DTYPE(dtype, swa::rope2d_kernel<T, 1><<<grid, block, 0, st>>>((T*)x, batch, n_tokens, xs[0], xs[1],
                                                                              xs[2], rp, sign));
  }
  return launch_ok("rope2d");
}

int rope2d_apply_to(int32_t dtype, const void* x, void* y, int64_t batch, int64_t n_tokens, int32_t n_dim,
                    const int64_t* xs, const int64_t* ys, const swa_rope_t* rope, int32_t inverse, void* stream) {
  if (dtype != SWA_F16 && dtype != SWA_BF16) return fail(E_DTYPE, "rope2d_apply_to takes fp16 / bf16 (dtype %d)", dtype);
  if (!x || !y || !xs || !ys) return fail(E_NULL, "x / y / strides are NULL");
  if (x == y) return fail(E_SHAPE, "rope2d_apply_to is out of place; use rope2d_apply for x == y");
  if (!rope || !rope->idx || !rope->row_cs || !rope->col_cs) return fail(E_ROPE, "rope index / tables are NULL");
  if (rope->n_rdim <= 0 || 4 * rope->n_rdim > n_dim)
    return fail(E_ROPE, "4*n_rdim (%d) must be in [4, n_dim=%d]", 4 * rope->n_rdim, n_dim);
  if (rope->max_h <= 0 || rope->max_w <= 0) return fail(E_ROPE, "rope table lengths must be positive");
  if (batch <= 0 || n_tokens <= 0) return fail(E_SHAPE, "batch and n_tokens must be positive");
  const swa::RopeDev rp = swa::make_rope(rope);
  auto rows16 = [](const void* p, const int64_t* st) {
    return st[2] == 1 && ((uintptr_t)p % 16) == 0 && st[0] % 8 == 0 && st[1] % 8 == 0;
  };
  if (rp.R % 8 || n_dim % 8 || !rows16(x, xs) || !rows16(y, ys) || ((uintptr_t)rp.row_cs % 16) || ((uintptr_t)rp.col_cs % 16))
    return fail(E_SHAPE, "rope2d_apply_to needs n_rdim %% 8 == 0, n_dim %% 8 == 0, unit last strides and 16-byte aligned rows");
  const int64_t rows = batch * n_tokens, threads = rows * (n_dim / 8);
  const unsigned blocks = (unsigned)((threads + 255) / 256);
  const float sign = inverse ? -1.f : 1.f;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == SWA_F16)
    swa::rope2d_copy_kernel<__half><<<blocks, 256, 0, st>>>((const __half*)x, (__half*)y, rows, n_tokens, n_dim, xs[0], xs[1],
                                                            ys[0], ys[1], rp, sign);
  else
    swa::rope2d_copy_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, rows, n_tokens,
                                                                   n_dim, xs[0], xs[1], ys[0], ys[1], rp, sign);
  return launch_ok("rope2d_copy");
}

}  // extern "C"
