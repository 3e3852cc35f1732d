/*
 * swa2d.h -- C ABI of the B200 (sm_100a) tiled 2D sliding-window attention library.
 *
 * The library is the device side of the call surface of the reference project's
 * src/tiled_swa.py and src/fused_rope2d.py.  Each entry point below replaces one
 * Triton launch site of the reference; the Python classes of the same names
 * (TiledSwa, RotaryPE2D, ...) in dl_templates_b200/ bind these with ctypes.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer of the current CUDA device; the caller
 *     owns all memory, the library allocates no device memory;
 *   - tensors are described by a pointer and four ELEMENT strides, shape
 *     [B, H, N, d] with N = t_height * t_width * b_size and token
 *     n = (tile_row * t_width + tile_col) * b_size + s   (src/tiled_swa.py:104,216);
 *   - work is enqueued on `stream` and the call returns without synchronising;
 *   - return value 0 = enqueued; negative = argument rejected before any launch
 *     (swa_last_error() returns the message for the calling thread);
 *   - `status` is an optional device int32[4] word the tensor-core kernels write
 *     to when one of their bounded waits gives up (0 = ok); may be NULL;
 *   - lse is the base-2 logsumexp of (sm_scale * log2(e) * q.k) over the window,
 *     fp32 [B,H,N] contiguous (the reference keeps the same quantity in fp16,
 *     src/tiled_swa.py:35,129).
 */
#ifndef SWA2D_H_
#define SWA2D_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { SWA_F32 = 0, SWA_F16 = 1, SWA_BF16 = 2 } swa_dtype_t;

/* which implementation a call may use */
typedef enum {
  SWA_IMPL_AUTO = 0,  /* tensor-core kernels when the shape qualifies, else the SIMT kernels */
  SWA_IMPL_SIMT = 1,  /* fp32-accumulate CUDA-core kernels (every dtype, every shape)        */
  SWA_IMPL_TC   = 2   /* tcgen05 kernels only; shapes they do not cover are rejected          */
} swa_impl_t;

typedef struct {
  void*   ptr;
  int64_t stride[4]; /* element strides of [B, H, N, d] */
} swa_tensor_t;

/* Geometry shared by all attention entry points (argument order of
 * TiledSwa.forward, src/tiled_swa.py:604). */
typedef struct {
  int32_t dtype;      /* swa_dtype_t of q, k, v, o, do, dq, dk, dv */
  int32_t B, H;
  int32_t b_size;     /* tokens per grid cell ("tile")                       */
  int32_t t_height, t_width;
  int32_t row_size, col_size; /* window half-extent in tiles; truncated at the border */
  int32_t d_qk, d_v;  /* any size on the SIMT kernels; the tensor-core kernels take 32, 64, 96, 128
                         (64, 128 where an entry rotates the rows it streams: swa_fwd, swa_bwd_dq,
                         swa_bwd_dkdv with rope != NULL) */
  float   sm_scale;
  int32_t impl;       /* swa_impl_t */
} swa_geom_t;

/* Optional fused RoPE-2D (src/fused_rope2d.py:204-225 semantics).  idx == NULL
 * disables it.  idx[n] = (row << 16) | col, each half an int16, a negative half
 * leaves that half of the token un-rotated.  Tables are fp32 [max, n_rdim, 2]
 * (cos, sin) contiguous.  Only the first 4*n_rdim dims of q/k are rotated. */
typedef struct {
  const int32_t* idx;     /* [N] */
  const float*   row_cs;  /* [max_h, n_rdim, 2] */
  const float*   col_cs;  /* [max_w, n_rdim, 2] */
  int32_t n_rdim, max_h, max_w;
} swa_rope_t;

/* Forward: o = softmax(sm_scale * rope(q) rope(k)^T + window mask) v, and lse.
 * Replaces the tiled_swa_fwd_kernel / tiled_swa_fwd_large_kernel launches of
 * TiledSwa.forward (src/tiled_swa.py:611-637); with rope != NULL also the two
 * rope2d_fwd_kernel launches on q and k that precede it (src/fused_rope2d.py:138). */
int swa_fwd(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q, const swa_tensor_t* k,
            const swa_tensor_t* v, const swa_tensor_t* o, float* lse, int32_t* status, void* stream);

/* delta[b,h,n] = sum_d o*do (fp32).  Replaces tiled_swa_bwd_preprocess_kernel
 * (src/tiled_swa.py:253-282, launch at :666). */
int swa_bwd_delta(const swa_geom_t* g, const swa_tensor_t* o, const swa_tensor_t* d_o, float* delta, void* stream);

/* dq (gradient of the UN-rotated q when rope != NULL).  Replaces phase 2 of
 * tiled_swa_bwd_large_kernel_decoupled_q (src/tiled_swa.py:520-562) plus the
 * rope2d_bwd_kernel launch on dq (src/fused_rope2d.py:163). */
int swa_bwd_dq(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q, const swa_tensor_t* k,
               const swa_tensor_t* v, const swa_tensor_t* d_o, const float* lse, const float* delta,
               const swa_tensor_t* dq, int32_t* status, void* stream);

/* dk (of the UN-rotated k) and dv.  Replaces phase 1 of
 * tiled_swa_bwd_large_kernel_decoupled_q (src/tiled_swa.py:475-518) plus the
 * rope2d_bwd_kernel launch on dk. */
int swa_bwd_dkdv(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q, const swa_tensor_t* k,
                 const swa_tensor_t* v, const swa_tensor_t* d_o, const float* lse, const float* delta,
                 const swa_tensor_t* dk, const swa_tensor_t* dv, int32_t* status, void* stream);

/* The same three steps with the rotation handed on from kernel to kernel, so that every q and k row is rotated
 * exactly once (swa_fwd / swa_bwd_* with rope != NULL rotate a streamed row once per tile whose window holds
 * it).  q_rot and k_rot are caller-provided tensors of the shapes of q and k; q and k stay untouched.
 *   swa_fwd_rot     - one streaming pass each writes rope(q) to q_rot and rope(k) to k_rot (clone + rotate, every
 *                     byte moved once), then the attention kernel runs on the rotated copies with no rotation
 *                     work of its own.  Same o and lse as swa_fwd(rope).  Replaces the same launches as swa_fwd (two
 *                     rope2d_fwd_kernel launches, src/fused_rope2d.py:138, and the forward kernel,
 *                     src/tiled_swa.py:611-637); what the reference leaves behind by rotating q and k in place
 *                     (src/fused_rope2d.py:143-145) is what q_rot / k_rot hold here.
 *   swa_bwd_dq_rot, swa_bwd_dkdv_rot - take q_rot / k_rot where swa_bwd_dq / swa_bwd_dkdv take q / k; no row
 *                     is rotated before the MMAs, dq / dk are rotated back in the epilogue registers, i.e. they
 *                     are the gradients of the UN-rotated q and k (the rope2d_bwd_kernel launches,
 *                     src/fused_rope2d.py:163, stay fused).  delta comes from swa_bwd_delta as before.
 * rope must not be NULL (without RoPE the plain entry points do the same work). */
int swa_fwd_rot(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q, const swa_tensor_t* k,
                const swa_tensor_t* v, const swa_tensor_t* o, float* lse, const swa_tensor_t* q_rot,
                const swa_tensor_t* k_rot, int32_t* status, void* stream);
int swa_bwd_dq_rot(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q_rot, const swa_tensor_t* k_rot,
                   const swa_tensor_t* v, const swa_tensor_t* d_o, const float* lse, const float* delta,
                   const swa_tensor_t* dq, int32_t* status, void* stream);
int swa_bwd_dkdv_rot(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q_rot, const swa_tensor_t* k_rot,
                     const swa_tensor_t* v, const swa_tensor_t* d_o, const float* lse, const float* delta,
                     const swa_tensor_t* dk, const swa_tensor_t* dv, int32_t* status, void* stream);

/* Stand-alone in-place RoPE-2D on x [batch, N, C] (element strides xs[3]).
 * inverse = 0 replaces rope2d_fwd_kernel (src/fused_rope2d.py:24-72), inverse = 1
 * replaces rope2d_bwd_kernel (src/fused_rope2d.py:74-122).  A negative index half
 * means identity for that half, as rope2d_ref defines it (src/fused_rope2d.py:215-219). */
int rope2d_apply(int32_t dtype, void* x, int64_t batch, int64_t n_tokens, int32_t n_dim, const int64_t* xs,
                 const swa_rope_t* rope, int32_t inverse, void* stream);

/* Out-of-place form for fp16 / bf16: y = rope(x) (or the inverse rotation), x untouched, dims beyond 4*n_rdim and
 * tokens with a negative index half copied.  The reference's RotaryPE2D rotates in place and its backward clones
 * the incoming gradient first (src/fused_rope2d.py:143,151); this entry does clone + rotate in one pass.
 * Needs n_rdim % 8 == 0, n_dim % 8 == 0, unit last strides and 16-byte aligned rows (negative return otherwise:
 * copy, then rope2d_apply). */
int rope2d_apply_to(int32_t dtype, const void* x, void* y, int64_t batch, int64_t n_tokens, int32_t n_dim,
                    const int64_t* xs, const int64_t* ys, const swa_rope_t* rope, int32_t inverse, void* stream);

/* Whole backward pass (delta, then dq, then dk/dv) for callers that must not allocate.
 * This entry point has no counterpart in the reference; it exists for hosts that cannot call
 * cudaMalloc around the op: a plugin running inside a runtime that has already handed all device
 * memory to its own arena, a serving loop that may not take the device-wide synchronisation an
 * allocation implies, or a caller that simply owns no allocator handle.  The backward pass
 * needs one scratch vector, delta[B*H*N] in fp32; the other entry points take it from the
 * caller, this one keeps it in a fixed array inside the library image, so
 *   - B*H*N may not exceed SWA_NOALLOC_MAX_ROWS (the call is rejected with an error otherwise);
 *   - every GPU that loads the library holds that array (SWA_NOALLOC_MAX_ROWS * 4 bytes) until
 *     the process exits, whether or not this entry point is ever used;
 *   - all calls on a device share the array: two calls whose kernels may overlap on the GPU
 *     (different streams, no dependency between them) race on it -- serialise them.  Nothing
 *     in it has to start at zero: each call overwrites the rows it then reads;
 *   - the first call on a device looks up the array's device address (no allocation); make that
 *     first call before starting any stream capture on that device.
 * The caller passes every input and every output (dq, dk, dv); nothing is allocated or freed.
 * Results are identical to swa_bwd_delta + swa_bwd_dq + swa_bwd_dkdv on the same arguments. */
#define SWA_NOALLOC_MAX_ROWS (1 << 21)
int swa_bwd_noalloc(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q, const swa_tensor_t* k,
                    const swa_tensor_t* v, const swa_tensor_t* o, const swa_tensor_t* d_o, const float* lse,
                    const swa_tensor_t* dq, const swa_tensor_t* dk, const swa_tensor_t* dv, int32_t* status,
                    void* stream);

/* Which kernel family swa_fwd / swa_bwd_dq / swa_bwd_dkdv would run for this
 * geometry: SWA_IMPL_SIMT or SWA_IMPL_TC (negative = rejected). `which`: 0 fwd, 1 dq, 2 dkdv. */
int swa_select_impl(const swa_geom_t* g, const swa_rope_t* rope, int32_t which);

/* Resource plan of the tensor-core kernel `which` for this geometry (0, 1, 2: what swa_fwd, swa_bwd_dq, swa_bwd_dkdv
 * would launch; 3, 4, 5: what swa_fwd_rot, swa_bwd_dq_rot, swa_bwd_dkdv_rot would launch); host-only, needs no
 * GPU.  A diagnostic without counterpart in the reference: tests use it to check that every plan stays inside
 * 227 KB of shared memory and 512 tensor-memory columns.  out[12] = tile rows, tile columns, block rows, block
 * columns, block tokens N, ring stages, score buffers (fwd) or (S, dP) pairs (bwd), resident-tile buffers,
 * staged cos/sin table bytes, dynamic shared memory requested, shared memory used by the layout (worst-case
 * alignment pad included), tensor-memory columns used.  Negative return: the shape runs on the SIMT kernels. */
int swa_describe_plan(const swa_geom_t* g, const swa_rope_t* rope, int32_t which, int32_t* out);

/* The planner's experiment knobs (environment variables SWA_TC_*) are read once per process and tile plans are
 * cached per geometry; this re-reads the environment and drops the cache.  A diagnostic without counterpart in
 * the reference (its Triton autotuner keeps a comparable per-shape cache, src/tiled_swa.py:135-142); host-only. */
void swa_refresh_env(void);

/* Number of kernel launches this library has enqueued from the calling process. */
int64_t swa_launch_count(void);

/* Message of the last rejected call on this thread ("" if none). */
const char* swa_last_error(void);

/* ABI version of this header. */
int swa_version(void);

#ifdef __cplusplus
}
#endif
#endif /* SWA2D_H_ */
