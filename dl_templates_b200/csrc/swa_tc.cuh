// tcgen05 (5th-generation tensor core) kernels: interface used by the C ABI.
#pragma once

#include "common.cuh"

namespace swa {
namespace tc {

// nullptr when the tensor-core kernels cover this call, else the reason they do not.
// `which`: 0 forward, 1 dQ, 2 dK/dV.  `tensors` may be null (shape-only query).
// `prerotated`: the call hands rotated copies of q / k between the kernels (swa_fwd_rot and the *_rot backward
// entries), so no kernel rotates streamed rows and the plan is the one without RoPE.
const char* unsupported_reason(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* const* tensors,
                               int n_tensors, int which, bool prerotated = false);
const char* last_error();

// Re-read the SWA_TC_* experiment knobs from the environment and drop the cached plans (both are otherwise read /
// computed once per process).
void refresh_env();

// Resource plan the tensor-core kernel `which` would run with (host-only, no GPU needed): out[0..11] =
// TH, TW, KR, KW, N, stages, score buffers (forward) / buffer pairs (backward), resident-tile buffers,
// staged-table bytes, dynamic shared memory requested, shared memory the kernel's layout really uses
// (with the worst-case alignment pad), tensor-memory columns used.  Returns false when no plan fits.
bool describe_plan(const swa_geom_t* g, const swa_rope_t* rope, int which, int32_t* out);

int launch_fwd(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q, const swa_tensor_t* k,
               const swa_tensor_t* v, const swa_tensor_t* o, float* lse, int32_t* status, cudaStream_t st);
// Forward without any rotation in the kernel: q and k are un-rotated inputs of a call without RoPE, or the
// rotated copies a streaming pass made.
int launch_fwd2(const swa_geom_t* g, const swa_tensor_t* q, const swa_tensor_t* k, const swa_tensor_t* v,
                const swa_tensor_t* o, float* lse, int32_t* status, cudaStream_t st);
int launch_dq(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q, const swa_tensor_t* k,
              const swa_tensor_t* v, const swa_tensor_t* d_o, const float* lse, const float* delta,
              const swa_tensor_t* dq, int32_t* status, cudaStream_t st, bool prerotated = false);
int launch_dkdv(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q, const swa_tensor_t* k,
                const swa_tensor_t* v, const swa_tensor_t* d_o, const float* lse, const float* delta,
                const swa_tensor_t* dk, const swa_tensor_t* dv, int32_t* status, cudaStream_t st, bool prerotated = false);

}  // namespace tc
}  // namespace swa
