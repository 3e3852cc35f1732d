// tcgen05 (5th-generation tensor core) kernels: interface used by the C ABI.
#pragma once

#include "common.cuh"

namespace swa {
namespace tc {

// nullptr when the tensor-core kernels cover this call, else the reason they do not.
// `which`: 0 forward, 1 dQ, 2 dK/dV.  `tensors` may be null (shape-only query).
const char* unsupported_reason(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* const* tensors,
                               int n_tensors, int which);
const char* last_error();

int launch_fwd(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q, const swa_tensor_t* k,
               const swa_tensor_t* v, const swa_tensor_t* o, float* lse, int32_t* status, cudaStream_t st);
int launch_dq(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q, const swa_tensor_t* k,
              const swa_tensor_t* v, const swa_tensor_t* d_o, const float* lse, const float* delta,
              const swa_tensor_t* dq, int32_t* status, cudaStream_t st);
int launch_dkdv(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q, const swa_tensor_t* k,
                const swa_tensor_t* v, const swa_tensor_t* d_o, const float* lse, const float* delta,
                const swa_tensor_t* dk, const swa_tensor_t* dv, int32_t* status, cudaStream_t st);

}  // namespace tc
}  // namespace swa
