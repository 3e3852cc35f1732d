// placeholder until the tcgen05 kernels land
#include "swa_tc.cuh"
namespace swa { namespace tc {
const char* unsupported_reason(const swa_geom_t*, const swa_rope_t*, const swa_tensor_t* const*, int, int) { return "tensor-core kernels not built"; }
const char* last_error() { return ""; }
int launch_fwd(const swa_geom_t*, const swa_rope_t*, const swa_tensor_t*, const swa_tensor_t*, const swa_tensor_t*, const swa_tensor_t*, float*, int32_t*, cudaStream_t) { return -1; }
int launch_dq(const swa_geom_t*, const swa_rope_t*, const swa_tensor_t*, const swa_tensor_t*, const swa_tensor_t*, const swa_tensor_t*, const float*, const float*, const swa_tensor_t*, int32_t*, cudaStream_t) { return -1; }
int launch_dkdv(const swa_geom_t*, const swa_rope_t*, const swa_tensor_t*, const swa_tensor_t*, const swa_tensor_t*, const swa_tensor_t*, const float*, const float*, const swa_tensor_t*, const swa_tensor_t*, int32_t*, cudaStream_t) { return -1; }
}}
