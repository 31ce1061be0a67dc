// Tensor-core decode kernels: query dtype __nv_bfloat16, cache of the same dtype.
#include "pa_decode_mma_inst.cuh"

namespace pa {
int launch_decode_mma_bf16(const DecodeParams& p, int head_size, int block_size, cudaStream_t stream) {
  return launch_decode_mma_impl<__nv_bfloat16, false>(p, head_size, block_size, stream);
}
}  // namespace pa
