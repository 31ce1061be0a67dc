// Tensor-core decode kernels: query dtype __nv_bfloat16, FP8 E4M3 cache.
#include "pa_decode_mma_inst.cuh"

namespace pa {
int launch_decode_mma_bf16_fp8(const DecodeParams& p, int head_size, int block_size, cudaStream_t stream) {
  return launch_decode_mma_impl<__nv_bfloat16, true>(p, head_size, block_size, stream);
}
}  // namespace pa
