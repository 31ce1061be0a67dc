// Tensor-core decode kernels: query dtype __half, FP8 E4M3 cache.
#include "pa_decode_mma_inst.cuh"

namespace pa {
int launch_decode_mma_f16_fp8(const DecodeParams& p, int head_size, int block_size, cudaStream_t stream) {
  return launch_decode_mma_impl<__half, true>(p, head_size, block_size, stream);
}
}  // namespace pa
