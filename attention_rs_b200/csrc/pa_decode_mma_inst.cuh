// Launcher of the tensor-core decode kernel family for one (query dtype, cache
// kind); included by one small translation unit per combination so the
// instantiations compile in parallel.
#pragma once

#include "pa_decode_mma.cuh"
#include "pa_launch.h"

namespace pa {

template <typename T, bool FP8, int HEAD, int BS, int NH>
int launch_decode_mma_nh(const DecodeParams& p, cudaStream_t stream) {
  using C = DecodeCfg<T, FP8, HEAD, BS, NH>;
  auto kernel = paged_decode_mma_kernel<T, FP8, HEAD, BS, NH>;
  // Opt in to the large dynamic shared-memory carve-out once per device instead
  // of on every call (the reference sets it per call, src/kernels/src/pagedattention.cu:570-573).
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return PA_ERR_CUDA;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess)
      return PA_ERR_CUDA;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int gsplit = (p.group + 8 * NH - 1) / (8 * NH);
  const bool partitioned = p.partition_size > 0;
  const int csize = partitioned ? 1 : (p.cluster < 1 ? 1 : p.cluster);
  const int ppc = p.parts_per_cta < 1 ? 1 : p.parts_per_cta;
  dim3 grid(p.num_kv_heads * gsplit, p.num_seqs, partitioned ? (p.max_parts + ppc - 1) / ppc : csize);
  if (csize > 1) {
    // Single pass over a long context: a thread-block cluster splits it and merges through distributed
    // shared memory, so no scratch buffer and no second launch are needed.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(C::THREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = csize;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return PA_ERR_CUDA;
    return PA_OK;
  }
  kernel<<<grid, C::THREADS, C::SMEM_BYTES, stream>>>(p);
  if (partitioned) {
    // The merge is launched as a programmatic dependent: it may be scheduled while the partition grid
    // drains and waits (griddepcontrol.wait) until that grid's memory is visible.
    const bool many = p.max_parts > 64;            // long contexts: sixteen warps share the loop over partitions
    const int nwarp = many ? 16 : 4;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.num_heads, p.num_seqs);
    cfg.blockDim = dim3(nwarp * 32);
    cfg.dynamicSmemBytes = (static_cast<size_t>(p.max_parts) + nwarp * HEAD) * sizeof(float);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    auto kernel = many ? paged_decode_merge_kernel<T, HEAD, 16> : paged_decode_merge_kernel<T, HEAD, 4>;
    if (cudaLaunchKernelEx(&cfg, kernel, reinterpret_cast<T*>(p.out), static_cast<const float*>(p.exp_sums),
                           static_cast<const float*>(p.max_logits), reinterpret_cast<const T*>(p.tmp_out), p.context_lens,
                           p.max_parts, p.partition_size) != cudaSuccess)
      return PA_ERR_CUDA;
  }
  return cudaGetLastError() == cudaSuccess ? PA_OK : PA_ERR_CUDA;
}

// Groups of up to 8 query heads per kv head take one n-tile of heads per CTA, larger groups two.
template <typename T, bool FP8, int HEAD, int BS>
int launch_decode_mma_one(const DecodeParams& p, cudaStream_t stream) {
  return p.group <= 8 ? launch_decode_mma_nh<T, FP8, HEAD, BS, 1>(p, stream)
                      : launch_decode_mma_nh<T, FP8, HEAD, BS, 2>(p, stream);
}

template <typename T, bool FP8, int HEAD>
int launch_decode_mma_head(const DecodeParams& p, int block_size, cudaStream_t stream) {
  switch (block_size) {
    case 16: return launch_decode_mma_one<T, FP8, HEAD, 16>(p, stream);
    case 32: return launch_decode_mma_one<T, FP8, HEAD, 32>(p, stream);
    case 8:
      if constexpr (!FP8) return launch_decode_mma_one<T, FP8, HEAD, 8>(p, stream);
      return PA_ERR_UNSUPPORTED;
    default: return PA_ERR_UNSUPPORTED;
  }
}

// Head sizes are the reference's list (src/paged_attention.rs:108-117,
// src/kernels/src/pagedattention.cu:635-662); the FP8 path takes those that are
// multiples of 32.
template <typename T, bool FP8>
int launch_decode_mma_impl(const DecodeParams& p, int head_size, int block_size, cudaStream_t stream) {
#ifdef PA_ONLY_HEAD128  // tuning builds: one head size, to keep variant libraries small
  if (head_size != 128) return PA_ERR_UNSUPPORTED;
  return launch_decode_mma_head<T, FP8, 128>(p, block_size, stream);
#else
  switch (head_size) {
    case 64: return launch_decode_mma_head<T, FP8, 64>(p, block_size, stream);
    case 96: return launch_decode_mma_head<T, FP8, 96>(p, block_size, stream);
    case 128: return launch_decode_mma_head<T, FP8, 128>(p, block_size, stream);
    case 192: return launch_decode_mma_head<T, FP8, 192>(p, block_size, stream);
    case 256: return launch_decode_mma_head<T, FP8, 256>(p, block_size, stream);
    case 80:
      if constexpr (!FP8) return launch_decode_mma_head<T, FP8, 80>(p, block_size, stream);
      return PA_ERR_UNSUPPORTED;
    case 112:
      if constexpr (!FP8) return launch_decode_mma_head<T, FP8, 112>(p, block_size, stream);
      return PA_ERR_UNSUPPORTED;
    default: return PA_ERR_UNSUPPORTED;
  }
#endif
}

}  // namespace pa
