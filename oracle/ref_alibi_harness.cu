// Test infrastructure only: launches the REFERENCE's own kernel templates with a
// non-null ALiBi slope pointer.
//
// The reference's device code implements the ALiBi bias
// (src/kernels/src/pagedattention.cu:151,235) but its two C entry points pass
// alibi_slopes = nullptr (src/kernels/src/pagedattention.cu:621-622, 795-796), so
// the bias cannot be exercised through the reference's C ABI.  This file includes
// the reference translation unit from where it lies (path given by the build
// recipe as REF_PAGEDATTENTION_CU) and instantiates a few of its templates.
// No reference code is copied here.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include REF_PAGEDATTENTION_CU

namespace {

template <typename T, int HEAD, int BLOCK>
int launch_v2(void* out, float* exp_sums, float* max_logits, void* tmp_out, void* query, void* key_cache,
              void* value_cache, int num_kv_heads, float scale, uint32_t* block_tables, uint32_t* context_lens,
              int max_context_len, int num_seqs, int num_heads, int max_num_blocks_per_seq, int q_stride,
              int kv_block_stride, int kv_head_stride, float softcapping, const float* alibi_slopes,
              cudaStream_t stream) {
  constexpr int THREADS = 128, PART = 512;
  const int max_parts = (max_context_len + PART - 1) / PART;
  const int smem = max(PART * (int)sizeof(float), (THREADS / 32 / 2) * HEAD * (int)sizeof(float));
  dim3 grid(num_heads, num_seqs, max_parts), block(THREADS);
  vllm::paged_attention_v2_kernel<T, HEAD, BLOCK, THREADS, PART><<<grid, block, smem, stream>>>(
      exp_sums, max_logits, reinterpret_cast<T*>(tmp_out), reinterpret_cast<T*>(query),
      reinterpret_cast<T*>(key_cache), reinterpret_cast<T*>(value_cache), num_kv_heads, scale, block_tables,
      context_lens, max_num_blocks_per_seq, alibi_slopes, q_stride, kv_block_stride, kv_head_stride, softcapping);
  dim3 rgrid(num_heads, num_seqs);
  vllm::paged_attention_v2_reduce_kernel<T, HEAD, THREADS, PART><<<rgrid, block, 2 * max_parts * sizeof(float), stream>>>(
      reinterpret_cast<T*>(out), exp_sums, max_logits, reinterpret_cast<T*>(tmp_out), context_lens, max_parts);
  return (int)cudaGetLastError();
}

template <typename T, int HEAD>
int by_block(int block_size, void* out, float* exp_sums, float* max_logits, void* tmp_out, void* query,
             void* key_cache, void* value_cache, int num_kv_heads, float scale, uint32_t* block_tables,
             uint32_t* context_lens, int max_context_len, int num_seqs, int num_heads, int max_num_blocks_per_seq,
             int q_stride, int kv_block_stride, int kv_head_stride, float softcapping, const float* alibi_slopes,
             cudaStream_t stream) {
#define GO(B)                                                                                                   \
  return launch_v2<T, HEAD, B>(out, exp_sums, max_logits, tmp_out, query, key_cache, value_cache, num_kv_heads,  \
                               scale, block_tables, context_lens, max_context_len, num_seqs, num_heads,          \
                               max_num_blocks_per_seq, q_stride, kv_block_stride, kv_head_stride, softcapping,   \
                               alibi_slopes, stream)
  if (block_size == 16) GO(16);
  if (block_size == 32) GO(32);
#undef GO
  return -1;
}

}  // namespace

// Same argument order as the reference's paged_attention_v2 plus the slope pointer.
// Supported here: dtype 0 (f16) / 1 (bf16), head_size 64 / 128, block_size 16 / 32.
extern "C" int ref_paged_attention_v2_alibi(void* out, float* exp_sums, float* max_logits, void* tmp_out,
                                            void* query, void* key_cache, void* value_cache, int32_t num_kv_heads,
                                            float scale, uint32_t* block_tables, uint32_t* context_lens,
                                            int32_t block_size, int32_t max_context_len, int32_t num_seqs,
                                            int32_t num_heads, int32_t head_size, int32_t max_num_blocks_per_seq,
                                            int32_t q_stride, int32_t kv_block_stride, int32_t kv_head_stride,
                                            uint32_t dtype, float softcapping, const float* alibi_slopes,
                                            int64_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
#define ARGS                                                                                                  \
  block_size, out, exp_sums, max_logits, tmp_out, query, key_cache, value_cache, num_kv_heads, scale,         \
      block_tables, context_lens, max_context_len, num_seqs, num_heads, max_num_blocks_per_seq, q_stride,     \
      kv_block_stride, kv_head_stride, softcapping, alibi_slopes, stream
  if (dtype == 1 && head_size == 128) return by_block<__nv_bfloat16, 128>(ARGS);
  if (dtype == 1 && head_size == 64) return by_block<__nv_bfloat16, 64>(ARGS);
  if (dtype == 0 && head_size == 128) return by_block<uint16_t, 128>(ARGS);
  if (dtype == 0 && head_size == 64) return by_block<uint16_t, 64>(ARGS);
#undef ARGS
  return -1;
}
