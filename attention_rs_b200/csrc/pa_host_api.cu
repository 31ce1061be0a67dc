// Host-side mirror of the reference's Rust operators: the same shape / dtype
// checks in the same order with the same messages (src/paged_attention.rs:68-152
// for paged_attention, :596-660 for reshape_and_cache), then kernel dispatch.
// The reference's host layer is compiled Rust inside the caller's process; this is
// its C++ counterpart behind a C ABI so that any host language can bind it.
#include <stdio.h>
#include <string>

#include "pa_common.cuh"
#include "pa_launch.h"

namespace {

using pa::fail;

std::string dims(const pa_tensor* t) {
  std::string s = "[";
  for (int i = 0; i < t->rank; ++i) {
    if (i) s += ", ";
    s += std::to_string(t->shape[i]);
  }
  return s + "]";
}

bool float_dtype(uint32_t dt) { return dt == PA_DTYPE_F16 || dt == PA_DTYPE_BF16 || dt == PA_DTYPE_F32; }

bool contiguous_from(const pa_tensor* t, int first_dim) {
  int64_t expect = 1;
  for (int i = t->rank - 1; i >= first_dim; --i) {
    if (t->shape[i] != 1 && t->stride[i] != expect) return false;
    expect *= t->shape[i];
  }
  return true;
}

bool fits_i32(int64_t v) { return v >= 0 && v <= 0x7fffffffLL; }

}  // namespace

extern "C" {

size_t pa_paged_attention_workspace_bytes(int64_t num_seqs, int64_t num_heads, int64_t head_size,
                                          int64_t max_context_len, uint32_t dtype) {
  const int64_t parts = (max_context_len + PA_PARTITION_SIZE - 1) / PA_PARTITION_SIZE;
  if (num_seqs <= 0 || num_heads <= 0 || head_size <= 0 || parts <= 0) return 0;
  const int64_t es = pa::dtype_size(dtype);
  // tmp_out, then exp_sums, then max_logits; each region rounded up to 256 bytes.
  auto up = [](int64_t v) { return (v + 255) / 256 * 256; };
  return static_cast<size_t>(up(num_seqs * num_heads * parts * head_size * es) + 2 * up(num_seqs * num_heads * parts * 4));
}

// Partition rule of this library.  The reference (src/paged_attention.rs:158-161)
// takes the single-pass kernel whenever num_seqs * num_heads > 512 because its
// single-pass grid is already large then.  Here a single-pass CTA covers a whole
// (sequence, kv head) pair, so long contexts are split whenever there is more than
// one partition: that keeps every CTA's work bounded and the SMs evenly loaded.
int pa_paged_attention_uses_partitions(int64_t num_seqs, int64_t num_heads, int64_t num_kv_heads,
                                       int64_t max_context_len) {
  (void)num_seqs;
  (void)num_heads;
  (void)num_kv_heads;
  const int64_t parts = (max_context_len + PA_PARTITION_SIZE - 1) / PA_PARTITION_SIZE;
  return parts > 1 ? 1 : 0;
}

static int paged_attention_impl(const pa_tensor* q, const pa_tensor* new_key, const pa_tensor* new_value,
                                const pa_tensor* key_cache, const pa_tensor* value_cache, const pa_tensor* block_tables,
                                const pa_tensor* context_lens, const pa_tensor* alibi_slopes, int64_t max_context_len,
                                float softmax_scale, float softcapping, float k_scale, float v_scale,
                                const pa_tensor* out, void* workspace, size_t workspace_bytes, int64_t stream) {
  if (!q || !key_cache || !value_cache || !block_tables || !context_lens || !out)
    return fail(PA_ERR_INVALID_ARGUMENT, "null tensor descriptor");
  if (!float_dtype(q->dtype)) return fail(PA_ERR_INVALID_ARGUMENT, "dtype code %u is not supported", q->dtype);
  if (q->rank != 3)
    return fail(PA_ERR_INVALID_ARGUMENT, "paged-attention expects `q` tensor to be of rank 3 (q: %s)", dims(q).c_str());
  if (key_cache->rank != 5)
    return fail(PA_ERR_INVALID_ARGUMENT, "paged-attention expects `key_cache` tensor to be of rank 5 (key_cache: %s)",
                dims(key_cache).c_str());
  if (value_cache->rank != 4)
    return fail(PA_ERR_INVALID_ARGUMENT, "paged-attention expects `value_cache` tensor to be of rank 4 (value_cache: %s)",
                dims(value_cache).c_str());
  const uint32_t kv_dtype = key_cache->dtype;
  if (value_cache->dtype != kv_dtype || (kv_dtype != q->dtype && kv_dtype != PA_DTYPE_FP8_E4M3))
    return fail(PA_ERR_INVALID_ARGUMENT, "key_cache / value_cache dtype must match q or be FP8 E4M3");
  if (block_tables->dtype != PA_DTYPE_U32 || context_lens->dtype != PA_DTYPE_U32)
    return fail(PA_ERR_INVALID_ARGUMENT, "block_tables and context_lens must be u32 tensors");

  const int64_t num_seqs = q->shape[0], num_heads = q->shape[1], head_size = q->shape[2];
  if (!(head_size == 64 || head_size == 80 || head_size == 96 || head_size == 112 || head_size == 128 ||
        head_size == 192 || head_size == 256))
    return fail(PA_ERR_INVALID_ARGUMENT, "`head_size` must be one of 64, 80, 96, 112, 128, 192 or 256");
  if (block_tables->rank != 2) return fail(PA_ERR_INVALID_ARGUMENT, "block_tables must be of rank 2");
  const int64_t max_blocks = block_tables->shape[1];
  if (block_tables->shape[0] != num_seqs)
    return fail(PA_ERR_INVALID_ARGUMENT, "shape mismatch block_tables %s, expected [%lld, %lld]", dims(block_tables).c_str(),
                (long long)num_seqs, (long long)max_blocks);
  const int64_t num_blocks = key_cache->shape[0], num_kv_heads = key_cache->shape[1], block_size = key_cache->shape[3],
                x = key_cache->shape[4];
  if (x <= 0 || key_cache->shape[2] != head_size / x)
    return fail(PA_ERR_INVALID_ARGUMENT, "shape mismatch value_cache %s, expected [%lld, %lld, %lld, %lld, %lld]",
                dims(value_cache).c_str(), (long long)num_blocks, (long long)num_heads, (long long)(x > 0 ? head_size / x : 0),
                (long long)block_size, (long long)x);
  if (value_cache->shape[0] != num_blocks || value_cache->shape[1] != num_kv_heads || value_cache->shape[2] != head_size ||
      value_cache->shape[3] != block_size)
    return fail(PA_ERR_INVALID_ARGUMENT, "shape mismatch key_cache %s and value_cache %s", dims(key_cache).c_str(),
                dims(value_cache).c_str());
  if (context_lens->rank != 1 || context_lens->shape[0] != num_seqs)
    return fail(PA_ERR_INVALID_ARGUMENT, "shape mismatch context_lens %s, expected [%lld]", dims(context_lens).c_str(),
                (long long)num_seqs);

  if (num_seqs == 0) return PA_OK;
  // Checks the reference leaves to the kernel's assumptions; made explicit here.
  if (x * pa::dtype_size(kv_dtype) != 16)
    return fail(PA_ERR_INVALID_ARGUMENT, "key_cache chunk width x must be 16 / sizeof(cache element), got %lld", (long long)x);
  if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0)
    return fail(PA_ERR_INVALID_ARGUMENT, "num_heads (%lld) must be a multiple of num_kv_heads (%lld)", (long long)num_heads,
                (long long)num_kv_heads);
  if (!(block_size == 8 || block_size == 16 || block_size == 32))
    return fail(PA_ERR_INVALID_ARGUMENT, "`block_size` must be one of 8, 16 or 32");
  if (q->stride[2] != 1 || q->stride[1] != head_size)
    return fail(PA_ERR_INVALID_ARGUMENT, "q must be contiguous in its last two dimensions");
  if (!contiguous_from(key_cache, 2) || !contiguous_from(value_cache, 2) ||
      key_cache->stride[0] != value_cache->stride[0] || key_cache->stride[1] != value_cache->stride[1])
    return fail(PA_ERR_INVALID_ARGUMENT, "key_cache / value_cache must be contiguous within a (block, head) tile and share strides");
  if (!contiguous_from(block_tables, 0) || !contiguous_from(context_lens, 0))
    return fail(PA_ERR_INVALID_ARGUMENT, "block_tables and context_lens must be contiguous");
  if (alibi_slopes && (alibi_slopes->dtype != PA_DTYPE_F32 || alibi_slopes->rank != 1 || alibi_slopes->shape[0] != num_heads ||
                       alibi_slopes->stride[0] != 1))
    return fail(PA_ERR_INVALID_ARGUMENT, "alibi_slopes must be a contiguous f32 tensor of shape [num_heads]");
  if (out->dtype != q->dtype || out->rank != 3 || out->shape[0] != num_seqs || out->shape[1] != num_heads ||
      out->shape[2] != head_size || !contiguous_from(out, 0))
    return fail(PA_ERR_INVALID_ARGUMENT, "out must be a contiguous tensor with the shape and dtype of q");
  if (max_context_len < 0 || max_blocks * block_size < max_context_len)
    return fail(PA_ERR_INVALID_ARGUMENT, "block_tables holds %lld blocks per sequence, fewer than max_context_len %lld needs",
                (long long)max_blocks, (long long)max_context_len);
  if (kv_dtype == PA_DTYPE_FP8_E4M3 && !(k_scale > 0.f && v_scale > 0.f))
    return fail(PA_ERR_INVALID_ARGUMENT, "FP8 cache needs positive k_scale / v_scale");
  if (!fits_i32(q->stride[0]) || !fits_i32(key_cache->stride[0]) || !fits_i32(key_cache->stride[1]) ||
      !fits_i32(max_context_len) || !fits_i32(max_blocks))
    return fail(PA_ERR_INVALID_ARGUMENT, "a stride or size does not fit the 32-bit fields of the kernel interface");
  // Fused decode step: the rows of each sequence's newest token.
  const bool step = new_key != nullptr || new_value != nullptr;
  if (step) {
    if (!new_key || !new_value) return fail(PA_ERR_INVALID_ARGUMENT, "key and value rows must be given together");
    for (const pa_tensor* t : {new_key, new_value}) {
      if (t->dtype != q->dtype || t->rank != 3 || t->shape[0] != num_seqs || t->shape[1] != num_kv_heads ||
          t->shape[2] != head_size || t->stride[2] != 1 || t->stride[1] != head_size || !fits_i32(t->stride[0]))
        return fail(PA_ERR_INVALID_ARGUMENT,
                    "decode-step key / value must be [num_seqs, num_kv_heads, head_size] tensors of q's dtype, "
                    "contiguous in their last two dimensions");
    }
  }

  const bool want_parts = pa_paged_attention_uses_partitions(num_seqs, num_heads, num_kv_heads, max_context_len) != 0;
  const size_t need = pa_paged_attention_workspace_bytes(num_seqs, num_heads, head_size, max_context_len, q->dtype);
  if (want_parts && workspace != nullptr && workspace_bytes < need)
    return fail(PA_ERR_WORKSPACE, "workspace of %zu bytes is smaller than the %zu bytes needed", workspace_bytes, need);
  const bool parts = want_parts && workspace != nullptr;
  const float* slopes = alibi_slopes ? static_cast<const float*>(alibi_slopes->data) : nullptr;
  if (parts) {
    const int64_t nparts = (max_context_len + PA_PARTITION_SIZE - 1) / PA_PARTITION_SIZE;
    auto up = [](int64_t v) { return (v + 255) / 256 * 256; };
    char* w = static_cast<char*>(workspace);
    void* tmp_out = w;
    float* exp_sums = reinterpret_cast<float*>(w + up(num_seqs * num_heads * nparts * head_size * pa::dtype_size(q->dtype)));
    float* max_logits = reinterpret_cast<float*>(reinterpret_cast<char*>(exp_sums) + up(num_seqs * num_heads * nparts * 4));
    if (step)
      return paged_decode_step_v2(out->data, exp_sums, max_logits, tmp_out, q->data, new_key->data, new_value->data,
                                  (int32_t)new_key->stride[0], (int32_t)new_value->stride[0], key_cache->data,
                                  value_cache->data, (int32_t)num_kv_heads, softmax_scale,
                                  static_cast<const uint32_t*>(block_tables->data),
                                  static_cast<const uint32_t*>(context_lens->data), (int32_t)block_size,
                                  (int32_t)max_context_len, (int32_t)num_seqs, (int32_t)num_heads, (int32_t)head_size,
                                  (int32_t)max_blocks, (int32_t)q->stride[0], (int32_t)key_cache->stride[0],
                                  (int32_t)key_cache->stride[1], q->dtype, softcapping, slopes, kv_dtype, k_scale,
                                  v_scale, stream);
    return paged_attention_v2_ex(out->data, exp_sums, max_logits, tmp_out, q->data, key_cache->data, value_cache->data,
                                 (int32_t)num_kv_heads, softmax_scale, static_cast<const uint32_t*>(block_tables->data),
                                 static_cast<const uint32_t*>(context_lens->data), (int32_t)block_size,
                                 (int32_t)max_context_len, (int32_t)num_seqs, (int32_t)num_heads, (int32_t)head_size,
                                 (int32_t)max_blocks, (int32_t)q->stride[0], (int32_t)key_cache->stride[0],
                                 (int32_t)key_cache->stride[1], q->dtype, softcapping, slopes, kv_dtype, k_scale, v_scale,
                                 stream);
  }
  if (step)
    return paged_decode_step_v1(out->data, q->data, new_key->data, new_value->data, (int32_t)new_key->stride[0],
                                (int32_t)new_value->stride[0], key_cache->data, value_cache->data, (int32_t)num_kv_heads,
                                softmax_scale, static_cast<const uint32_t*>(block_tables->data),
                                static_cast<const uint32_t*>(context_lens->data), (int32_t)block_size,
                                (int32_t)max_context_len, (int32_t)num_seqs, (int32_t)num_heads, (int32_t)head_size,
                                (int32_t)max_blocks, (int32_t)q->stride[0], (int32_t)key_cache->stride[0],
                                (int32_t)key_cache->stride[1], q->dtype, softcapping, slopes, kv_dtype, k_scale, v_scale,
                                stream);
  return paged_attention_v1_ex(out->data, q->data, key_cache->data, value_cache->data, (int32_t)num_kv_heads, softmax_scale,
                               static_cast<const uint32_t*>(block_tables->data),
                               static_cast<const uint32_t*>(context_lens->data), (int32_t)block_size,
                               (int32_t)max_context_len, (int32_t)num_seqs, (int32_t)num_heads, (int32_t)head_size,
                               (int32_t)max_blocks, (int32_t)q->stride[0], (int32_t)key_cache->stride[0],
                               (int32_t)key_cache->stride[1], q->dtype, softcapping, slopes, kv_dtype, k_scale, v_scale,
                               stream);
}

int pa_paged_attention(const pa_tensor* q, const pa_tensor* key_cache, const pa_tensor* value_cache,
                       const pa_tensor* block_tables, const pa_tensor* context_lens, const pa_tensor* alibi_slopes,
                       int64_t max_context_len, float softmax_scale, float softcapping, float k_scale, float v_scale,
                       const pa_tensor* out, void* workspace, size_t workspace_bytes, int64_t stream) {
  return paged_attention_impl(q, nullptr, nullptr, key_cache, value_cache, block_tables, context_lens, alibi_slopes,
                              max_context_len, softmax_scale, softcapping, k_scale, v_scale, out, workspace,
                              workspace_bytes, stream);
}

int pa_decode_step(const pa_tensor* q, const pa_tensor* key, const pa_tensor* value, const pa_tensor* key_cache,
                   const pa_tensor* value_cache, const pa_tensor* block_tables, const pa_tensor* context_lens,
                   const pa_tensor* alibi_slopes, int64_t max_context_len, float softmax_scale, float softcapping,
                   float k_scale, float v_scale, const pa_tensor* out, void* workspace, size_t workspace_bytes,
                   int64_t stream) {
  if (!key || !value) return fail(PA_ERR_INVALID_ARGUMENT, "null tensor descriptor");
  return paged_attention_impl(q, key, value, key_cache, value_cache, block_tables, context_lens, alibi_slopes,
                              max_context_len, softmax_scale, softcapping, k_scale, v_scale, out, workspace,
                              workspace_bytes, stream);
}

int pa_reshape_and_cache(const pa_tensor* key, const pa_tensor* value, const pa_tensor* key_cache,
                         const pa_tensor* value_cache, const pa_tensor* slot_mapping, float k_scale, float v_scale,
                         int64_t stream) {
  if (!key || !value || !key_cache || !value_cache || !slot_mapping)
    return fail(PA_ERR_INVALID_ARGUMENT, "null tensor descriptor");
  if (!float_dtype(key->dtype)) return fail(PA_ERR_INVALID_ARGUMENT, "dtype code %u is not supported", key->dtype);
  if (key->rank != 3 || value->rank != 3)
    return fail(PA_ERR_INVALID_ARGUMENT, "paged-attention expects input tensors of rank 3 (k: %s, v: %s)", dims(key).c_str(),
                dims(value).c_str());
  if (key_cache->rank != 5)
    return fail(PA_ERR_INVALID_ARGUMENT, "paged-attention expects `key_cache` tensor to be of rank 5 (key_cache: %s)",
                dims(key_cache).c_str());
  if (value_cache->rank != 4)
    return fail(PA_ERR_INVALID_ARGUMENT, "paged-attention expects `value_cache` tensor to be of rank 4 (value_cache: %s)",
                dims(value_cache).c_str());
  if (value->dtype != key->dtype) return fail(PA_ERR_INVALID_ARGUMENT, "key and value must share a dtype");
  const uint32_t cache_dtype = key_cache->dtype;
  if (value_cache->dtype != cache_dtype || (cache_dtype != key->dtype && cache_dtype != PA_DTYPE_FP8_E4M3))
    return fail(PA_ERR_INVALID_ARGUMENT, "key_cache / value_cache dtype must match key or be FP8 E4M3");
  if (slot_mapping->dtype != PA_DTYPE_I64) return fail(PA_ERR_INVALID_ARGUMENT, "slot_mapping must be an i64 tensor");
  const int64_t num_tokens = key->shape[0], num_heads = key->shape[1], head_size = key->shape[2];
  if (value->shape[0] != num_tokens || value->shape[1] != num_heads || value->shape[2] != head_size)
    return fail(PA_ERR_INVALID_ARGUMENT, "shape mismatch k %s and v %s", dims(key).c_str(), dims(value).c_str());
  const int64_t num_blocks = key_cache->shape[0], block_size = key_cache->shape[3], x = key_cache->shape[4];
  if (key_cache->shape[1] != num_heads || x <= 0 || key_cache->shape[2] != head_size / x)
    return fail(PA_ERR_INVALID_ARGUMENT, "shape mismatch value_cache %s, expected [%lld, %lld, %lld, %lld, %lld]",
                dims(value_cache).c_str(), (long long)num_blocks, (long long)num_heads, (long long)(x > 0 ? head_size / x : 0),
                (long long)block_size, (long long)x);
  if (value_cache->shape[0] != num_blocks || value_cache->shape[1] != num_heads || value_cache->shape[2] != head_size ||
      value_cache->shape[3] != block_size)
    return fail(PA_ERR_INVALID_ARGUMENT, "shape mismatch key_cache %s and value_cache %s", dims(key_cache).c_str(),
                dims(value_cache).c_str());
  if (slot_mapping->rank != 1 || slot_mapping->shape[0] != num_tokens)
    return fail(PA_ERR_INVALID_ARGUMENT, "shape mismatch slot_mapping %s, expected [%lld]", dims(slot_mapping).c_str(),
                (long long)num_tokens);
  if (num_tokens == 0) return PA_OK;
  // Made explicit here; the reference's kernel assumes them.
  if (head_size % x != 0) return fail(PA_ERR_INVALID_ARGUMENT, "head_size %lld is not a multiple of x %lld", (long long)head_size, (long long)x);
  if (key->stride[2] != 1 || key->stride[1] != head_size || value->stride[2] != 1 || value->stride[1] != head_size)
    return fail(PA_ERR_INVALID_ARGUMENT, "key and value must be contiguous in their last two dimensions");
  if (!contiguous_from(key_cache, 0) || !contiguous_from(value_cache, 0))
    return fail(PA_ERR_INVALID_ARGUMENT, "key_cache and value_cache must be contiguous");
  if (slot_mapping->stride[0] != 1 && num_tokens > 1) return fail(PA_ERR_INVALID_ARGUMENT, "slot_mapping must be contiguous");
  if (!fits_i32(key->stride[0]) || !fits_i32(value->stride[0]) || !fits_i32(num_tokens))
    return fail(PA_ERR_INVALID_ARGUMENT, "a stride or size does not fit the 32-bit fields of the kernel interface");
  return call_reshape_and_cache_ex(key->data, value->data, key_cache->data, value_cache->data,
                                   static_cast<const int64_t*>(slot_mapping->data), (int32_t)num_tokens, (int32_t)num_heads,
                                   (int32_t)head_size, (int32_t)block_size, (int32_t)x, (int32_t)key->stride[0],
                                   (int32_t)value->stride[0], key->dtype, cache_dtype, k_scale, v_scale, stream);
}

}  // extern "C"
