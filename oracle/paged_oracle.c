/*
 * CPU oracle for the paged-attention hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a checker: it is linked or loaded only by the test-suite, by the
 * smoke check and by the CPU-baseline / reference legs of the benchmark.  The
 * product library never calls into it and has no CPU fallback.
 *
 * It restates, in plain C, the algorithm of the reference's CUDA path
 * (paths are relative to the reference project root):
 *
 *   - cache layouts and the scatter rule ......... src/kernels/src/reshape_and_cache_kernel.cu:14-59
 *   - query-head -> kv-head mapping .............. src/kernels/src/pagedattention.cu:147-150
 *                                                  (same as repeat_kv, src/lib.rs:131-143)
 *   - logits: scale * q.k, optional tanh soft-cap,
 *     optional ALiBi bias, context-length mask ... src/kernels/src/pagedattention.cu:229-244
 *     (soft-cap also in src/lib.rs:187-189)
 *   - softmax over the context in fp32 ........... src/kernels/src/pagedattention.cu:248-284,
 *                                                  src/lib.rs:198-200
 *   - probability-weighted sum of values ......... src/kernels/src/pagedattention.cu:309-348
 *   - split of the context in partitions and the
 *     log-sum-exp merge of the partial results ... src/kernels/src/pagedattention.cu:116-136, 286-296, 508-565
 *
 * The reference has no CPU implementation of this path (its cpu_fwd bails,
 * src/paged_attention.rs:475-477 and :830-832) and ships no tests or golden
 * vectors, so parity of this restatement is pinned against outputs of the
 * reference's own CUDA kernels compiled unchanged and run on a B200; those
 * outputs are committed as fixtures under tests/golden/.
 *
 * The FP8-E4M3 cache mode (dtype code 3) has no counterpart in the reference:
 * PARITY UNPINNED for that mode.  Its definition is: cache byte =
 * sat_e4m3_rn(x / scale) computed with an IEEE fp32 division, and decode reads
 * float(e4m3) * scale.
 *
 * ALiBi.  The bias of the algorithm is slope * (token - context_len + 1), a value <= 0.
 * The reference's device code writes exactly that expression
 * (src/kernels/src/pagedattention.cu:235; same line in its Metal twin,
 * src/metal-kernels/src/pagedattention.metal:1122) but with context_len declared
 * uint32_t (:119), so the subtraction is carried out in unsigned arithmetic and wraps:
 * every token but the last receives a bias near slope * 2^32.  Its C ABI never reaches
 * that line (alibi_slopes is hard-wired to nullptr, :621-622 and :795-796).  The oracle
 * implements the signed formula (alibi_mode 0), which is what the product computes, and
 * can also evaluate the reference's literal unsigned expression (alibi_mode 1) so that the
 * golden outputs of the reference's kernel templates pin this file for ALiBi as well.
 *
 * dtype codes follow src/kernels/src/pagedattention.cu:723: 0 = f16, 1 = bf16,
 * 2 = f32; 3 = FP8 E4M3 (cache only).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { DT_F16 = 0, DT_BF16 = 1, DT_F32 = 2, DT_FP8_E4M3 = 3 };

/* ---------------------------------------------------------------- scalar codecs */

static inline float u32_as_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_as_u32(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static inline float bf16_to_f32(uint16_t h) { return u32_as_f32((uint32_t)h << 16); }

static inline float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  if (exp == 0) {
    if (man == 0) return u32_as_f32(sign);
    /* subnormal: man * 2^-24 */
    float v = (float)man * (1.0f / 16777216.0f);
    return (sign ? -v : v);
  }
  if (exp == 31) return u32_as_f32(sign | 0x7f800000u | (man << 13));
  return u32_as_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

/* Decode of one FP8 E4M3 ("fn": no infinities, 0x7f/0xff are NaN) byte. */
static inline float e4m3_to_f32(uint8_t b) {
  uint32_t sign = b & 0x80u;
  uint32_t exp = (b >> 3) & 0xfu;
  uint32_t man = b & 0x7u;
  float v;
  if (exp == 0xf && man == 0x7) return NAN;
  if (exp == 0) v = (float)man * (1.0f / 512.0f);             /* man/8 * 2^-6 */
  else v = ldexpf(1.0f + (float)man / 8.0f, (int)exp - 7);
  return sign ? -v : v;
}

/* Round-to-nearest-even, saturate-to-finite encode of fp32 into FP8 E4M3. */
static inline uint8_t f32_to_e4m3_satfinite(float x) {
  uint32_t u = f32_as_u32(x);
  uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
  float a = fabsf(x);
  if (isnan(x)) return (uint8_t)(sign | 0x7f);
  if (a >= 464.0f) return (uint8_t)(sign | 0x7e);             /* >= halfway past 448 saturates to 448 */
  if (a < 0.0009765625f) {                                    /* below 2^-10: rounds to 0 or to 2^-9 */
    /* exactly 2^-10 is a tie between 0 and 2^-9 (odd mantissa 1) -> even = 0 */
    return sign;
  }
  if (a < 0.015625f) {                                        /* subnormal range: step 2^-9 */
    float q = a * 512.0f;                                     /* exact */
    float r = nearbyintf(q);                                  /* RN-even in default rounding mode */
    uint32_t m = (uint32_t)r;                                 /* 0..8; 8 means the smallest normal */
    return (uint8_t)(sign | m);                               /* m == 8 encodes exp=1, man=0 */
  }
  {
    int e;
    float fr = frexpf(a, &e);                                 /* a = fr * 2^e, fr in [0.5,1) */
    float mant = fr * 2.0f;                                   /* [1,2) */
    int ee = e - 1;                                           /* a = mant * 2^ee, ee in [-6, 8] */
    float q = (mant - 1.0f) * 8.0f;                           /* [0,8) exact */
    float r = nearbyintf(q);
    uint32_t m = (uint32_t)r;
    if (m == 8) { m = 0; ee += 1; }
    if (ee > 8 || (ee == 8 && m > 6)) return (uint8_t)(sign | 0x7e);
    return (uint8_t)(sign | (uint32_t)((ee + 7) << 3) | m);
  }
}

static inline int elem_size(int dtype) {
  switch (dtype) {
    case DT_F16: case DT_BF16: return 2;
    case DT_F32: return 4;
    case DT_FP8_E4M3: return 1;
    default: return 0;
  }
}

static inline float load_elem(const void* base, int64_t idx, int dtype) {
  switch (dtype) {
    case DT_F16: return f16_to_f32(((const uint16_t*)base)[idx]);
    case DT_BF16: return bf16_to_f32(((const uint16_t*)base)[idx]);
    case DT_F32: return ((const float*)base)[idx];
    default: return e4m3_to_f32(((const uint8_t*)base)[idx]);
  }
}

/* Exposed for table tests of the codecs. */
float oracle_e4m3_decode(uint8_t b) { return e4m3_to_f32(b); }
uint8_t oracle_e4m3_encode(float x) { return f32_to_e4m3_satfinite(x); }
float oracle_f16_decode(uint16_t h) { return f16_to_f32(h); }
float oracle_bf16_decode(uint16_t h) { return bf16_to_f32(h); }

int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Thread count of the following parallel regions.  A launcher may have exported OMP_NUM_THREADS=1 for its ranks
 * (torch.distributed.run does); the timed CPU legs of the benchmark ask for every host core instead. */
void oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ---------------------------------------------------------------- reshape_and_cache */

/*
 * Scatter of new key/value rows into the paged caches
 * (src/kernels/src/reshape_and_cache_kernel.cu:27-58).
 *
 *   key, value ........ [num_tokens, num_heads, head_size], row strides in elements
 *   key_cache ......... [num_blocks, num_heads, head_size/x, block_size, x]
 *   value_cache ....... [num_blocks, num_heads, head_size, block_size]
 *   slot_mapping[i] ... destination slot of token i; negative = padding, skipped
 *
 * cache_dtype == dtype: pure copy (bit-exact).  cache_dtype == 3 with a 16/32-bit
 * source: per-tensor FP8 quantisation with k_scale / v_scale.
 */
int oracle_reshape_and_cache(const void* key, const void* value, void* key_cache, void* value_cache,
                             const int64_t* slot_mapping, int32_t num_tokens, int32_t num_heads,
                             int32_t head_size, int32_t block_size, int32_t x, int32_t key_stride,
                             int32_t value_stride, uint32_t dtype, uint32_t cache_dtype,
                             float k_scale, float v_scale) {
  const int es = elem_size((int)dtype);
  if (es == 0 || dtype == DT_FP8_E4M3) return -1;
  if (cache_dtype != dtype && cache_dtype != DT_FP8_E4M3) return -1;
  if (x <= 0 || head_size % x != 0) return -2;
  const int quant = (cache_dtype == DT_FP8_E4M3);
  const int n = num_heads * head_size;
  for (int64_t t = 0; t < num_tokens; ++t) {
    const int64_t slot = slot_mapping[t];
    if (slot < 0) continue;
    const int64_t blk = slot / block_size;
    const int64_t off = slot % block_size;
    for (int i = 0; i < n; ++i) {
      const int h = i / head_size, d = i % head_size;
      const int64_t src_k = t * (int64_t)key_stride + i;
      const int64_t src_v = t * (int64_t)value_stride + i;
      const int64_t dst_k = (((blk * num_heads + h) * (head_size / x) + d / x) * block_size + off) * x + d % x;
      const int64_t dst_v = ((blk * num_heads + h) * (int64_t)head_size + d) * block_size + off;
      if (!quant) {
        memcpy((char*)key_cache + dst_k * es, (const char*)key + src_k * es, (size_t)es);
        memcpy((char*)value_cache + dst_v * es, (const char*)value + src_v * es, (size_t)es);
      } else {
        ((uint8_t*)key_cache)[dst_k] = f32_to_e4m3_satfinite(load_elem(key, src_k, (int)dtype) / k_scale);
        ((uint8_t*)value_cache)[dst_v] = f32_to_e4m3_satfinite(load_elem(value, src_v, (int)dtype) / v_scale);
      }
    }
  }
  return 0;
}

/* ---------------------------------------------------------------- paged attention */

typedef struct {
  float m;   /* max logit of the range, -inf if empty */
  float l;   /* sum of exp(logit - m) */
} softmax_state;

/*
 * Attention of one query head over tokens [t0, t1) of one sequence.
 * acc[head_size] receives sum_t exp(s_t - m) * v_t (un-normalised).
 * logits is scratch of at least t1 - t0 floats.
 */
static softmax_state attend_range(const void* q, int64_t q_off, int dtype, const void* kc, const void* vc,
                                  int kv_dtype, const uint32_t* table, int64_t kv_block_stride,
                                  int64_t kv_head_off, int head_size, int block_size, int x, float scale,
                                  float softcap, float slope, int alibi_mode, float k_scale, float v_scale,
                                  int ctx, int t0, int t1, float* logits, float* qf, double* acc) {
  softmax_state st;
  st.m = -INFINITY;
  st.l = 0.f;
  for (int d = 0; d < head_size; ++d) { qf[d] = load_elem(q, q_off + d, dtype); acc[d] = 0.0; }
  for (int t = t0; t < t1; ++t) {
    const int64_t blk = (int64_t)table[t / block_size];
    const int off = t % block_size;
    const int64_t base = blk * kv_block_stride + kv_head_off;
    double dot = 0.0;
    for (int d = 0; d < head_size; ++d) {
      const int64_t ki = base + ((int64_t)(d / x) * block_size + off) * x + d % x;
      dot += (double)qf[d] * (double)(load_elem(kc, ki, kv_dtype) * k_scale);
    }
    float s = scale * (float)dot;
    if (softcap != 1.0f) s = tanhf(s / softcap) * softcap;
    if (slope != 0.f) {
      if (alibi_mode == 0) s += slope * (float)(t - ctx + 1);
      else s += slope * (float)((uint32_t)t - (uint32_t)ctx + 1u);   /* the reference's literal arithmetic */
    }
    logits[t - t0] = s;
    if (s > st.m) st.m = s;
  }
  double l = 0.0;
  for (int t = t0; t < t1; ++t) {
    const float p = expf(logits[t - t0] - st.m);
    logits[t - t0] = p;
    l += p;
  }
  st.l = (float)l;
  for (int t = t0; t < t1; ++t) {
    const int64_t blk = (int64_t)table[t / block_size];
    const int off = t % block_size;
    const int64_t base = blk * kv_block_stride + kv_head_off;
    const double p = logits[t - t0];
    for (int d = 0; d < head_size; ++d) {
      const int64_t vi = base + (int64_t)d * block_size + off;
      acc[d] += p * (double)(load_elem(vc, vi, kv_dtype) * v_scale);
    }
  }
  return st;
}

/*
 * Decode attention over a paged KV cache; out is fp32 [num_seqs, num_heads, head_size].
 *
 * partition_size == 0: one pass over the whole context (the v1 formulation).
 * partition_size  > 0: independent passes over partitions of that many tokens,
 *   merged by log-sum-exp (the v2 formulation, src/kernels/src/pagedattention.cu:508-565);
 *   in exact arithmetic both give the same result.
 *
 * A sequence with context_len == 0 yields zeros (the reference's loops are empty
 * and its accumulators start at zero).
 * alibi_slopes may be NULL; alibi_mode 0 = signed bias (the algorithm), 1 = the
 * reference's literal unsigned expression (see the file header).  softcapping == 1.0 means "off"
 * (src/kernels/src/pagedattention.cu:231-233).
 * x, the key-cache chunk width in elements, is 16 / sizeof(cache element)
 * (src/kernels/src/pagedattention.cu:192).
 */
int oracle_paged_attention(float* out, const void* query, const void* key_cache, const void* value_cache,
                           int32_t num_kv_heads, float scale, const uint32_t* block_tables,
                           const uint32_t* context_lens, int32_t block_size, int32_t max_context_len,
                           int32_t num_seqs, int32_t num_heads, int32_t head_size,
                           int32_t max_num_blocks_per_seq, int32_t q_stride, int32_t kv_block_stride,
                           int32_t kv_head_stride, uint32_t dtype, uint32_t kv_dtype, float softcapping,
                           const float* alibi_slopes, float k_scale, float v_scale, int32_t partition_size,
                           int32_t alibi_mode) {
  if (elem_size((int)dtype) == 0 || dtype == DT_FP8_E4M3 || elem_size((int)kv_dtype) == 0) return -1;
  if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0) return -2;
  const int x = 16 / elem_size((int)kv_dtype);
  if (head_size % x != 0) return -3;
  const int group = num_heads / num_kv_heads;
  if (kv_dtype != DT_FP8_E4M3) { k_scale = 1.f; v_scale = 1.f; }
  int status = 0;
  const int64_t work = (int64_t)num_seqs * num_heads;
#pragma omp parallel
  {
    float* logits = (float*)malloc(sizeof(float) * (size_t)(max_context_len > 0 ? max_context_len : 1));
    float* qf = (float*)malloc(sizeof(float) * (size_t)head_size);
    double* acc = (double*)malloc(sizeof(double) * (size_t)head_size);
    double* tot = (double*)malloc(sizeof(double) * (size_t)head_size);
#pragma omp for schedule(dynamic, 1)
    for (int64_t w = 0; w < work; ++w) {
      const int seq = (int)(w / num_heads), head = (int)(w % num_heads);
      const int ctx = (int)context_lens[seq];
      float* o = out + ((int64_t)seq * num_heads + head) * head_size;
      if (ctx > max_context_len) {
#pragma omp atomic write
        status = -4;
        continue;
      }
      if (ctx == 0) { for (int d = 0; d < head_size; ++d) o[d] = 0.f; continue; }
      const uint32_t* table = block_tables + (int64_t)seq * max_num_blocks_per_seq;
      const int64_t kv_head_off = (int64_t)(head / group) * kv_head_stride;
      const int64_t q_off = (int64_t)seq * q_stride + (int64_t)head * head_size;
      const float slope = alibi_slopes ? alibi_slopes[head] : 0.f;
      const int part = partition_size > 0 ? partition_size : ctx;
      float M = -INFINITY;
      double L = 0.0;
      for (int d = 0; d < head_size; ++d) tot[d] = 0.0;
      for (int t0 = 0; t0 < ctx; t0 += part) {
        const int t1 = t0 + part < ctx ? t0 + part : ctx;
        softmax_state st = attend_range(query, q_off, (int)dtype, key_cache, value_cache, (int)kv_dtype, table,
                                        kv_block_stride, kv_head_off, head_size, block_size, x, scale,
                                        softcapping, slope, alibi_mode, k_scale, v_scale, ctx, t0, t1, logits, qf,
                                        acc);
        const float Mn = st.m > M ? st.m : M;
        const double a = exp((double)M - (double)Mn), b = exp((double)st.m - (double)Mn);
        for (int d = 0; d < head_size; ++d) tot[d] = tot[d] * a + acc[d] * b;
        L = L * a + (double)st.l * b;
        M = Mn;
      }
      for (int d = 0; d < head_size; ++d) o[d] = (float)(tot[d] / L);
    }
    free(logits); free(qf); free(acc); free(tot);
  }
  return status;
}

/*
 * The same decode attention written the way the reference's only CPU-capable
 * attention code is written (src/lib.rs:185-201): gather the sequence's K and V
 * out of the paged cache into dense fp32 matrices, logits = (q K^T) * scale,
 * optional soft-cap, softmax in fp32, then probabilities times V.  All
 * arithmetic is fp32.  This is the function the benchmark times as the CPU
 * baseline; it runs on every host thread OpenMP gives it.
 */
int oracle_paged_attention_naive_f32(float* out, const void* query, const void* key_cache,
                                     const void* value_cache, int32_t num_kv_heads, float scale,
                                     const uint32_t* block_tables, const uint32_t* context_lens,
                                     int32_t block_size, int32_t max_context_len, int32_t num_seqs,
                                     int32_t num_heads, int32_t head_size, int32_t max_num_blocks_per_seq,
                                     int32_t q_stride, int32_t kv_block_stride, int32_t kv_head_stride,
                                     uint32_t dtype, uint32_t kv_dtype, float softcapping,
                                     const float* alibi_slopes, float k_scale, float v_scale) {
  if (elem_size((int)dtype) == 0 || dtype == DT_FP8_E4M3 || elem_size((int)kv_dtype) == 0) return -1;
  if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0) return -2;
  const int x = 16 / elem_size((int)kv_dtype);
  const int group = num_heads / num_kv_heads;
  if (kv_dtype != DT_FP8_E4M3) { k_scale = 1.f; v_scale = 1.f; }
  const int64_t work = (int64_t)num_seqs * num_heads;
#pragma omp parallel
  {
    const size_t cap = (size_t)(max_context_len > 0 ? max_context_len : 1);
    float* K = (float*)malloc(sizeof(float) * cap * (size_t)head_size);
    float* V = (float*)malloc(sizeof(float) * cap * (size_t)head_size);
    float* p = (float*)malloc(sizeof(float) * cap);
    float* qf = (float*)malloc(sizeof(float) * (size_t)head_size);
#pragma omp for schedule(dynamic, 1)
    for (int64_t w = 0; w < work; ++w) {
      /* One work item per (sequence, query head): every query head gathers its own copy of
       * its kv head's rows, which is what repeat_kv does (src/lib.rs:131-143). */
      const int seq = (int)(w / num_heads), head = (int)(w % num_heads);
      const int kvh = head / group;
      int ctx = (int)context_lens[seq];
      if (ctx > max_context_len) ctx = max_context_len;
      const uint32_t* table = block_tables + (int64_t)seq * max_num_blocks_per_seq;
      for (int t = 0; t < ctx; ++t) {
        const int64_t base = (int64_t)table[t / block_size] * kv_block_stride + (int64_t)kvh * kv_head_stride;
        const int off = t % block_size;
        for (int d = 0; d < head_size; ++d) {
          K[(size_t)t * head_size + d] =
              load_elem(key_cache, base + ((int64_t)(d / x) * block_size + off) * x + d % x, (int)kv_dtype) * k_scale;
          V[(size_t)t * head_size + d] =
              load_elem(value_cache, base + (int64_t)d * block_size + off, (int)kv_dtype) * v_scale;
        }
      }
      {
        float* o = out + ((int64_t)seq * num_heads + head) * head_size;
        for (int d = 0; d < head_size; ++d) {
          qf[d] = load_elem(query, (int64_t)seq * q_stride + (int64_t)head * head_size + d, (int)dtype);
          o[d] = 0.f;
        }
        if (ctx == 0) continue;
        const float slope = alibi_slopes ? alibi_slopes[head] : 0.f;
        float m = -INFINITY;
        for (int t = 0; t < ctx; ++t) {
          const float* kr = K + (size_t)t * head_size;
          float s = 0.f;
          for (int d = 0; d < head_size; ++d) s += qf[d] * kr[d];
          s *= scale;
          if (softcapping != 1.0f) s = tanhf(s / softcapping) * softcapping;
          if (slope != 0.f) s += slope * (float)(t - ctx + 1);
          p[t] = s;
          if (s > m) m = s;
        }
        float l = 0.f;
        for (int t = 0; t < ctx; ++t) { p[t] = expf(p[t] - m); l += p[t]; }
        const float inv = 1.0f / l;
        for (int t = 0; t < ctx; ++t) {
          const float pt = p[t] * inv;
          const float* vr = V + (size_t)t * head_size;
          for (int d = 0; d < head_size; ++d) o[d] += pt * vr[d];
        }
      }
    }
    free(K); free(V); free(p); free(qf);
  }
  return 0;
}

/* ---------------------------------------------------------------- prefill attention */

/*
 * Causal self-attention over packed prompts: the function the reference's layer computes for a prefill
 * (src/lib.rs:145-213 without its flash-attn feature: per sequence, logits = q k^T * scale, optional
 * tanh soft-cap (:187-189), + causal mask (:191-195), softmax in f32 (:198-200), times v; kv heads repeated
 * for grouped queries, :131-143; with the feature, flash_attn_varlen with causal = true, :103-125).
 * q / k / v: [total_tokens, heads, head_size] with token strides in elements; cu_seqlens [num_seqs + 1].
 * out: fp32 [total_tokens, num_heads, head_size].  The reference's own code for this function is Rust on
 * candle tensors and cannot run where this oracle is tested: PARITY UNPINNED for this function.
 */
int oracle_prefill_attention(float* out, const void* q, const void* k, const void* v, const uint32_t* cu_seqlens,
                             int32_t num_seqs, int32_t num_heads, int32_t num_kv_heads, int32_t head_size,
                             int64_t q_stride, int64_t k_stride, int64_t v_stride, uint32_t dtype, float scale,
                             float softcapping, const float* alibi_slopes) {
  if (elem_size((int)dtype) == 0 || dtype == DT_FP8_E4M3) return -1;
  if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0) return -2;
  const int group = num_heads / num_kv_heads;
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
  for (int s = 0; s < num_seqs; ++s) {
    for (int h = 0; h < num_heads; ++h) {
      const int lo = (int)cu_seqlens[s], hi = (int)cu_seqlens[s + 1];
      const int kvh = h / group;
      const float slope = alibi_slopes ? alibi_slopes[h] : 0.f;
      double* logits = (double*)malloc(sizeof(double) * (size_t)(hi - lo + 1));
      for (int r = lo; r < hi; ++r) {
        double mx = -INFINITY;
        for (int c = lo; c <= r; ++c) {
          double dot = 0.0;
          for (int d = 0; d < head_size; ++d)
            dot += (double)load_elem(q, (int64_t)r * q_stride + (int64_t)h * head_size + d, (int)dtype) *
                   (double)load_elem(k, (int64_t)c * k_stride + (int64_t)kvh * head_size + d, (int)dtype);
          float x = scale * (float)dot;
          if (softcapping != 1.0f) x = tanhf(x / softcapping) * softcapping;
          x += slope * (float)(c - r);
          logits[c - lo] = x;
          if (x > mx) mx = x;
        }
        double sum = 0.0;
        for (int c = lo; c <= r; ++c) { logits[c - lo] = exp(logits[c - lo] - mx); sum += logits[c - lo]; }
        float* o = out + ((int64_t)r * num_heads + h) * head_size;
        for (int d = 0; d < head_size; ++d) {
          double acc = 0.0;
          for (int c = lo; c <= r; ++c)
            acc += logits[c - lo] * (double)load_elem(v, (int64_t)c * v_stride + (int64_t)kvh * head_size + d, (int)dtype);
          o[d] = (float)(acc / sum);
        }
      }
      free(logits);
    }
  }
  return 0;
}
