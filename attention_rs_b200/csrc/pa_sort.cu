// Row-wise argsort (the asort_* symbols of the reference's FFI, src/kernels/src/ffi.rs:75-186, defined in
// src/kernels/src/sort.cu:57-120).  Not part of the attention path; provided so that this library satisfies
// every symbol the reference's `kernels` crate declares.
//
// The reference sorts one row at a time from the host: a padded copy per row, log^2(n) kernel launches per
// row, host-to-device index uploads and a stream synchronisation at the end.  Here all rows are sorted by the
// same launches: keys are mapped to order-preserving unsigned integers, a row of up to 4096 columns is sorted
// entirely in shared memory by one CTA, longer rows run the bitonic network with its wide strides in global
// memory and its narrow strides in shared memory.  Ties keep their original order (the reference leaves them
// unspecified).  Nothing synchronises; scratch for long rows comes from the stream-ordered allocator.
#include <stdint.h>

#include "pa_common.cuh"
#include "pa_launch.h"

namespace {

constexpr int SORT_CHUNK = 4096;     // elements one CTA sorts in shared memory (8 + 4 bytes each: 48 KB)
constexpr int SORT_THREADS = 1024;

// ---- order-preserving maps to uint64 and back
template <typename T> struct KeyMap;
template <> struct KeyMap<float> {
  static __device__ uint64_t enc(float v) { uint32_t u = __float_as_uint(v); return u ^ ((u >> 31) ? 0xffffffffu : 0x80000000u); }
  static __device__ float dec(uint64_t k) { uint32_t u = static_cast<uint32_t>(k); return __uint_as_float(u ^ ((u >> 31) ? 0x80000000u : 0xffffffffu)); }
  static constexpr uint64_t mask = 0xffffffffull;
};
template <> struct KeyMap<double> {
  static __device__ uint64_t enc(double v) { uint64_t u = static_cast<uint64_t>(__double_as_longlong(v)); return u ^ ((u >> 63) ? ~0ull : (1ull << 63)); }
  static __device__ double dec(uint64_t u) { return __longlong_as_double(static_cast<long long>(u ^ ((u >> 63) ? (1ull << 63) : ~0ull))); }
  static constexpr uint64_t mask = ~0ull;
};
template <> struct KeyMap<__half> {
  static __device__ uint64_t enc(__half v) { uint16_t u = __half_as_ushort(v); return static_cast<uint16_t>(u ^ ((u >> 15) ? 0xffffu : 0x8000u)); }
  static __device__ __half dec(uint64_t k) { uint16_t u = static_cast<uint16_t>(k); return __ushort_as_half(static_cast<uint16_t>(u ^ ((u >> 15) ? 0x8000u : 0xffffu))); }
  static constexpr uint64_t mask = 0xffffull;
};
template <> struct KeyMap<__nv_bfloat16> {
  static __device__ uint64_t enc(__nv_bfloat16 v) { uint16_t u = __bfloat16_as_ushort(v); return static_cast<uint16_t>(u ^ ((u >> 15) ? 0xffffu : 0x8000u)); }
  static __device__ __nv_bfloat16 dec(uint64_t k) { uint16_t u = static_cast<uint16_t>(k); return __ushort_as_bfloat16(static_cast<uint16_t>(u ^ ((u >> 15) ? 0x8000u : 0xffffu))); }
  static constexpr uint64_t mask = 0xffffull;
};
template <> struct KeyMap<uint8_t> {
  static __device__ uint64_t enc(uint8_t v) { return v; }
  static __device__ uint8_t dec(uint64_t k) { return static_cast<uint8_t>(k); }
  static constexpr uint64_t mask = 0xffull;
};
template <> struct KeyMap<uint32_t> {
  static __device__ uint64_t enc(uint32_t v) { return v; }
  static __device__ uint32_t dec(uint64_t k) { return static_cast<uint32_t>(k); }
  static constexpr uint64_t mask = 0xffffffffull;
};
template <> struct KeyMap<int64_t> {
  static __device__ uint64_t enc(int64_t v) { return static_cast<uint64_t>(v) ^ (1ull << 63); }
  static __device__ int64_t dec(uint64_t k) { return static_cast<int64_t>(k ^ (1ull << 63)); }
  static constexpr uint64_t mask = ~0ull;
};

__device__ __forceinline__ bool before(uint64_t ka, uint32_t ia, uint64_t kb, uint32_t ib) {
  return ka < kb || (ka == kb && ia < ib);
}

// Compare-exchange steps j = j_hi, j_hi / 2, ..., 1 of merge size k on a chunk held in shared memory;
// `base` is the chunk's first position within the (padded) row, which decides the direction.
__device__ __forceinline__ void smem_steps(uint64_t* key, uint32_t* idx, int n_chunk, int64_t base, int64_t k, int j_hi) {
  for (int j = j_hi; j >= 1; j >>= 1) {
    for (int t = threadIdx.x; t < n_chunk / 2; t += blockDim.x) {
      const int i = 2 * t - (t & (j - 1));          // lower element of the t-th pair at stride j
      const int ij = i + j;
      const bool up = ((base + i) & k) == 0;
      const uint64_t ka = key[i], kb = key[ij];
      const uint32_t ia = idx[i], ib = idx[ij];
      if (before(kb, ib, ka, ia) == up) {
        key[i] = kb; key[ij] = ka;
        idx[i] = ib; idx[ij] = ia;
      }
    }
    __syncthreads();
  }
}

// Rows of at most SORT_CHUNK (padded) columns: load, sort and store in one kernel, one CTA per row.
template <typename T, bool ASC>
__global__ void __launch_bounds__(SORT_THREADS)
sort_rows_smem_kernel(T* __restrict__ x, uint32_t* __restrict__ dst, int ncols, int ncols_pad, bool inplace) {
  extern __shared__ __align__(16) unsigned char sort_smem[];
  uint64_t* key = reinterpret_cast<uint64_t*>(sort_smem);
  uint32_t* idx = reinterpret_cast<uint32_t*>(key + ncols_pad);
  T* xr = x + static_cast<int64_t>(blockIdx.x) * ncols;
  uint32_t* dr = dst + static_cast<int64_t>(blockIdx.x) * ncols;
  for (int i = threadIdx.x; i < ncols_pad; i += blockDim.x) {
    uint64_t k = ~0ull;                               // padding sorts last
    if (i < ncols) {
      k = KeyMap<T>::enc(xr[i]);
      if (!ASC) k = (~k) & KeyMap<T>::mask;
    }
    key[i] = k;
    idx[i] = i;
  }
  __syncthreads();
  for (int64_t k = 2; k <= ncols_pad; k <<= 1) smem_steps(key, idx, ncols_pad, 0, k, static_cast<int>(k >> 1));
  for (int i = threadIdx.x; i < ncols; i += blockDim.x) {
    dr[i] = idx[i];
    if (inplace) {
      uint64_t k = key[i];
      if (!ASC) k = (~k) & KeyMap<T>::mask;
      xr[i] = KeyMap<T>::dec(k);
    }
  }
}

// Long rows, phase 1: encode one chunk and sort it in shared memory (all merge sizes up to the chunk).
template <typename T, bool ASC>
__global__ void __launch_bounds__(SORT_THREADS)
sort_chunks_kernel(const T* __restrict__ x, uint64_t* __restrict__ keys, uint32_t* __restrict__ idxs, int ncols, int64_t ncols_pad) {
  __shared__ uint64_t key[SORT_CHUNK];
  __shared__ uint32_t idx[SORT_CHUNK];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * SORT_CHUNK;
  const T* xr = x + static_cast<int64_t>(blockIdx.y) * ncols;
  for (int i = threadIdx.x; i < SORT_CHUNK; i += blockDim.x) {
    const int64_t c = base + i;
    uint64_t k = ~0ull;
    if (c < ncols) {
      k = KeyMap<T>::enc(xr[c]);
      if (!ASC) k = (~k) & KeyMap<T>::mask;
    }
    key[i] = k;
    idx[i] = static_cast<uint32_t>(c);
  }
  __syncthreads();
  for (int64_t k = 2; k <= SORT_CHUNK; k <<= 1) smem_steps(key, idx, SORT_CHUNK, base, k, static_cast<int>(k >> 1));
  uint64_t* kr = keys + static_cast<int64_t>(blockIdx.y) * ncols_pad + base;
  uint32_t* ir = idxs + static_cast<int64_t>(blockIdx.y) * ncols_pad + base;
  for (int i = threadIdx.x; i < SORT_CHUNK; i += blockDim.x) { kr[i] = key[i]; ir[i] = idx[i]; }
}

// Long rows: one compare-exchange step at a stride that spans chunks.
__global__ void sort_global_step_kernel(uint64_t* __restrict__ keys, uint32_t* __restrict__ idxs, int64_t ncols_pad, int64_t j, int64_t k) {
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= ncols_pad / 2) return;
  const int64_t i = 2 * t - (t & (j - 1)), ij = i + j;
  uint64_t* kr = keys + static_cast<int64_t>(blockIdx.y) * ncols_pad;
  uint32_t* ir = idxs + static_cast<int64_t>(blockIdx.y) * ncols_pad;
  const bool up = (i & k) == 0;
  const uint64_t ka = kr[i], kb = kr[ij];
  const uint32_t ia = ir[i], ib = ir[ij];
  if (before(kb, ib, ka, ia) == up) { kr[i] = kb; kr[ij] = ka; ir[i] = ib; ir[ij] = ia; }
}

// Long rows: the remaining steps of merge size k (strides below the chunk size), chunk by chunk in shared memory.
__global__ void __launch_bounds__(SORT_THREADS)
sort_finish_kernel(uint64_t* __restrict__ keys, uint32_t* __restrict__ idxs, int64_t ncols_pad, int64_t k) {
  __shared__ uint64_t key[SORT_CHUNK];
  __shared__ uint32_t idx[SORT_CHUNK];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * SORT_CHUNK;
  uint64_t* kr = keys + static_cast<int64_t>(blockIdx.y) * ncols_pad + base;
  uint32_t* ir = idxs + static_cast<int64_t>(blockIdx.y) * ncols_pad + base;
  for (int i = threadIdx.x; i < SORT_CHUNK; i += blockDim.x) { key[i] = kr[i]; idx[i] = ir[i]; }
  __syncthreads();
  smem_steps(key, idx, SORT_CHUNK, base, k, SORT_CHUNK / 2);
  for (int i = threadIdx.x; i < SORT_CHUNK; i += blockDim.x) { kr[i] = key[i]; ir[i] = idx[i]; }
}

template <typename T, bool ASC>
__global__ void sort_write_kernel(T* __restrict__ x, uint32_t* __restrict__ dst, const uint64_t* __restrict__ keys,
                                  const uint32_t* __restrict__ idxs, int ncols, int64_t ncols_pad, bool inplace) {
  const int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (c >= ncols) return;
  const int64_t row = blockIdx.y;
  dst[row * ncols + c] = idxs[row * ncols_pad + c];
  if (inplace) {
    uint64_t k = keys[row * ncols_pad + c];
    if (!ASC) k = (~k) & KeyMap<T>::mask;
    x[row * ncols + c] = KeyMap<T>::dec(k);
  }
}

template <typename T, bool ASC>
void asort(void* x1, void* dst1, int nrows, int ncols, bool inplace, int64_t stream_) {
  if (nrows <= 0 || ncols <= 0 || !x1 || !dst1) return;
  T* x = reinterpret_cast<T*>(x1);
  uint32_t* dst = reinterpret_cast<uint32_t*>(dst1);
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int64_t pad = 1;
  while (pad < ncols) pad <<= 1;
  if (pad <= SORT_CHUNK) {
    const int smem = static_cast<int>(pad) * 12;
    auto kernel = sort_rows_smem_kernel<T, ASC>;
    const int threads = pad / 2 < SORT_THREADS ? (pad / 2 < 32 ? 32 : static_cast<int>(pad / 2)) : SORT_THREADS;
    kernel<<<nrows, threads, smem, stream>>>(x, dst, ncols, static_cast<int>(pad), inplace);
    return;
  }
  uint64_t* keys = nullptr;
  uint32_t* idxs = nullptr;
  if (cudaMallocAsync(reinterpret_cast<void**>(&keys), sizeof(uint64_t) * pad * nrows, stream) != cudaSuccess) return;
  if (cudaMallocAsync(reinterpret_cast<void**>(&idxs), sizeof(uint32_t) * pad * nrows, stream) != cudaSuccess) {
    cudaFreeAsync(keys, stream);
    return;
  }
  const dim3 cgrid(static_cast<unsigned>(pad / SORT_CHUNK), nrows);
  sort_chunks_kernel<T, ASC><<<cgrid, SORT_THREADS, 0, stream>>>(x, keys, idxs, ncols, pad);
  const dim3 ggrid(static_cast<unsigned>((pad / 2 + 255) / 256), nrows);
  for (int64_t k = 2 * SORT_CHUNK; k <= pad; k <<= 1) {
    for (int64_t j = k >> 1; j >= SORT_CHUNK; j >>= 1) sort_global_step_kernel<<<ggrid, 256, 0, stream>>>(keys, idxs, pad, j, k);
    sort_finish_kernel<<<cgrid, SORT_THREADS, 0, stream>>>(keys, idxs, pad, k);
  }
  const dim3 wgrid(static_cast<unsigned>((ncols + 255) / 256), nrows);
  sort_write_kernel<T, ASC><<<wgrid, 256, 0, stream>>>(x, dst, keys, idxs, ncols, pad, inplace);
  cudaFreeAsync(keys, stream);
  cudaFreeAsync(idxs, stream);
}

}  // namespace

#define PA_ASORT(T, NAME, ASC)                                                                              \
  extern "C" void NAME(void* x, void* dst, const int nrows, const int ncols, bool inplace, int64_t stream) { \
    asort<T, ASC>(x, dst, nrows, ncols, inplace, stream);                                                    \
  }

// The fourteen symbols of src/kernels/src/sort.cu:104-120.
PA_ASORT(__nv_bfloat16, asort_asc_bf16, true)
PA_ASORT(__nv_bfloat16, asort_desc_bf16, false)
PA_ASORT(__half, asort_asc_f16, true)
PA_ASORT(__half, asort_desc_f16, false)
PA_ASORT(float, asort_asc_f32, true)
PA_ASORT(double, asort_asc_f64, true)
PA_ASORT(uint8_t, asort_asc_u8, true)
PA_ASORT(uint32_t, asort_asc_u32, true)
PA_ASORT(int64_t, asort_asc_i64, true)
PA_ASORT(float, asort_desc_f32, false)
PA_ASORT(double, asort_desc_f64, false)
PA_ASORT(uint8_t, asort_desc_u8, false)
PA_ASORT(uint32_t, asort_desc_u32, false)
PA_ASORT(int64_t, asort_desc_i64, false)
