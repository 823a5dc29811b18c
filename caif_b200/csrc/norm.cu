// RMSNorm in front of the frozen projections: CAIF_DevicePreNormBlock normalizes, hands the rows to the
// frozen linear (src/caif_device_pre_norm_block.cpp:97-135) and adds the residual.  The reference's kernels
// (src/caif_cuda_kernels_normalization.cu:46-119 forward, :129-203 backward) run one 256-thread block per row,
// thread t owning columns t, t + 256, ..., and read the row twice from global memory with 2- or 4-byte loads.
//
// Here a CTA walks rows round robin; a row comes in once with 16-byte loads into shared memory, both passes
// read it there, the result leaves with 16-byte stores, and the backward pass keeps its share of grad_gamma in
// registers over all its rows and adds it with one atomic per column at the end (the reference issues one
// atomic per element).  The usual case (even row length, 16-byte aligned rows) runs on 128 threads that each
// play two adjacent threads of the reference's block; the kernels with one thread per reference thread take
// the rest.  The arithmetic of y, rms and dx is the reference's, operation for
// operation: the same columns per thread in the same order with a fused multiply-add per step, the same
// shuffle-down tree inside a warp, the eight warp sums folded by the same tree, IEEE sqrt and divisions -- so
// those three come out bit-identical.  grad_gamma is a sum over rows whose order the reference leaves to its
// atomics; it agrees to rounding.
#include "common.cuh"

namespace caifq
{

namespace
{

constexpr int kNormThreads = 256;
constexpr int kNormWarps = kNormThreads / 32;
constexpr int kNormMaxPerThread = 32;   // columns a thread can keep of grad_gamma: dim <= 8192

template <typename T>
__device__ __forceinline__ float nf(T v);
template <>
__device__ __forceinline__ float nf<float>(float v) { return v; }
template <>
__device__ __forceinline__ float nf<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float nf<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T nt(float v);
template <>
__device__ __forceinline__ float nt<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half nt<__half>(float v) { return __float2half(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 nt<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

// sum over the CTA in the reference's order: shuffle-down tree per warp, then the warp sums in lanes 0..7 of
// warp 0 through the same tree; every thread gets the result
__device__ __forceinline__ float block_sum(float v, float *warp_sums)
{
#pragma unroll
  for (int off = 16; off > 0; off >>= 1)
  {
    v += __shfl_down_sync(0xFFFFFFFFu, v, off);
  }
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  __syncthreads();   // the slot array may still be read from the row before
  if (lane == 0)
  {
    warp_sums[warp] = v;
  }
  __syncthreads();
  if (warp == 0)
  {
    v = lane < kNormWarps ? warp_sums[lane] : 0.0f;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
    {
      v += __shfl_down_sync(0xFFFFFFFFu, v, off);
    }
    if (lane == 0)
    {
      warp_sums[kNormWarps] = v;
    }
  }
  __syncthreads();
  return warp_sums[kNormWarps];
}

// row [dim] of T between global and shared memory with 16-byte accesses when `vec`, else element by element
template <int THREADS, typename T>
__device__ __forceinline__ void row_in(T *dst, const T *src, int dim, bool vec)
{
  if (vec)
  {
    const int n16 = dim * static_cast<int>(sizeof(T)) / 16;
    for (int i = threadIdx.x; i < n16; i += THREADS)
    {
      reinterpret_cast<uint4 *>(dst)[i] = __ldg(reinterpret_cast<const uint4 *>(src) + i);
    }
  }
  else
  {
    for (int i = threadIdx.x; i < dim; i += THREADS)
    {
      dst[i] = src[i];
    }
  }
}

template <int THREADS, typename T>
__device__ __forceinline__ void row_out(T *dst, const T *src, int dim, bool vec)
{
  if (vec)
  {
    const int n16 = dim * static_cast<int>(sizeof(T)) / 16;
    for (int i = threadIdx.x; i < n16; i += THREADS)
    {
      reinterpret_cast<uint4 *>(dst)[i] = reinterpret_cast<const uint4 *>(src)[i];
    }
  }
  else
  {
    for (int i = threadIdx.x; i < dim; i += THREADS)
    {
      dst[i] = src[i];
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kNormThreads, 8)
rmsnorm_fwd_kernel(const T *__restrict__ input, const float *__restrict__ gamma, T *__restrict__ output,
                   float *__restrict__ rms_cache, float epsilon, int rows, int dim, int vec)
{
  extern __shared__ __align__(16) unsigned char norm_smem[];
  __shared__ float warp_sums[kNormWarps + 1];
  T *row = reinterpret_cast<T *>(norm_smem);
  for (int r = blockIdx.x; r < rows; r += gridDim.x)
  {
    __syncthreads();   // the row buffer is free again
    row_in<kNormThreads>(row, input + static_cast<int64_t>(r) * dim, dim, vec != 0);
    __syncthreads();
    float local = 0.0f;
    for (int c = threadIdx.x; c < dim; c += kNormThreads)
    {
      const float v = nf<T>(row[c]);
      local = __fmaf_rn(v, v, local);
    }
    const float total = block_sum(local, warp_sums);
    const float rms = __fsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(dim)), epsilon));
    if (threadIdx.x == 0 && rms_cache != nullptr)
    {
      rms_cache[r] = rms;
    }
    const float rstd = __fdiv_rn(1.0f, rms);
    for (int c = threadIdx.x; c < dim; c += kNormThreads)
    {
      row[c] = nt<T>(__fmul_rn(__fmul_rn(nf<T>(row[c]), rstd), __ldg(gamma + c)));
    }
    __syncthreads();
    row_out<kNormThreads>(output + static_cast<int64_t>(r) * dim, row, dim, vec != 0);
  }
}

// ---- forward with two of the reference's threads per thread ----
// Thread t of 128 plays threads 2t and 2t + 1 of the reference's 256-thread block: their columns are adjacent,
// so one 4-byte (8-byte for fp32) shared-memory access serves both, and the instruction count per element
// halves (the one-thread-per-reference-thread kernel above spent its time on shared-memory latency, not on
// DRAM).  Each of the two partial sums runs over the same columns in the same order; the reference's
// shuffle-down tree over 32 lanes becomes offsets 8, 4, 2, 1 over 16 threads for either sum followed by
// sum0 += sum1, which adds the same pairs in the same order; the eight warp results are folded as before.
constexpr int kPairThreads = 128;

template <typename T>
__device__ __forceinline__ void load2(const T *row, int i, float &a, float &b);
template <>
__device__ __forceinline__ void load2<float>(const float *row, int i, float &a, float &b)
{
  const float2 v = reinterpret_cast<const float2 *>(row)[i];
  a = v.x;
  b = v.y;
}
template <>
__device__ __forceinline__ void load2<__half>(const __half *row, int i, float &a, float &b)
{
  const __half2 h = reinterpret_cast<const __half2 *>(row)[i];
  a = __low2float(h);
  b = __high2float(h);
}
template <>
__device__ __forceinline__ void load2<__nv_bfloat16>(const __nv_bfloat16 *row, int i, float &a, float &b)
{
  const uint32_t w = reinterpret_cast<const uint32_t *>(row)[i];
  a = __uint_as_float(w << 16);
  b = __uint_as_float(w & 0xFFFF0000u);
}

template <typename T>
__device__ __forceinline__ void store2(T *row, int i, float a, float b);
template <>
__device__ __forceinline__ void store2<float>(float *row, int i, float a, float b)
{
  reinterpret_cast<float2 *>(row)[i] = make_float2(a, b);
}
template <>
__device__ __forceinline__ void store2<__half>(__half *row, int i, float a, float b)
{
  reinterpret_cast<__half2 *>(row)[i] = __floats2half2_rn(a, b);
}
template <>
__device__ __forceinline__ void store2<__nv_bfloat16>(__nv_bfloat16 *row, int i, float a, float b)
{
  reinterpret_cast<__nv_bfloat162 *>(row)[i] = __floats2bfloat162_rn(a, b);
}

template <typename T>
__global__ void __launch_bounds__(kPairThreads, 16)
rmsnorm_fwd_pair_kernel(const T *__restrict__ input, const float *__restrict__ gamma, T *__restrict__ output,
                        float *__restrict__ rms_cache, float epsilon, int rows, int dim)
{
  extern __shared__ __align__(16) unsigned char norm_smem[];
  __shared__ float warp_sums[kNormWarps + 1];
  T *row = reinterpret_cast<T *>(norm_smem);
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int pairs = dim >> 1;
  for (int r = blockIdx.x; r < rows; r += gridDim.x)
  {
    __syncthreads();   // the row buffer and the slot array are free again
    row_in<kPairThreads>(row, input + static_cast<int64_t>(r) * dim, dim, true);
    __syncthreads();
    float s0 = 0.0f;
    float s1 = 0.0f;
    for (int i = tid; i < pairs; i += kPairThreads)
    {
      float a, b;
      load2<T>(row, i, a, b);
      s0 = __fmaf_rn(a, a, s0);
      s1 = __fmaf_rn(b, b, s1);
    }
#pragma unroll
    for (int off = 8; off > 0; off >>= 1)
    {
      s0 += __shfl_down_sync(0xFFFFFFFFu, s0, off, 16);
      s1 += __shfl_down_sync(0xFFFFFFFFu, s1, off, 16);
    }
    s0 += s1;
    if ((tid & 15) == 0)
    {
      warp_sums[tid >> 4] = s0;   // lane 0 of the reference's warp tid / 16
    }
    __syncthreads();
    if (tid < 32)
    {
      float v = lane < kNormWarps ? warp_sums[lane] : 0.0f;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
      {
        v += __shfl_down_sync(0xFFFFFFFFu, v, off);
      }
      if (lane == 0)
      {
        warp_sums[kNormWarps] = v;
      }
    }
    __syncthreads();
    const float rms = __fsqrt_rn(__fadd_rn(__fdiv_rn(warp_sums[kNormWarps], static_cast<float>(dim)), epsilon));
    if (tid == 0 && rms_cache != nullptr)
    {
      rms_cache[r] = rms;
    }
    const float rstd = __fdiv_rn(1.0f, rms);
    for (int i = tid; i < pairs; i += kPairThreads)
    {
      float a, b;
      load2<T>(row, i, a, b);
      const float2 g = __ldg(reinterpret_cast<const float2 *>(gamma) + i);
      store2<T>(row, i, __fmul_rn(__fmul_rn(a, rstd), g.x), __fmul_rn(__fmul_rn(b, rstd), g.y));
    }
    __syncthreads();
    row_out<kPairThreads>(output + static_cast<int64_t>(r) * dim, row, dim, true);
  }
}

// dy * gamma - x_hat * sum_term is evaluated as fma(dy, gamma, -(x_hat * sum_term)): the fusion the reference
// build makes of that expression (of the three possible evaluations only this one reproduces its dx bit for bit,
// fp32 and bf16).
template <typename T>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_kernel(const T *__restrict__ grad_output, const T *__restrict__ input, const float *__restrict__ gamma,
                   const float *__restrict__ rms_cache, T *__restrict__ grad_input, float *__restrict__ grad_gamma,
                   int rows, int dim, int vec)
{
  extern __shared__ __align__(16) unsigned char norm_smem[];
  __shared__ float warp_sums[kNormWarps + 1];
  T *xrow = reinterpret_cast<T *>(norm_smem);
  T *grow = xrow + dim;
  float gg[kNormMaxPerThread];
#pragma unroll
  for (int j = 0; j < kNormMaxPerThread; ++j)
  {
    gg[j] = 0.0f;
  }
  for (int r = blockIdx.x; r < rows; r += gridDim.x)
  {
    __syncthreads();
    row_in<kNormThreads>(xrow, input + static_cast<int64_t>(r) * dim, dim, vec != 0);
    row_in<kNormThreads>(grow, grad_output + static_cast<int64_t>(r) * dim, dim, vec != 0);
    __syncthreads();
    const float rstd = __fdiv_rn(1.0f, __ldg(rms_cache + r));
    float local = 0.0f;
    for (int c = threadIdx.x; c < dim; c += kNormThreads)
    {
      const float x_hat = __fmul_rn(nf<T>(xrow[c]), rstd);
      local = __fmaf_rn(__fmul_rn(nf<T>(grow[c]), __ldg(gamma + c)), x_hat, local);
    }
    const float sum_term = __fdiv_rn(block_sum(local, warp_sums), static_cast<float>(dim));
#pragma unroll
    for (int j = 0; j < kNormMaxPerThread; ++j)
    {
      const int c = threadIdx.x + j * kNormThreads;
      if (c < dim)
      {
        const float x_hat = __fmul_rn(nf<T>(xrow[c]), rstd);
        const float dy = nf<T>(grow[c]);
        const float g = __ldg(gamma + c);
        const float inner = __fmaf_rn(dy, g, -__fmul_rn(x_hat, sum_term));
        gg[j] = __fmaf_rn(dy, x_hat, gg[j]);
        xrow[c] = nt<T>(__fmul_rn(rstd, inner));
      }
    }
    __syncthreads();
    row_out<kNormThreads>(grad_input + static_cast<int64_t>(r) * dim, xrow, dim, vec != 0);
  }
  if (grad_gamma != nullptr)
  {
#pragma unroll
    for (int j = 0; j < kNormMaxPerThread; ++j)
    {
      const int c = threadIdx.x + j * kNormThreads;
      if (c < dim)
      {
        atomicAdd(grad_gamma + c, gg[j]);
      }
    }
  }
}

// backward with two of the reference's threads per thread (rows up to 4096 wide: a thread keeps 32 sums of
// grad_gamma); same reading as the paired forward kernel
constexpr int kPairMaxTrips = kNormMaxPerThread / 2;

template <typename T>
__global__ void __launch_bounds__(kPairThreads, 6)
rmsnorm_bwd_pair_kernel(const T *__restrict__ grad_output, const T *__restrict__ input,
                        const float *__restrict__ gamma, const float *__restrict__ rms_cache,
                        T *__restrict__ grad_input, float *__restrict__ grad_gamma, int rows, int dim)
{
  extern __shared__ __align__(16) unsigned char norm_smem[];
  __shared__ float warp_sums[kNormWarps + 1];
  T *xrow = reinterpret_cast<T *>(norm_smem);
  T *grow = xrow + dim;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int pairs = dim >> 1;
  float gg[kNormMaxPerThread];
#pragma unroll
  for (int j = 0; j < kNormMaxPerThread; ++j)
  {
    gg[j] = 0.0f;
  }
  for (int r = blockIdx.x; r < rows; r += gridDim.x)
  {
    __syncthreads();
    row_in<kPairThreads>(xrow, input + static_cast<int64_t>(r) * dim, dim, true);
    row_in<kPairThreads>(grow, grad_output + static_cast<int64_t>(r) * dim, dim, true);
    __syncthreads();
    const float rstd = __fdiv_rn(1.0f, __ldg(rms_cache + r));
    float s0 = 0.0f;
    float s1 = 0.0f;
    for (int i = tid; i < pairs; i += kPairThreads)
    {
      float xa, xb, da, db;
      load2<T>(xrow, i, xa, xb);
      load2<T>(grow, i, da, db);
      const float2 g = __ldg(reinterpret_cast<const float2 *>(gamma) + i);
      s0 = __fmaf_rn(__fmul_rn(da, g.x), __fmul_rn(xa, rstd), s0);
      s1 = __fmaf_rn(__fmul_rn(db, g.y), __fmul_rn(xb, rstd), s1);
    }
#pragma unroll
    for (int off = 8; off > 0; off >>= 1)
    {
      s0 += __shfl_down_sync(0xFFFFFFFFu, s0, off, 16);
      s1 += __shfl_down_sync(0xFFFFFFFFu, s1, off, 16);
    }
    s0 += s1;
    if ((tid & 15) == 0)
    {
      warp_sums[tid >> 4] = s0;
    }
    __syncthreads();
    if (tid < 32)
    {
      float v = lane < kNormWarps ? warp_sums[lane] : 0.0f;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
      {
        v += __shfl_down_sync(0xFFFFFFFFu, v, off);
      }
      if (lane == 0)
      {
        warp_sums[kNormWarps] = v;
      }
    }
    __syncthreads();
    const float sum_term = __fdiv_rn(warp_sums[kNormWarps], static_cast<float>(dim));
#pragma unroll
    for (int j = 0; j < kPairMaxTrips; ++j)
    {
      const int i = tid + j * kPairThreads;
      if (i < pairs)
      {
        float xa, xb, da, db;
        load2<T>(xrow, i, xa, xb);
        load2<T>(grow, i, da, db);
        const float2 g = __ldg(reinterpret_cast<const float2 *>(gamma) + i);
        const float ha = __fmul_rn(xa, rstd);
        const float hb = __fmul_rn(xb, rstd);
        gg[2 * j] = __fmaf_rn(da, ha, gg[2 * j]);
        gg[2 * j + 1] = __fmaf_rn(db, hb, gg[2 * j + 1]);
        store2<T>(xrow, i, __fmul_rn(rstd, __fmaf_rn(da, g.x, -__fmul_rn(ha, sum_term))),
                  __fmul_rn(rstd, __fmaf_rn(db, g.y, -__fmul_rn(hb, sum_term))));
      }
    }
    __syncthreads();
    row_out<kPairThreads>(grad_input + static_cast<int64_t>(r) * dim, xrow, dim, true);
  }
  if (grad_gamma != nullptr)
  {
#pragma unroll
    for (int j = 0; j < kPairMaxTrips; ++j)
    {
      const int i = tid + j * kPairThreads;
      if (i < pairs)
      {
        atomicAdd(grad_gamma + 2 * i, gg[2 * j]);
        atomicAdd(grad_gamma + 2 * i + 1, gg[2 * j + 1]);
      }
    }
  }
}

int norm_grid(int rows, int ctas_per_sm)
{
  const int cap = 148 * ctas_per_sm;
  return rows < cap ? rows : cap;
}

bool rows_vectorizable(const void *a, const void *b, int dim, size_t elem)
{
  return (dim * elem) % 16 == 0 && (reinterpret_cast<uintptr_t>(a) & 15u) == 0 &&
         (reinterpret_cast<uintptr_t>(b) & 15u) == 0;
}

}  // namespace

int launch_rmsnorm_fwd(const void *input, const float *gamma, void *output, float *rms_cache, float epsilon, int dtype,
                       int rows, int dim, cudaStream_t s)
{
  if (rows <= 0)
  {
    return CAIFQ_OK;
  }
  const size_t elem = (dtype == CAIFQ_F32) ? 4 : 2;
  const size_t smem = static_cast<size_t>(dim) * elem;
  if (smem > 96 * 1024)
  {
    set_error("rmsnorm: rows of %d elements do not fit the row buffer", dim);
    return CAIFQ_ERR_UNSUPPORTED;
  }
  const int vec = rows_vectorizable(input, output, dim, elem) ? 1 : 0;
  const bool pair = vec != 0 && (dim % 2) == 0 && (reinterpret_cast<uintptr_t>(gamma) & 7u) == 0;
#define CAIFQ_NORM_FWD(T)                                                                                        \
  {                                                                                                               \
    if (smem > 48 * 1024)                                                                                         \
    {                                                                                                             \
      cudaFuncSetAttribute(rmsnorm_fwd_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);        \
    }                                                                                                             \
    if (pair)                                                                                                     \
    {                                                                                                             \
      if (smem > 48 * 1024)                                                                                       \
      {                                                                                                           \
        cudaFuncSetAttribute(rmsnorm_fwd_pair_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); \
      }                                                                                                           \
      rmsnorm_fwd_pair_kernel<T><<<norm_grid(rows, 16), kPairThreads, smem, s>>>(                                 \
          static_cast<const T *>(input), gamma, static_cast<T *>(output), rms_cache, epsilon, rows, dim);         \
    }                                                                                                             \
    else                                                                                                          \
    {                                                                                                             \
      rmsnorm_fwd_kernel<T><<<norm_grid(rows, 8), kNormThreads, smem, s>>>(static_cast<const T *>(input), gamma,  \
                                                                           static_cast<T *>(output), rms_cache,   \
                                                                           epsilon, rows, dim, vec);              \
    }                                                                                                             \
  }
  if (dtype == CAIFQ_F32)
    CAIFQ_NORM_FWD(float)
  else if (dtype == CAIFQ_F16)
    CAIFQ_NORM_FWD(__half)
  else
    CAIFQ_NORM_FWD(__nv_bfloat16)
#undef CAIFQ_NORM_FWD
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_rmsnorm_bwd(const void *grad_output, const void *input, const float *gamma, const float *rms_cache,
                       void *grad_input, float *grad_gamma, int dtype, int rows, int dim, cudaStream_t s)
{
  if (rows <= 0)
  {
    return CAIFQ_OK;
  }
  const size_t elem = (dtype == CAIFQ_F32) ? 4 : 2;
  const size_t smem = 2 * static_cast<size_t>(dim) * elem;
  if (smem > 96 * 1024 || dim > kNormThreads * kNormMaxPerThread)
  {
    set_error("rmsnorm backward: rows of %d elements are too long", dim);
    return CAIFQ_ERR_UNSUPPORTED;
  }
  const int vec = (rows_vectorizable(input, grad_input, dim, elem) && rows_vectorizable(grad_output, grad_output, dim, elem))
                      ? 1
                      : 0;
  const bool pair = vec != 0 && (dim % 2) == 0 && dim <= kPairThreads * 2 * kPairMaxTrips && smem <= 48 * 1024 &&
                    (reinterpret_cast<uintptr_t>(gamma) & 7u) == 0;
#define CAIFQ_NORM_BWD(T)                                                                                        \
  {                                                                                                               \
    if (pair)                                                                                                     \
    {                                                                                                             \
      rmsnorm_bwd_pair_kernel<T><<<norm_grid(rows, 6), kPairThreads, smem, s>>>(                                  \
          static_cast<const T *>(grad_output), static_cast<const T *>(input), gamma, rms_cache,                   \
          static_cast<T *>(grad_input), grad_gamma, rows, dim);                                                   \
    }                                                                                                             \
    else                                                                                                          \
    {                                                                                                             \
      if (smem > 48 * 1024)                                                                                       \
      {                                                                                                           \
        cudaFuncSetAttribute(rmsnorm_bwd_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);      \
      }                                                                                                           \
      rmsnorm_bwd_kernel<T><<<norm_grid(rows, 4), kNormThreads, smem, s>>>(                                       \
          static_cast<const T *>(grad_output), static_cast<const T *>(input), gamma, rms_cache,                   \
          static_cast<T *>(grad_input), grad_gamma, rows, dim, vec);                                              \
    }                                                                                                             \
  }
  if (dtype == CAIFQ_F32)
    CAIFQ_NORM_BWD(float)
  else if (dtype == CAIFQ_F16)
    CAIFQ_NORM_BWD(__half)
  else
    CAIFQ_NORM_BWD(__nv_bfloat16)
#undef CAIFQ_NORM_BWD
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

}  // namespace caifq
