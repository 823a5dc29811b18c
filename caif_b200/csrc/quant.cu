// Quantize / dequantize / cast kernels.
//
// Results are bit-identical to the reference's kernels in
// src/caif_cuda_kernels_quant.cu (same fp32 operations in the same order per
// element; only the parallel decomposition differs):
//   int8 per-tensor   :384-483    int8 per-channel  :502-620
//   int4 per-group    :205-362    casts             :38-199
// The reference quantizes int4 with one thread per group and serial 128-element
// loops; here a warp owns a group (coalesced float4/float2 loads, shuffle
// max-reduce), which is what makes load-time quantization of a multi-GB model
// bandwidth-bound instead of latency-bound.
#include "common.cuh"

namespace caifq
{

namespace
{

constexpr int kBlock = 256;

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
  {
    v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  }
  return v;
}

// |x| maximum that ignores NaN exactly like `if (fabsf(x) > m) m = fabsf(x)`.
__device__ __forceinline__ float absmax_step(float m, float x)
{
  const float a = fabsf(x);
  return (a > m) ? a : m;
}

__device__ __forceinline__ float clamp_sym(float v, float lim)
{
  if (v > lim)
  {
    v = lim;
  }
  else if (v < -lim)
  {
    v = -lim;
  }
  return v;
}

// ---------------------------------------------------------------- int8 / tensor

// scale[0] accumulates max|x| through an integer atomicMax on the bit pattern
// (non-negative floats order like ints), as the reference does.
__global__ void absmax_kernel(const float *__restrict__ x, float *scale, int64_t n)
{
  float m = 0.0f;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t n4 = n >> 2;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) == 0)
  {
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    for (int64_t j = i; j < n4; j += stride)
    {
      const float4 v = x4[j];
      m = absmax_step(absmax_step(absmax_step(absmax_step(m, v.x), v.y), v.z), v.w);
    }
    for (int64_t j = (n4 << 2) + i; j < n; j += stride)
    {
      m = absmax_step(m, x[j]);
    }
  }
  else
  {
    for (; i < n; i += stride)
    {
      m = absmax_step(m, x[i]);
    }
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0 && m > 0.0f)
  {
    atomicMax(reinterpret_cast<int *>(scale), __float_as_int(m));
  }
}

__global__ void finalize_scale_kernel(float *scale)
{
  const float m = scale[0];
  scale[0] = (m > 0.0f) ? __fdiv_rn(m, 127.0f) : 1.0f;
}

__global__ void quantize_int8_pt_kernel(const float *__restrict__ x, int8_t *__restrict__ q,
                                        const float *__restrict__ scale, int64_t n)
{
  const float s = scale[0];
  const float inv = (s > 0.0f) ? __fdiv_rn(1.0f, s) : 0.0f;
  const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i + 3 < n && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(q)) & 15u) == 0)
  {
    const float4 v = *reinterpret_cast<const float4 *>(x + i);
    char4 o;
    o.x = static_cast<int8_t>(rintf(clamp_sym(__fmul_rn(v.x, inv), 127.0f)));
    o.y = static_cast<int8_t>(rintf(clamp_sym(__fmul_rn(v.y, inv), 127.0f)));
    o.z = static_cast<int8_t>(rintf(clamp_sym(__fmul_rn(v.z, inv), 127.0f)));
    o.w = static_cast<int8_t>(rintf(clamp_sym(__fmul_rn(v.w, inv), 127.0f)));
    *reinterpret_cast<char4 *>(q + i) = o;
  }
  else
  {
    for (int64_t j = i; j < n && j < i + 4; ++j)
    {
      q[j] = static_cast<int8_t>(rintf(clamp_sym(__fmul_rn(x[j], inv), 127.0f)));
    }
  }
}

__global__ void dequantize_int8_pt_kernel(const int8_t *__restrict__ q, float *__restrict__ out,
                                          const float *__restrict__ scale, int64_t n)
{
  const float s = scale[0];
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
  {
    out[i] = __fmul_rn(static_cast<float>(q[i]), s);
  }
}

// --------------------------------------------------------------- int8 / channel

// One thread per column, rows walked in order: neighbouring threads read
// neighbouring columns, so each row pass is coalesced.
__global__ void channel_scale_kernel(const float *__restrict__ x, float *__restrict__ scales, int rows, int cols)
{
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols)
  {
    return;
  }
  float m = 0.0f;
  for (int r = 0; r < rows; ++r)
  {
    m = absmax_step(m, x[static_cast<int64_t>(r) * cols + c]);
  }
  scales[c] = (m > 0.0f) ? __fdiv_rn(m, 127.0f) : 1.0f;
}

__global__ void quantize_int8_pc_kernel(const float *__restrict__ x, int8_t *__restrict__ q,
                                        const float *__restrict__ scales, int64_t total, int cols)
{
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
  {
    const float s = scales[i % cols];
    const float inv = (s > 0.0f) ? __fdiv_rn(1.0f, s) : 0.0f;
    q[i] = static_cast<int8_t>(rintf(clamp_sym(__fmul_rn(x[i], inv), 127.0f)));
  }
}

__global__ void dequantize_int8_pc_kernel(const int8_t *__restrict__ q, float *__restrict__ out,
                                          const float *__restrict__ scales, int64_t total, int cols)
{
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
  {
    out[i] = __fmul_rn(static_cast<float>(q[i]), scales[i % cols]);
  }
}

// ------------------------------------------------------------------ int4 / group

__device__ __forceinline__ int quant_nibble(float x, float inv)
{
  return static_cast<int>(rintf(clamp_sym(__fmul_rn(x, inv), 7.0f))) & 0xF;
}

// Even group size: a warp per group, lanes take element pairs (one byte each).
__global__ void quantize_int4_warp_kernel(const float *__restrict__ x, uint8_t *__restrict__ packed,
                                          __half *__restrict__ scales, int64_t n, int group, int64_t num_groups)
{
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t g = warp; g < num_groups; g += warps)
  {
    const int64_t start = g * group;
    const int64_t end = (start + group < n) ? (start + group) : n;
    float m = 0.0f;
    for (int64_t i = start + 2 * lane; i < end; i += 64)
    {
      m = absmax_step(m, x[i]);
      if (i + 1 < end)
      {
        m = absmax_step(m, x[i + 1]);
      }
    }
    m = warp_max(m);
    const float scale = (m == 0.0f) ? 0.0f : __fdiv_rn(m, 7.0f);
    const float inv = (scale == 0.0f) ? 0.0f : __fdiv_rn(1.0f, scale);
    if (lane == 0)
    {
      scales[g] = __float2half(scale);
    }
    for (int64_t i = start + 2 * lane; i < end; i += 64)
    {
      const int q0 = quant_nibble(x[i], inv);
      const int q1 = (i + 1 < end) ? quant_nibble(x[i + 1], inv) : 0;
      packed[i >> 1] = static_cast<uint8_t>(q0 | (q1 << 4));
    }
  }
}

// Odd group size: groups share bytes; keep the reference's thread-per-group
// form so the result is whatever the reference's write order yields.
__global__ void quantize_int4_serial_kernel(const float *__restrict__ x, uint8_t *__restrict__ packed,
                                            __half *__restrict__ scales, int64_t n, int group, int64_t num_groups)
{
  const int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (g >= num_groups)
  {
    return;
  }
  const int64_t start = g * group;
  const int64_t end = (start + group < n) ? (start + group) : n;
  float m = 0.0f;
  for (int64_t i = start; i < end; ++i)
  {
    m = absmax_step(m, x[i]);
  }
  const float scale = (m == 0.0f) ? 0.0f : __fdiv_rn(m, 7.0f);
  const float inv = (scale == 0.0f) ? 0.0f : __fdiv_rn(1.0f, scale);
  scales[g] = __float2half(scale);
  for (int64_t i = start; i < end; i += 2)
  {
    const int q0 = quant_nibble(x[i], inv);
    const int q1 = (i + 1 < end) ? quant_nibble(x[i + 1], inv) : 0;
    packed[i >> 1] = static_cast<uint8_t>(q0 | (q1 << 4));
  }
}

__global__ void dequantize_int4_kernel(const uint8_t *__restrict__ packed, const __half *__restrict__ scales,
                                       float *__restrict__ out, int64_t n, int group)
{
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  // one byte (two elements) per thread-iteration
  const int64_t nbytes = (n + 1) >> 1;
  for (int64_t b = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; b < nbytes; b += stride)
  {
    const uint8_t v = packed[b];
    const int64_t i0 = b << 1;
    out[i0] = __fmul_rn(static_cast<float>(sign_extend_nibble(v & 0xF)), __half2float(scales[i0 / group]));
    if (i0 + 1 < n)
    {
      out[i0 + 1] = __fmul_rn(static_cast<float>(sign_extend_nibble(v >> 4)), __half2float(scales[(i0 + 1) / group]));
    }
  }
}

// ------------------------------------------------------------------------ casts

template <typename S, typename D>
__device__ __forceinline__ D cast_one(S v);

template <>
__device__ __forceinline__ float cast_one<float, float>(float v) { return v; }
template <>
__device__ __forceinline__ __half cast_one<float, __half>(float v) { return __float2half(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 cast_one<float, __nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <>
__device__ __forceinline__ int8_t cast_one<float, int8_t>(float v)
{
  return static_cast<int8_t>(rintf(clamp_sym(v, 127.0f)));
}
template <>
__device__ __forceinline__ float cast_one<__half, float>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float cast_one<__nv_bfloat16, float>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float cast_one<int8_t, float>(int8_t v) { return static_cast<float>(v); }

// Any pair goes through fp32, which is how CAIF_DeviceTensor::To composes them.
template <typename S, typename D>
__global__ void cast_kernel(const S *__restrict__ src, D *__restrict__ dst, int64_t n)
{
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
  {
    dst[i] = cast_one<float, D>(cast_one<S, float>(src[i]));
  }
}

template <int STORAGE>
__global__ void materialize_kernel(caifq_weight w, void *dst, int dst_dtype, int64_t total)
{
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
  {
    store_from_float(dst, i, dst_dtype, weight_value<STORAGE>(w, i));
  }
}

inline int grid_for(int64_t n, int per_thread = 1)
{
  const int64_t threads = (n + per_thread - 1) / per_thread;
  int64_t g = (threads + kBlock - 1) / kBlock;
  const int64_t cap = 148 * 16;
  if (g > cap)
  {
    g = cap;
  }
  if (g < 1)
  {
    g = 1;
  }
  return static_cast<int>(g);
}

template <typename S>
int cast_from(const S *src, void *dst, int dst_dtype, int64_t n, cudaStream_t s)
{
  const int g = grid_for(n);
  switch (dst_dtype)
  {
    case CAIFQ_F32:
      cast_kernel<S, float><<<g, kBlock, 0, s>>>(src, static_cast<float *>(dst), n);
      break;
    case CAIFQ_F16:
      cast_kernel<S, __half><<<g, kBlock, 0, s>>>(src, static_cast<__half *>(dst), n);
      break;
    case CAIFQ_BF16:
      cast_kernel<S, __nv_bfloat16><<<g, kBlock, 0, s>>>(src, static_cast<__nv_bfloat16 *>(dst), n);
      break;
    case CAIFQ_I8:
      cast_kernel<S, int8_t><<<g, kBlock, 0, s>>>(src, static_cast<int8_t *>(dst), n);
      break;
    default:
      set_error("caifq_cast: unsupported destination dtype %d", dst_dtype);
      return CAIFQ_ERR_INVALID;
  }
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

}  // namespace

int launch_quantize_int8_per_tensor(const float *x, int8_t *q, float *scale, int64_t n, cudaStream_t s)
{
  if (n <= 0)
  {
    return CAIFQ_OK;
  }
  CAIFQ_CHECK_CUDA(cudaMemsetAsync(scale, 0, sizeof(float), s));
  absmax_kernel<<<grid_for(n, 16), kBlock, 0, s>>>(x, scale, n);
  CAIFQ_CHECK_LAUNCH();
  finalize_scale_kernel<<<1, 1, 0, s>>>(scale);
  CAIFQ_CHECK_LAUNCH();
  const int64_t threads = (n + 3) / 4;
  const int64_t grid = (threads + kBlock - 1) / kBlock;
  quantize_int8_pt_kernel<<<static_cast<unsigned>(grid), kBlock, 0, s>>>(x, q, scale, n);
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_dequantize_int8_per_tensor(const int8_t *q, float *out, const float *scale, int64_t n, cudaStream_t s)
{
  if (n <= 0)
  {
    return CAIFQ_OK;
  }
  dequantize_int8_pt_kernel<<<grid_for(n), kBlock, 0, s>>>(q, out, scale, n);
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_quantize_int8_per_channel(const float *x, int8_t *q, float *scales, int rows, int cols, cudaStream_t s)
{
  if (rows <= 0 || cols <= 0)
  {
    return CAIFQ_OK;
  }
  channel_scale_kernel<<<(cols + kBlock - 1) / kBlock, kBlock, 0, s>>>(x, scales, rows, cols);
  CAIFQ_CHECK_LAUNCH();
  const int64_t total = static_cast<int64_t>(rows) * cols;
  quantize_int8_pc_kernel<<<grid_for(total), kBlock, 0, s>>>(x, q, scales, total, cols);
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_dequantize_int8_per_channel(const int8_t *q, float *out, const float *scales, int rows, int cols,
                                       cudaStream_t s)
{
  if (rows <= 0 || cols <= 0)
  {
    return CAIFQ_OK;
  }
  const int64_t total = static_cast<int64_t>(rows) * cols;
  dequantize_int8_pc_kernel<<<grid_for(total), kBlock, 0, s>>>(q, out, scales, total, cols);
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_quantize_int4(const float *x, uint8_t *packed, uint16_t *scales, int64_t n, int group, cudaStream_t s)
{
  if (n <= 0)
  {
    return CAIFQ_OK;
  }
  const int64_t num_groups = (n + group - 1) / group;
  if ((group & 1) == 0)
  {
    const int64_t blocks = (num_groups + (kBlock / 32) - 1) / (kBlock / 32);
    const int64_t cap = 148 * 32;
    quantize_int4_warp_kernel<<<static_cast<unsigned>(blocks < cap ? blocks : cap), kBlock, 0, s>>>(
        x, packed, reinterpret_cast<__half *>(scales), n, group, num_groups);
  }
  else
  {
    quantize_int4_serial_kernel<<<static_cast<unsigned>((num_groups + kBlock - 1) / kBlock), kBlock, 0, s>>>(
        x, packed, reinterpret_cast<__half *>(scales), n, group, num_groups);
  }
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_dequantize_int4(const uint8_t *packed, const uint16_t *scales, float *out, int64_t n, int group,
                           cudaStream_t s)
{
  if (n <= 0)
  {
    return CAIFQ_OK;
  }
  dequantize_int4_kernel<<<grid_for((n + 1) / 2), kBlock, 0, s>>>(packed, reinterpret_cast<const __half *>(scales),
                                                                  out, n, group);
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_cast(const void *src, int src_dtype, void *dst, int dst_dtype, int64_t n, cudaStream_t s)
{
  if (n <= 0)
  {
    return CAIFQ_OK;
  }
  switch (src_dtype)
  {
    case CAIFQ_F32:
      return cast_from(static_cast<const float *>(src), dst, dst_dtype, n, s);
    case CAIFQ_F16:
      return cast_from(static_cast<const __half *>(src), dst, dst_dtype, n, s);
    case CAIFQ_BF16:
      return cast_from(static_cast<const __nv_bfloat16 *>(src), dst, dst_dtype, n, s);
    case CAIFQ_I8:
      return cast_from(static_cast<const int8_t *>(src), dst, dst_dtype, n, s);
    default:
      set_error("caifq_cast: unsupported source dtype %d", src_dtype);
      return CAIFQ_ERR_INVALID;
  }
}

// ---- codes -> bf16 operand matrix (many-token calls expand the weight once per call / step) ----
// One thread per 16 bytes of OUTPUT (eight weights: 8 bytes of int8 codes or 4 bytes of int4 codes), so a
// warp reads 256 / 128 contiguous bytes and writes 512 contiguous bytes per instruction.  int8: exact bf16
// integers with byte permutes and one bf16 subtraction per pair.  int4: the offset-binary nibble is dropped
// into the mantissa of 2^23 (exact), 2^23 + 8 subtracted (exact), the product with the group's fp16 scale
// rounded once in fp32 and once to bf16 -- the value the reference's dequantize kernel followed by its cast
// to bf16 gives (src/caif_cuda_kernels_quant.cu:364-420, src/caif_device_frozen_linear.cpp:319-334).
// `units` = weights / 8 of one matrix; blockIdx.y selects the matrix (expert) of a stacked run
constexpr int kExpandGroup = 64;
struct ExpandTable
{
  const void *codes[kExpandGroup];
  const __half *scales[kExpandGroup];
};

template <int STORAGE>
__global__ void expand_kernel(const __grid_constant__ ExpandTable t, uint4 *dst, int64_t units, int group_size)
{
  const int e = blockIdx.y;
  uint4 *out = dst + static_cast<int64_t>(e) * units;
  // four units per thread and trip, a block width apart: all four loads are in flight before the first
  // conversion, and a warp's accesses stay contiguous
  constexpr int kPerTrip = 4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x * kPerTrip;
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * blockDim.x * kPerTrip + threadIdx.x; base < units;
       base += stride)
  {
    if (STORAGE == CAIFQ_I8)
    {
      uint2 c[kPerTrip];
#pragma unroll
      for (int u = 0; u < kPerTrip; ++u)
      {
        const int64_t i = base + static_cast<int64_t>(u) * blockDim.x;
        c[u] = (i < units) ? __ldg(static_cast<const uint2 *>(t.codes[e]) + i) : make_uint2(0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < kPerTrip; ++u)
      {
        const int64_t i = base + static_cast<int64_t>(u) * blockDim.x;
        if (i < units)
        {
          out[i] = expand_int8x8(c[u]);
        }
      }
    }
    else
    {
      uint32_t c[kPerTrip];
      __half sc[kPerTrip];
#pragma unroll
      for (int u = 0; u < kPerTrip; ++u)
      {
        const int64_t i = base + static_cast<int64_t>(u) * blockDim.x;
        c[u] = 0u;
        sc[u] = __half();
        if (i < units)
        {
          c[u] = __ldg(static_cast<const uint32_t *>(t.codes[e]) + i);
          sc[u] = __ldg(t.scales[e] + (i * 8) / group_size);   // eight codes lie in one group
        }
      }
#pragma unroll
      for (int u = 0; u < kPerTrip; ++u)
      {
        const int64_t i = base + static_cast<int64_t>(u) * blockDim.x;
        if (i < units)
        {
          out[i] = expand_int4x8(c[u], __half2float(sc[u]));
        }
      }
    }
  }
}

int launch_expand_grouped_to_bf16(const caifq_weight *ws, int count, void *dst, cudaStream_t s)
{
  const caifq_weight &w0 = ws[0];
  const int64_t total = static_cast<int64_t>(w0.in_dim) * w0.out_dim;
  const bool i8 = (w0.storage == CAIFQ_I8);
  if ((total % 8) != 0 || (!i8 && !(w0.storage == CAIFQ_I4 && w0.group_size > 0 && (w0.group_size % 8) == 0)))
  {
    set_error("expand_to_bf16: unsupported weight (storage %d)", w0.storage);
    return CAIFQ_ERR_UNSUPPORTED;
  }
  const int64_t units = total / 8;
  for (int first = 0; first < count; first += kExpandGroup)
  {
    const int n = (count - first < kExpandGroup) ? (count - first) : kExpandGroup;
    ExpandTable t{};
    for (int e = 0; e < n; ++e)
    {
      t.codes[e] = ws[first + e].codes;
      t.scales[e] = static_cast<const __half *>(ws[first + e].scales);
      if (!i8 && t.scales[e] == nullptr)
      {
        set_error("expand_to_bf16: int4 weight %d has no scales", first + e);
        return CAIFQ_ERR_INVALID;
      }
      if ((reinterpret_cast<uintptr_t>(t.codes[e]) & 7u) != 0)
      {
        set_error("expand_to_bf16: codes of weight %d are not 8-byte aligned", first + e);
        return CAIFQ_ERR_INVALID;
      }
    }
    int gx = grid_for(units);
    const int cap = (148 * 8 + n - 1) / n;   // about eight CTAs per SM over all matrices
    if (gx > cap)
    {
      gx = cap;
    }
    uint4 *out = static_cast<uint4 *>(dst) + static_cast<int64_t>(first) * units;
    const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(n));
    if (i8)
    {
      expand_kernel<CAIFQ_I8><<<grid, kBlock, 0, s>>>(t, out, units, 0);
    }
    else
    {
      expand_kernel<CAIFQ_I4><<<grid, kBlock, 0, s>>>(t, out, units, w0.group_size);
    }
    CAIFQ_CHECK_LAUNCH();
  }
  return CAIFQ_OK;
}

int launch_expand_to_bf16(const caifq_weight &w, void *dst, cudaStream_t s) { return launch_expand_grouped_to_bf16(&w, 1, dst, s); }

// ---- a weight as the bf16 matrix the reference's ConvertToComputeDtype would hold for bf16 compute ----
// (src/caif_device_frozen_linear.cpp:288-378): int8 per-tensor bf16(float(code) * scale), int4 as
// expand_int4x8, bf16 copied, fp32 / fp16 rounded to bf16.  Used where several layers' weights are laid one
// under the other into one operand (fused q/k/v), so the scale has to be inside the values.
__global__ void expand_int8_scaled_kernel(const uint2 *__restrict__ codes, const float *__restrict__ scale,
                                          uint4 *__restrict__ dst, int64_t units)
{
  const float sc = __ldg(scale);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < units; i += stride)
  {
    const uint2 v = __ldg(codes + i);
    const uint32_t w[2] = {v.x, v.y};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 2; ++k)
    {
#pragma unroll
      for (int h = 0; h < 2; ++h)
      {
        const float lo = __fmul_rn(static_cast<float>(static_cast<int8_t>((w[k] >> (16 * h)) & 0xFFu)), sc);
        const float hi = __fmul_rn(static_cast<float>(static_cast<int8_t>((w[k] >> (16 * h + 8)) & 0xFFu)), sc);
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[2 * k + h]) : "f"(hi), "f"(lo));
      }
    }
    dst[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

int launch_weight_to_bf16_scaled(const caifq_weight &w, void *dst, cudaStream_t s)
{
  const int64_t total = static_cast<int64_t>(w.in_dim) * w.out_dim;
  if (w.storage == CAIFQ_I4)
  {
    return launch_expand_to_bf16(w, dst, s);
  }
  if (w.storage == CAIFQ_I8)
  {
    if (w.scheme != CAIFQ_PER_TENSOR || w.scales == nullptr || (total % 8) != 0 ||
        (reinterpret_cast<uintptr_t>(w.codes) & 7u) != 0)
    {
      set_error("weight_to_bf16: int8 needs one per-tensor scale, 8-byte aligned codes and a multiple of 8 weights");
      return CAIFQ_ERR_UNSUPPORTED;
    }
    const int64_t units = total / 8;
    expand_int8_scaled_kernel<<<grid_for(units), kBlock, 0, s>>>(static_cast<const uint2 *>(w.codes),
                                                               static_cast<const float *>(w.scales),
                                                               static_cast<uint4 *>(dst), units);
    CAIFQ_CHECK_LAUNCH();
    return CAIFQ_OK;
  }
  if (w.storage == CAIFQ_BF16)
  {
    const cudaError_t err = cudaMemcpyAsync(dst, w.codes, static_cast<size_t>(total) * 2, cudaMemcpyDeviceToDevice, s);
    if (err != cudaSuccess)
    {
      set_error("weight_to_bf16: copy failed: %s", cudaGetErrorString(err));
      return CAIFQ_ERR_CUDA;
    }
    return CAIFQ_OK;
  }
  return launch_cast(w.codes, w.storage, dst, CAIFQ_BF16, total, s);
}

int launch_weight_materialize(const caifq_weight &w, void *dst, int dst_dtype, cudaStream_t s)
{
  const int64_t total = static_cast<int64_t>(w.in_dim) * w.out_dim;
  if (total <= 0)
  {
    return CAIFQ_OK;
  }
  const int g = grid_for(total);
  switch (w.storage)
  {
    case CAIFQ_F32:
      materialize_kernel<CAIFQ_F32><<<g, kBlock, 0, s>>>(w, dst, dst_dtype, total);
      break;
    case CAIFQ_F16:
      materialize_kernel<CAIFQ_F16><<<g, kBlock, 0, s>>>(w, dst, dst_dtype, total);
      break;
    case CAIFQ_BF16:
      materialize_kernel<CAIFQ_BF16><<<g, kBlock, 0, s>>>(w, dst, dst_dtype, total);
      break;
    case CAIFQ_I8:
      materialize_kernel<CAIFQ_I8><<<g, kBlock, 0, s>>>(w, dst, dst_dtype, total);
      break;
    case CAIFQ_I4:
      materialize_kernel<CAIFQ_I4><<<g, kBlock, 0, s>>>(w, dst, dst_dtype, total);
      break;
    default:
      set_error("weight_materialize: unsupported storage dtype %d", w.storage);
      return CAIFQ_ERR_INVALID;
  }
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

}  // namespace caifq
