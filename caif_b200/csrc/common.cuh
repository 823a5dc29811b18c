// Shared declarations of the caifq kernels: dtype codes, error plumbing,
// scalar conversions and the launcher prototypes that c_api.cu calls.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "caifq.h"

namespace caifq
{

void set_error(const char *fmt, ...);
void set_path(const char *name);

#define CAIFQ_CHECK_ARG(cond, ...)        \
  do                                      \
  {                                       \
    if (!(cond))                          \
    {                                     \
      ::caifq::set_error(__VA_ARGS__);    \
      return CAIFQ_ERR_INVALID;           \
    }                                     \
  } while (0)

#define CAIFQ_CHECK_CUDA(expr)                                                            \
  do                                                                                      \
  {                                                                                       \
    cudaError_t err__ = (expr);                                                           \
    if (err__ != cudaSuccess)                                                             \
    {                                                                                     \
      ::caifq::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(err__), __FILE__, __LINE__); \
      return CAIFQ_ERR_CUDA;                                                              \
    }                                                                                     \
  } while (0)

#define CAIFQ_CHECK_LAUNCH() CAIFQ_CHECK_CUDA(cudaGetLastError())

// SMs of the current device (cached per device ordinal) and the number of CTAs a persistent kernel
// may launch: one per SM unless the host has asked for fewer (caifq_set_cta_limit, or the
// CAIFQ_DECODE_CTAS / CAIFQ_UMMA_CTAS environment variables read at the first launch).
constexpr int kMaxDevices = 64;
int device_sm_count();
int persistent_ctas(const char *env_name);

inline bool is_float_dtype(int d) { return d == CAIFQ_F32 || d == CAIFQ_F16 || d == CAIFQ_BF16; }

inline size_t dtype_bytes(int d)
{
  switch (d)
  {
    case CAIFQ_F32:
      return 4;
    case CAIFQ_F16:
    case CAIFQ_BF16:
      return 2;
    case CAIFQ_I8:
      return 1;
    default:
      return 0;
  }
}

// ---- device-side scalar helpers -------------------------------------------

__device__ __forceinline__ float load_as_float(const void *p, int64_t i, int dtype)
{
  if (dtype == CAIFQ_F32)
  {
    return static_cast<const float *>(p)[i];
  }
  if (dtype == CAIFQ_BF16)
  {
    return __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
  }
  return __half2float(static_cast<const __half *>(p)[i]);
}

__device__ __forceinline__ void store_from_float(void *p, int64_t i, int dtype, float v)
{
  if (dtype == CAIFQ_F32)
  {
    static_cast<float *>(p)[i] = v;
  }
  else if (dtype == CAIFQ_BF16)
  {
    static_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16(v);
  }
  else
  {
    static_cast<__half *>(p)[i] = __float2half(v);
  }
}

// ---- eight quantized codes -> eight bf16 values (one 16-byte store), used by the expansion kernels
__device__ __forceinline__ uint4 expand_int8x8(const uint2 v)
{
  const uint32_t w[2] = {v.x, v.y};
  uint32_t o[4];
#pragma unroll
  for (int k = 0; k < 2; ++k)
  {
    const uint32_t a = __byte_perm(w[k], 0u, 0x4140);   // [b0, 0, b1, 0]
    const uint32_t b = __byte_perm(w[k], 0u, 0x4342);   // [b2, 0, b3, 0]
    // low 7 bits in the mantissa of 128.0; the sign bit selects 128.0 or 256.0 to subtract
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(o[2 * k]) : "r"((a & 0x007F007Fu) | 0x43004300u), "r"((a & 0x00800080u) | 0x43004300u));
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(o[2 * k + 1]) : "r"((b & 0x007F007Fu) | 0x43004300u), "r"((b & 0x00800080u) | 0x43004300u));
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

__device__ __forceinline__ uint4 expand_int4x8(const uint32_t w, const float scale)
{
  const float base = 8388616.0f;   // 2^23 + 8
  const uint32_t ev = (w & 0x0F0F0F0Fu) ^ 0x08080808u;          // elements 0, 2, 4, 6 of the word
  const uint32_t od = ((w >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;   // elements 1, 3, 5, 7
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
  {
    const float e = __fmul_rn(__uint_as_float(__byte_perm(ev, 0x4B000000u, 0x7440 + j)) - base, scale);
    const float d = __fmul_rn(__uint_as_float(__byte_perm(od, 0x4B000000u, 0x7440 + j)) - base, scale);
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[j]) : "f"(d), "f"(e));
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// Round an fp32 value through a 16-bit float dtype (nearest even) and back.
template <int DTYPE>
__device__ __forceinline__ float round_through(float v)
{
  if constexpr (DTYPE == CAIFQ_BF16)
  {
    return __bfloat162float(__float2bfloat16(v));
  }
  else if constexpr (DTYPE == CAIFQ_F16)
  {
    return __half2float(__float2half(v));
  }
  else
  {
    return v;
  }
}

__device__ __forceinline__ float round_through_rt(float v, int dtype)
{
  if (dtype == CAIFQ_BF16)
  {
    return __bfloat162float(__float2bfloat16(v));
  }
  if (dtype == CAIFQ_F16)
  {
    return __half2float(__float2half(v));
  }
  return v;
}

__device__ __forceinline__ int sign_extend_nibble(int v) { return (v ^ 8) - 8; }

// Element (flat index) of a frozen weight as the fp32 value the reference's
// dequantize kernels produce, before any rounding to a compute dtype.
template <int STORAGE>
__device__ __forceinline__ float weight_value(const caifq_weight &w, int64_t flat)
{
  if constexpr (STORAGE == CAIFQ_F32)
  {
    return static_cast<const float *>(w.codes)[flat];
  }
  else if constexpr (STORAGE == CAIFQ_F16)
  {
    return __half2float(static_cast<const __half *>(w.codes)[flat]);
  }
  else if constexpr (STORAGE == CAIFQ_BF16)
  {
    return __bfloat162float(static_cast<const __nv_bfloat16 *>(w.codes)[flat]);
  }
  else if constexpr (STORAGE == CAIFQ_I8)
  {
    const float q = static_cast<float>(static_cast<const int8_t *>(w.codes)[flat]);
    if (w.scales == nullptr)
    {
      return q;
    }
    const float *s = static_cast<const float *>(w.scales);
    if (w.scheme == CAIFQ_PER_TENSOR)
    {
      return __fmul_rn(q, s[0]);
    }
    return __fmul_rn(q, s[flat % w.out_dim]);
  }
  else
  {
    const uint8_t b = static_cast<const uint8_t *>(w.codes)[flat >> 1];
    const int nib = (flat & 1) ? (b >> 4) : (b & 0xF);
    const float q = static_cast<float>(sign_extend_nibble(nib));
    const float s = __half2float(static_cast<const __half *>(w.scales)[flat / w.group_size]);
    return __fmul_rn(q, s);
  }
}

// ---- launchers implemented in the individual .cu files ----------------------

int launch_quantize_int8_per_tensor(const float *x, int8_t *q, float *scale, int64_t n, cudaStream_t s);
int launch_quantize_int8_per_channel(const float *x, int8_t *q, float *scales, int rows, int cols, cudaStream_t s);
int launch_quantize_int4(const float *x, uint8_t *packed, uint16_t *scales, int64_t n, int group, cudaStream_t s);
int launch_dequantize_int8_per_tensor(const int8_t *q, float *out, const float *scale, int64_t n, cudaStream_t s);
int launch_dequantize_int8_per_channel(const int8_t *q, float *out, const float *scales, int rows, int cols,
                                       cudaStream_t s);
int launch_dequantize_int4(const uint8_t *packed, const uint16_t *scales, float *out, int64_t n, int group,
                           cudaStream_t s);
int launch_cast(const void *src, int src_dtype, void *dst, int dst_dtype, int64_t n, cudaStream_t s);
int launch_weight_materialize(const caifq_weight &w, void *dst, int dst_dtype, cudaStream_t s);
// int8 / int4 codes -> a bf16 [out, in] matrix for the tensor core: int8 codes as exact integers (the scale
// is left to the epilogue), int4 as bf16(scale * code), the reference's dequantize-then-cast value
int launch_expand_to_bf16(const caifq_weight &w, void *dst, cudaStream_t s);
// the weight as the bf16 matrix bf16 compute sees (scales inside the values): int4, int8 per-tensor, floats
int launch_weight_to_bf16_scaled(const caifq_weight &w, void *dst, cudaStream_t s);
// the same for `count` experts of one shape in one launch; expert e lands at dst + e * out * in elements
int launch_expand_grouped_to_bf16(const caifq_weight *ws, int count, void *dst, cudaStream_t s);

// One frozen-linear product.  forward: c[m,out] = a[m,in] . W^T;  backward:
// c[m,in] = a[m,out] . W.  `a_prescale` != 1 multiplies a on load and rounds the
// product to a_dtype (LoRA's alpha/r on dY).  `accumulate` makes the epilogue
// c = round_c( round_c(acc) + c_old ), the reference's cast-then-Add.
struct LinearArgs
{
  caifq_weight w;
  bool backward;
  const void *a;
  int a_dtype;
  float a_prescale;
  int64_t m;
  void *c;
  int c_dtype;
  bool accumulate;
  int compute_dtype;
  // Optional rank-padded LoRA product folded into the same accumulation as one extra
  // k-block (tensor-core path only): lora_lhs is [m, 64] bf16 (zero beyond the rank),
  // lora_rhs is [N, 64] bf16 for forward (rows follow the output features) or [64, N] bf16
  // for backward.  Both already carry every scale so that acc_total * epilogue scale is right.
  const void *lora_lhs;
  const void *lora_rhs;
  // bf16 weights on the tensor-core path only: a device scalar the fp32 accumulator is multiplied by in the
  // epilogue (the per-tensor scale of int8 codes that were expanded to exact bf16 integers); null = 1
  const float *c_scale;
  // Optional fused all-gather of a column-parallel forward (few-token kernel only): when
  // num_peers > 0 every output element goes to c_peers[r] for all r (this GPU's own buffer
  // included, `c` is ignored) at row pitch c_ld and column offset c_col0.
  void *const *c_peers;
  int num_peers;
  int64_t c_ld;
  int64_t c_col0;
  // Optional further layers that share the input (few-token kernel only): their rows follow w's in one
  // launch and their outputs follow w's in the columns of c ([m, out + sum of their out_dims]).
  const caifq_weight *more;
  int num_more;
};

constexpr int kMaxPeers = 8;

// generic tiled fp32-FMA GEMM over every (storage, compute) cell
int launch_linear_generic(const LinearArgs &args, cudaStream_t s);

// weight-streaming kernel for few tokens (forward only)
// The same product for a run of experts over one packed activation buffer:
// rows offsets[e] .. offsets[e+1] (host array of num_experts + 1 entries) belong to weights[e].
struct GroupedLinearArgs
{
  const caifq_weight *weights;
  int num_experts;
  const int32_t *offsets;
  bool backward;
  const void *a;
  int a_dtype;
  void *c;
  int c_dtype;
  bool accumulate;
  int compute_dtype;
  // Optional second operand pair (stacked bf16 experts only): c = a . W + a2 . W2 in one accumulation, rounded once
  const caifq_weight *weights2;
  const void *a2;
  // Optional SwiGLU backward in the epilogue of the dX launch that produces the hidden activation's gradient
  // (backward, bf16, no accumulate): c receives g_gate, sb_g_up receives g_up; sb_gate / sb_up are the forward's
  // gate(x) and up(x), all [total_rows, in_dim of the weights]
  const void *sb_gate;
  const void *sb_up;
  void *sb_g_up;
};
// gate(x), up(x) and silu(gate(x)) * up(x) of a run of frozen experts in one launch
// (CAIF_DeviceMoEFrozenExpert::ForwardImpl up to the down projection,
// src/caif_device_moe_frozen_expert.cpp:104-153).
struct GroupedSwigluArgs
{
  const caifq_weight *gate;
  const caifq_weight *up;
  int num_experts;
  const int32_t *offsets;
  const void *x;
  void *gate_out;
  void *up_out;
  void *hidden;
  int dtype;
  int compute_dtype;
};
bool umma_swiglu_supported(const GroupedSwigluArgs &args);
int launch_linear_umma_swiglu(const GroupedSwigluArgs &args, cudaStream_t s);
bool umma_grouped_supported(const GroupedLinearArgs &args);
int launch_linear_umma_grouped(const GroupedLinearArgs &args, cudaStream_t s);
// The few-token kernel reads codes and scales ahead of the previous kernel's completion (dependent
// launch).  The library's own quantize and cast kernels produce codes: the first few-token launch
// on the same device and stream after one of them is a plain launch, which orders it (and
// everything after it) behind that kernel.
void note_codes_written(cudaStream_t s);
bool take_codes_written(cudaStream_t s);
// self-test hook: the next few-token launch of this thread waits for bytes that never arrive
void decode_stall_next_launch();
int umma_pair_capacity();   // resident CTA pairs of the tensor-core kernel seen on the current device (0: none launched yet)
void umma_stall_next_launch();
bool decode_supported(const LinearArgs &args);
int launch_linear_decode(const LinearArgs &args, cudaStream_t s);

// tcgen05 / TMEM tensor-core kernel for many tokens
bool umma_supported(const LinearArgs &args);
int launch_linear_umma(const LinearArgs &args, cudaStream_t s);

}  // namespace caifq
