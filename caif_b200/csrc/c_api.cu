// The extern "C" surface declared in include/caifq.h: argument checks, kernel
// family selection, and the compositions (LoRA, grouped experts) that are
// several launches.  No entry point allocates device memory or synchronises.
#include <atomic>
#include <cstdarg>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace caifq
{

// each kernel file owns its flag and the code that reads it (device symbols are per translation unit)
int take_decode_timeout_flag();
int take_umma_timeout_flag();

namespace
{
thread_local char t_error[512] = "";
thread_local const char *t_path = "none";
}  // namespace

void set_error(const char *fmt, ...)
{
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
}

void set_path(const char *name) { t_path = name; }

namespace
{
std::atomic<int> g_cta_limit{0};   // 0 = no limit set through the API
}

int device_sm_count()
{
  static std::atomic<int> cached[kMaxDevices];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDevices)
  {
    dev = 0;
  }
  int v = cached[dev].load(std::memory_order_relaxed);
  if (v == 0)
  {
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    if (v <= 0)
    {
      v = 148;
    }
    cached[dev].store(v, std::memory_order_relaxed);
  }
  return v;
}

int persistent_ctas(const char *env_name)
{
  int n = device_sm_count();
  const int api = g_cta_limit.load(std::memory_order_relaxed);
  if (api >= 1 && api < n)
  {
    return api;
  }
  if (const char *e = std::getenv(env_name))
  {
    const int v = std::atoi(e);
    if (v >= 1 && v < n)
    {
      n = v;
    }
  }
  return n;
}

// moe.cu
int launch_moe_topk(const void *probs, int dtype, int *indices, void *values, int batch, int dim, int k,
                    cudaStream_t s);
int launch_moe_normalize_rows(const void *input, void *output, int dtype, int batch, int dim, cudaStream_t s);
int launch_moe_router_softmax(const void *logits, const void *bias, void *probs, int dtype, int rows, int cols,
                              cudaStream_t s);
int launch_moe_build_dispatch(const int *expert_indices, int num_tokens, int top_k, int num_experts, int capacity,
                              int *dispatch_map, int *expert_offsets, cudaStream_t s);
int launch_moe_dispatch(const void *input, int dtype, const int *expert_indices, const int *dispatch_map,
                        const int *expert_offsets, void *buffer, int num_tokens, int dim, int top_k, cudaStream_t s);
int launch_moe_combine_bwd_grad_expert(const void *grad_output, int dtype, const int *expert_indices,
                                       const void *expert_weights, const int *dispatch_map, const int *expert_offsets,
                                       void *grad_buffer, int num_tokens, int dim, int top_k, cudaStream_t s);
int launch_moe_combine_bwd_grad_weights(const void *grad_output, const void *buffer, int dtype,
                                        const int *expert_indices, const int *dispatch_map,
                                        const int *expert_offsets, void *grad_weights, int num_tokens, int dim,
                                        int top_k, cudaStream_t s);
int launch_moe_dispatch_bwd(const void *grad_buffer, int dtype, const int *expert_indices, const int *dispatch_map,
                            const int *expert_offsets, void *grad_input, int num_tokens, int dim, int top_k,
                            cudaStream_t s);
int launch_moe_combine(const void *buffer, int dtype, const int *expert_indices, const void *expert_weights,
                       const int *dispatch_map, const int *expert_offsets, void *output, int num_tokens, int dim,
                       int top_k, cudaStream_t s);
int launch_swiglu_fwd(const void *gate, const void *up, void *hidden, int dtype, int64_t n, cudaStream_t s);
int launch_swiglu_bwd(const void *g_hidden, const void *gate, const void *up, void *g_gate, void *g_up, int dtype,
                      int64_t n, cudaStream_t s);
int launch_add(const void *a, const void *b, void *out, int dtype, int64_t n, cudaStream_t s);
int launch_silu_fwd(const void *x, void *out, int dtype, int64_t n, cudaStream_t s);
int launch_silu_bwd(const void *x, const void *grad, void *out, int dtype, int64_t n, cudaStream_t s);
// lora.cu
size_t gemm_tn_scratch_bytes(int p, int q);
int launch_gemm_tn(const void *u, const void *v, void *c, float *scratch, int dtype, int compute_dtype,
                   float u_prescale, int64_t m, int p, int q, cudaStream_t s);
int launch_scale(const void *src, void *dst, int dtype, float scale, int64_t n, cudaStream_t s);
int launch_moe_bias_update(void *bias, const int *counts, int dtype, int experts, float rate, int from_offsets,
                           cudaStream_t s);
int launch_rmsnorm_fwd(const void *input, const float *gamma, void *output, float *rms_cache, float epsilon, int dtype,
                       int rows, int dim, cudaStream_t s);
int launch_rmsnorm_bwd(const void *grad_output, const void *input, const float *gamma, const float *rms_cache,
                       void *grad_input, float *grad_gamma, int dtype, int rows, int dim, cudaStream_t s);
int launch_moe_router_bwd(const void *grad_w, const void *probs, const int *indices, const void *balance_bias,
                          const void *z_lse_scaled, void *grad_topk, void *grad_logits, int dtype, int tokens,
                          int experts, int top_k, int sigmoid_gate, int normalize, float scaling, int exact_jacobian,
                          cudaStream_t s);
int launch_moe_aux_losses(const void *logits, const void *probs, const int *expert_offsets, void *balance_bias,
                          void *lse, void *z_lse_scaled, float *sums, int dtype, int tokens, int experts, int top_k,
                          float balance_weight, float z_weight, cudaStream_t s);
int launch_moe_route_grouped(const void *input, const void *bias, void *scores_out, int *indices, void *weights,
                             int dtype, int batch, int dim, int k, int n_group, int topk_group, int apply_sigmoid,
                             cudaStream_t s);
int launch_lora_adamw(void *a, void *b, const void *d_a, const void *d_b, float *m_a, float *v_a, float *m_b,
                      float *v_b, int64_t n_a, int64_t n_b, int dtype, float lr, float beta1, float beta2,
                      float epsilon, float weight_decay, float bias_correction1, float bias_correction2,
                      cudaStream_t s);
bool skinny_supported(int dtype, int rank, int k);
int launch_skinny_nt(const void *x, const void *a, void *h, void *hs, float x_prescale, float hs_mul,
                     const float *hs_div, int64_t m, int k, int rank, cudaStream_t s);
int launch_skinny_tn(const void *u, const void *v, void *c, float *scratch, float u_prescale, int64_t m, int big,
                     int rank, bool transpose_out, cudaStream_t s);
int launch_lora_pad_b(const void *b, void *bp, int n, int rank, cudaStream_t s);
int launch_lora_transpose_b(const void *b, void *bt, int n, int rank, cudaStream_t s);
int launch_lora_pad_a(const void *a, void *ap, int n, int rank, cudaStream_t s);
int launch_expand_prepare(const caifq_weight &w, void *wb, const void *a, const void *b, void *bp, void *bt, void *ap,
                          int rank, cudaStream_t s);

namespace
{

int check_weight(const caifq_weight *w, const char *who)
{
  CAIFQ_CHECK_ARG(w != nullptr, "%s: weight is null", who);
  CAIFQ_CHECK_ARG(w->codes != nullptr, "%s: weight not loaded", who);
  CAIFQ_CHECK_ARG(w->in_dim > 0 && w->out_dim > 0, "%s: bad dims in=%d out=%d", who, w->in_dim, w->out_dim);
  switch (w->storage)
  {
    case CAIFQ_F32:
    case CAIFQ_F16:
    case CAIFQ_BF16:
      break;
    case CAIFQ_I8:
      CAIFQ_CHECK_ARG(w->scheme == CAIFQ_PER_TENSOR || w->scheme == CAIFQ_PER_CHANNEL, "%s: bad int8 scheme %d", who,
                      w->scheme);
      break;
    case CAIFQ_I4:
      CAIFQ_CHECK_ARG(w->scales != nullptr, "%s: int4 weight needs scales", who);
      CAIFQ_CHECK_ARG(w->group_size > 0, "%s: bad group size %d", who, w->group_size);
      break;
    default:
      set_error("%s: unsupported storage dtype %d", who, w->storage);
      return CAIFQ_ERR_INVALID;
  }
  return CAIFQ_OK;
}

enum class Force
{
  None,
  Generic,
  Umma,
  Decode
};

Force forced_path()
{
  const char *e = std::getenv("CAIFQ_FORCE_PATH");
  if (e == nullptr || e[0] == '\0')
  {
    return Force::None;
  }
  if (std::strcmp(e, "generic") == 0)
  {
    return Force::Generic;
  }
  if (std::strcmp(e, "umma") == 0)
  {
    return Force::Umma;
  }
  if (std::strcmp(e, "decode") == 0)
  {
    return Force::Decode;
  }
  return Force::None;
}

int linear_any(const caifq_weight *w, bool backward, const void *a, int a_dtype, float a_prescale, int64_t m,
               void *c, int c_dtype, bool accumulate, int compute_dtype, cudaStream_t s, const char *who,
               const void *lora_lhs = nullptr, const void *lora_rhs = nullptr, const float *c_scale = nullptr)
{
  const int rc = check_weight(w, who);
  if (rc != CAIFQ_OK)
  {
    return rc;
  }
  CAIFQ_CHECK_ARG(m >= 0, "%s: negative m", who);
  CAIFQ_CHECK_ARG(is_float_dtype(a_dtype) && is_float_dtype(c_dtype) && is_float_dtype(compute_dtype),
                  "%s: activation/output/compute dtypes must be F32, F16 or BF16", who);
  if (m == 0)
  {
    return CAIFQ_OK;
  }
  CAIFQ_CHECK_ARG(a != nullptr && c != nullptr, "%s: null activation or output pointer", who);
  LinearArgs args{};
  args.w = *w;
  args.backward = backward;
  args.a = a;
  args.a_dtype = a_dtype;
  args.a_prescale = a_prescale;
  args.m = m;
  args.c = c;
  args.c_dtype = c_dtype;
  args.accumulate = accumulate;
  args.compute_dtype = compute_dtype;
  args.lora_lhs = lora_lhs;
  args.lora_rhs = lora_rhs;
  args.c_scale = c_scale;
  if (lora_lhs != nullptr)
  {
    // the fused LoRA k-block exists on the tensor-core path only; callers check fused_lora_ok() first
    if (!umma_supported(args))
    {
      set_error("%s: fused LoRA needs the tensor-core path", who);
      return CAIFQ_ERR_UNSUPPORTED;
    }
    set_path("umma");
    return launch_linear_umma(args, s);
  }
  const Force force = forced_path();
  if ((force == Force::None || force == Force::Decode) && decode_supported(args))
  {
    set_path("decode");
    return launch_linear_decode(args, s);
  }
  if ((force == Force::None || force == Force::Umma) && umma_supported(args))
  {
    set_path("umma");
    return launch_linear_umma(args, s);
  }
  if (force == Force::Umma || force == Force::Decode)
  {
    set_error("%s: forced kernel family does not support this call", who);
    return CAIFQ_ERR_UNSUPPORTED;
  }
  set_path("generic");
  return launch_linear_generic(args, s);
}

caifq_weight float_weight(const void *data, int dtype, int out_dim, int in_dim)
{
  caifq_weight w{};
  w.codes = data;
  w.scales = nullptr;
  w.storage = dtype;
  w.scheme = CAIFQ_PER_TENSOR;
  w.group_size = 128;
  w.in_dim = in_dim;
  w.out_dim = out_dim;
  return w;
}

inline size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

// The fast LoRA path: bf16 adapter of rank 8/16/32/64 on a quantized base that the tensor-core
// kernel takes (forward and backward), enough tokens, and no forced kernel family.
bool fused_lora_ok(const caifq_weight *w, const caifq_lora *l, const void *act, int64_t m, int compute_dtype)
{
  if (forced_path() != Force::None || l->dtype != CAIFQ_BF16 || m < 32)
  {
    return false;
  }
  if (w->storage != CAIFQ_I8 && w->storage != CAIFQ_I4)
  {
    return false;
  }
  if (!skinny_supported(l->dtype, l->rank, w->in_dim) || !skinny_supported(l->dtype, l->rank, w->out_dim))
  {
    return false;
  }
  LinearArgs probe{};
  probe.w = *w;
  probe.a = act;
  probe.a_dtype = CAIFQ_BF16;
  probe.a_prescale = 1.0f;
  probe.m = m;
  probe.c = const_cast<void *>(act);  // only alignment is looked at
  probe.c_dtype = CAIFQ_BF16;
  probe.compute_dtype = compute_dtype;
  probe.backward = false;
  if (!umma_supported(probe))
  {
    return false;
  }
  probe.backward = true;
  return umma_supported(probe);
}

// Many-token calls may expand the weight once per call into a bf16 matrix in the caller's workspace and feed
// it to the tensor core with plain tile copies on CTA pairs (1.43-1.55 PFLOP/s per launch at 4096 x 4096,
// 8192 tokens) instead of converting every tile again in the dequant warps of every CTA (1.1-1.3): the
// conversion is then done once per weight, not once per weight and 256 rows of tokens.  Worth its 10-15 us
// from a few thousand tokens on.  int4 needs bf16 compute (fp32 compute keeps the two-term form).
bool expand_ok(const caifq_weight *w, const caifq_lora *l, const void *act, int64_t m, int compute_dtype)
{
  if (m < 4096 || !fused_lora_ok(w, l, act, m, compute_dtype))
  {
    return false;
  }
  if (w->storage == CAIFQ_I4 && compute_dtype != CAIFQ_BF16)
  {
    return false;
  }
  return (w->in_dim % 256) == 0 && (w->out_dim % 256) == 0;
}

size_t expanded_weight_bytes(const caifq_weight *w)
{
  return align256(static_cast<size_t>(w->in_dim) * static_cast<size_t>(w->out_dim) * 2);
}

// scale the base kernel applies in its epilogue (what the padded LoRA operand must be divided by)
const float *epilogue_scale_ptr(const caifq_weight *w)
{
  return (w->storage == CAIFQ_I8 && w->scales != nullptr) ? static_cast<const float *>(w->scales) : nullptr;
}

struct LoraFwdWs
{
  size_t hs;      // [m, 64] bf16
  size_t bp;      // [out, 64] bf16
  size_t total;
};

LoraFwdWs lora_fwd_ws(const caifq_weight *w, int64_t m)
{
  LoraFwdWs l{};
  l.hs = 0;
  l.bp = align256(static_cast<size_t>(m) * 64 * 2);
  l.total = l.bp + align256(static_cast<size_t>(w->out_dim) * 64 * 2);
  return l;
}

struct LoraBwdWs
{
  size_t d_hidden;  // [m, r] in <= 4-byte elements
  size_t scratch;   // fp32 [max(in,out), r]
  size_t bt;        // [r, out] bf16
  size_t dhs;       // [m, 64] bf16
  size_t ap;        // [64, in] bf16
  size_t total;
};

LoraBwdWs lora_bwd_ws(const caifq_weight *w, const caifq_lora *l, int64_t m)
{
  LoraBwdWs o{};
  const size_t big = static_cast<size_t>(w->in_dim > w->out_dim ? w->in_dim : w->out_dim);
  o.d_hidden = 0;
  o.scratch = align256(static_cast<size_t>(m) * static_cast<size_t>(l->rank) * 4);
  o.bt = o.scratch + align256(big * static_cast<size_t>(l->rank) * sizeof(float));
  o.dhs = o.bt + align256(static_cast<size_t>(l->rank) * w->out_dim * 2);
  o.ap = o.dhs + align256(static_cast<size_t>(m) * 64 * 2);
  o.total = o.ap + align256(static_cast<size_t>(64) * w->in_dim * 2);
  return o;
}

}  // namespace
}  // namespace caifq

using namespace caifq;

extern "C" {

const char *caifq_last_error(void) { return t_error; }

const char *caifq_last_path(void) { return t_path; }

const char *caifq_version(void) { return "caifq 0.1 (sm_100a)"; }

int caifq_device_status(void)
{
  // bit 0: the decode kernel gave up on a wait; bit 1: the tensor-core kernel did
  if (cudaDeviceSynchronize() != cudaSuccess)
  {
    set_error("caifq_device_status: %s", cudaGetErrorString(cudaGetLastError()));
    return -1;
  }
  const int decode_flag = take_decode_timeout_flag();
  const int umma_flag = take_umma_timeout_flag();
  if (decode_flag < 0 || umma_flag < 0)
  {
    set_error("caifq_device_status: %s", cudaGetErrorString(cudaGetLastError()));
    return -1;
  }
  return (decode_flag ? 1 : 0) | (umma_flag ? 2 : 0);
}

void caifq_selftest_stall_next_decode(void) { decode_stall_next_launch(); }

void caifq_selftest_stall_next_umma(void) { umma_stall_next_launch(); }

int32_t caifq_umma_pair_capacity(void) { return umma_pair_capacity(); }

void caifq_set_cta_limit(int32_t max_ctas) { g_cta_limit.store(max_ctas > 0 ? max_ctas : 0, std::memory_order_relaxed); }

int caifq_device_ok(void)
{
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess)
  {
    cudaGetLastError();
    return 0;
  }
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
  {
    cudaGetLastError();
    return 0;
  }
  return major == 10 ? 1 : 0;
}

int caifq_quantize_int8_per_tensor(const float *x, int8_t *q, float *scale, int64_t n, void *stream)
{
  note_codes_written(static_cast<cudaStream_t>(stream));
  CAIFQ_CHECK_ARG(n >= 0, "quantize_int8_per_tensor: negative n");
  CAIFQ_CHECK_ARG(n == 0 || (x && q && scale), "quantize_int8_per_tensor: null pointer");
  return launch_quantize_int8_per_tensor(x, q, scale, n, static_cast<cudaStream_t>(stream));
}

int caifq_quantize_int8_per_channel(const float *x, int8_t *q, float *scales, int32_t rows, int32_t cols, void *stream)
{
  note_codes_written(static_cast<cudaStream_t>(stream));
  CAIFQ_CHECK_ARG(rows >= 0 && cols >= 0, "quantize_int8_per_channel: negative shape");
  CAIFQ_CHECK_ARG(rows == 0 || cols == 0 || (x && q && scales), "quantize_int8_per_channel: null pointer");
  return launch_quantize_int8_per_channel(x, q, scales, rows, cols, static_cast<cudaStream_t>(stream));
}

int caifq_quantize_int4_per_group(const float *x, uint8_t *packed, uint16_t *scales_f16, int64_t n, int32_t group_size,
                                  void *stream)
{
  note_codes_written(static_cast<cudaStream_t>(stream));
  CAIFQ_CHECK_ARG(n >= 0, "quantize_int4_per_group: negative n");
  CAIFQ_CHECK_ARG(group_size > 0, "quantize_int4_per_group: group_size must be positive");
  CAIFQ_CHECK_ARG(n == 0 || (x && packed && scales_f16), "quantize_int4_per_group: null pointer");
  return launch_quantize_int4(x, packed, scales_f16, n, group_size, static_cast<cudaStream_t>(stream));
}

int caifq_dequantize_int8_per_tensor(const int8_t *q, float *out, const float *scale, int64_t n, void *stream)
{
  CAIFQ_CHECK_ARG(n >= 0, "dequantize_int8_per_tensor: negative n");
  CAIFQ_CHECK_ARG(n == 0 || (q && out && scale), "dequantize_int8_per_tensor: null pointer");
  return launch_dequantize_int8_per_tensor(q, out, scale, n, static_cast<cudaStream_t>(stream));
}

int caifq_dequantize_int8_per_channel(const int8_t *q, float *out, const float *scales, int32_t rows, int32_t cols,
                                      void *stream)
{
  CAIFQ_CHECK_ARG(rows >= 0 && cols >= 0, "dequantize_int8_per_channel: negative shape");
  CAIFQ_CHECK_ARG(rows == 0 || cols == 0 || (q && out && scales), "dequantize_int8_per_channel: null pointer");
  return launch_dequantize_int8_per_channel(q, out, scales, rows, cols, static_cast<cudaStream_t>(stream));
}

int caifq_dequantize_int4(const uint8_t *packed, const uint16_t *scales_f16, float *out, int64_t n, int32_t group_size,
                          void *stream)
{
  CAIFQ_CHECK_ARG(n >= 0, "dequantize_int4: negative n");
  CAIFQ_CHECK_ARG(group_size > 0, "dequantize_int4: group_size must be positive");
  CAIFQ_CHECK_ARG(n == 0 || (packed && scales_f16 && out), "dequantize_int4: null pointer");
  return launch_dequantize_int4(packed, scales_f16, out, n, group_size, static_cast<cudaStream_t>(stream));
}

int caifq_cast(const void *src, int32_t src_dtype, void *dst, int32_t dst_dtype, int64_t n, void *stream)
{
  CAIFQ_CHECK_ARG(n >= 0, "cast: negative n");
  CAIFQ_CHECK_ARG(n == 0 || (src && dst), "cast: null pointer");
  if (dst_dtype == CAIFQ_I8)
  {
    note_codes_written(static_cast<cudaStream_t>(stream));  // int8 codes without scales are a valid weight
  }
  return launch_cast(src, src_dtype, dst, dst_dtype, n, static_cast<cudaStream_t>(stream));
}

int caifq_weight_materialize(const caifq_weight *w, void *dst, int32_t dst_dtype, void *stream)
{
  const int rc = check_weight(w, "caifq_weight_materialize");
  if (rc != CAIFQ_OK)
  {
    return rc;
  }
  CAIFQ_CHECK_ARG(dst != nullptr && is_float_dtype(dst_dtype), "caifq_weight_materialize: bad destination");
  return launch_weight_materialize(*w, dst, dst_dtype, static_cast<cudaStream_t>(stream));
}

int caifq_linear_fwd(const caifq_weight *w, const void *x, int32_t x_dtype, int64_t m, void *y, int32_t y_dtype,
                     int32_t compute_dtype, void *stream)
{
  return linear_any(w, false, x, x_dtype, 1.0f, m, y, y_dtype, false, compute_dtype,
                    static_cast<cudaStream_t>(stream), "caifq_linear_fwd");
}

int caifq_linear_fwd_residual(const caifq_weight *w, const void *x, int32_t x_dtype, int64_t m, void *y_inout,
                              int32_t y_dtype, int32_t compute_dtype, void *stream)
{
  return linear_any(w, false, x, x_dtype, 1.0f, m, y_inout, y_dtype, true, compute_dtype,
                    static_cast<cudaStream_t>(stream), "caifq_linear_fwd_residual");
}

int caifq_linear_fwd_gather(const caifq_weight *w, const void *x, int32_t x_dtype, int64_t m, void *const *y_peers,
                            int32_t num_peers, int64_t y_ld, int64_t y_col0, int32_t y_dtype, int32_t compute_dtype,
                            void *stream)
{
  const char *who = "caifq_linear_fwd_gather";
  const int rc = check_weight(w, who);
  if (rc != CAIFQ_OK)
  {
    return rc;
  }
  CAIFQ_CHECK_ARG(m >= 0, "%s: negative m", who);
  CAIFQ_CHECK_ARG(is_float_dtype(x_dtype) && is_float_dtype(y_dtype) && is_float_dtype(compute_dtype),
                  "%s: activation/output/compute dtypes must be F32, F16 or BF16", who);
  CAIFQ_CHECK_ARG(y_peers != nullptr && num_peers >= 1 && num_peers <= kMaxPeers, "%s: 1 to %d result buffers", who,
                  kMaxPeers);
  CAIFQ_CHECK_ARG(y_col0 >= 0 && y_ld >= y_col0 + w->out_dim, "%s: the slice does not fit the row pitch", who);
  if (m == 0)
  {
    return CAIFQ_OK;
  }
  CAIFQ_CHECK_ARG(x != nullptr, "%s: null activation pointer", who);
  LinearArgs args{};
  args.w = *w;
  args.backward = false;
  args.a = x;
  args.a_dtype = x_dtype;
  args.a_prescale = 1.0f;
  args.m = m;
  args.c = y_peers[0];
  args.c_dtype = y_dtype;
  args.accumulate = false;
  args.compute_dtype = compute_dtype;
  args.c_peers = y_peers;
  args.num_peers = num_peers;
  args.c_ld = y_ld;
  args.c_col0 = y_col0;
  if (!decode_supported(args))
  {
    set_error("%s: only few-token calls the decode kernel takes (m <= 16, bf16 x, int4 or per-tensor int8)", who);
    return CAIFQ_ERR_UNSUPPORTED;
  }
  set_path("decode");
  return launch_linear_decode(args, static_cast<cudaStream_t>(stream));
}

int caifq_linear_fwd_multi(const caifq_weight *ws, int32_t num_weights, const void *x, int32_t x_dtype, int64_t m,
                           void *y, int32_t y_dtype, int32_t compute_dtype, void *stream)
{
  const char *who = "caifq_linear_fwd_multi";
  CAIFQ_CHECK_ARG(ws != nullptr && num_weights >= 1 && num_weights <= 4, "%s: 1 to 4 weights", who);
  for (int i = 0; i < num_weights; ++i)
  {
    const int rc = check_weight(&ws[i], who);
    if (rc != CAIFQ_OK)
    {
      return rc;
    }
  }
  CAIFQ_CHECK_ARG(m >= 0, "%s: negative m", who);
  CAIFQ_CHECK_ARG(is_float_dtype(x_dtype) && is_float_dtype(y_dtype) && is_float_dtype(compute_dtype),
                  "%s: activation/output/compute dtypes must be F32, F16 or BF16", who);
  if (m == 0)
  {
    return CAIFQ_OK;
  }
  CAIFQ_CHECK_ARG(x != nullptr && y != nullptr, "%s: null activation or output pointer", who);
  LinearArgs args{};
  args.w = ws[0];
  args.backward = false;
  args.a = x;
  args.a_dtype = x_dtype;
  args.a_prescale = 1.0f;
  args.m = m;
  args.c = y;
  args.c_dtype = y_dtype;
  args.accumulate = false;
  args.compute_dtype = compute_dtype;
  args.more = ws + 1;
  args.num_more = num_weights - 1;
  if (!decode_supported(args))
  {
    set_error("%s: only few-token calls the decode kernel takes (m <= 16, bf16 x, int4 or per-tensor int8, weights of "
              "one storage, row length and scale rule, each but the last with a multiple of 8 rows)", who);
    return CAIFQ_ERR_UNSUPPORTED;
  }
  set_path("decode");
  return launch_linear_decode(args, static_cast<cudaStream_t>(stream));
}

int caifq_linear_dx(const caifq_weight *w, const void *dy, int32_t dy_dtype, int64_t m, void *dx, int32_t dx_dtype,
                    int32_t compute_dtype, void *stream)
{
  return linear_any(w, true, dy, dy_dtype, 1.0f, m, dx, dx_dtype, false, compute_dtype,
                    static_cast<cudaStream_t>(stream), "caifq_linear_dx");
}

// ---------------------------------------------------------------------- LoRA

static int check_lora(const caifq_weight *w, const caifq_lora *l, const char *who)
{
  const int rc = check_weight(w, who);
  if (rc != CAIFQ_OK)
  {
    return rc;
  }
  CAIFQ_CHECK_ARG(l != nullptr && l->a != nullptr && l->b != nullptr, "%s: LoRA factors are null", who);
  CAIFQ_CHECK_ARG(l->rank > 0, "%s: LoRA rank must be positive", who);
  CAIFQ_CHECK_ARG(is_float_dtype(l->dtype), "%s: LoRA dtype must be F32, F16 or BF16", who);
  return CAIFQ_OK;
}

size_t caifq_lora_fwd_workspace_bytes(const caifq_weight *w, const caifq_lora *lora, int64_t m)
{
  if (w == nullptr || lora == nullptr || m <= 0)
  {
    return 0;
  }
  return lora_fwd_ws(w, m).total;
}

}  // extern "C"

namespace
{
const void *const kAlignedProbe = reinterpret_cast<const void *>(static_cast<uintptr_t>(256));

int lora_fwd_impl(const caifq_weight *w, const caifq_lora *lora, const void *x, int64_t m, void *y, void *hidden,
                  void *workspace, int32_t compute_dtype, void *stream, bool may_expand, const char *who)
{
  const int rc = check_lora(w, lora, who);
  if (rc != CAIFQ_OK)
  {
    return rc;
  }
  CAIFQ_CHECK_ARG(m >= 0, "%s: negative m", who);
  if (m == 0)
  {
    return CAIFQ_OK;
  }
  CAIFQ_CHECK_ARG(x && y && hidden, "%s: x, y and hidden must be non-null", who);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int sd = lora->dtype;
  const float scale = lora->alpha / static_cast<float>(lora->rank);
  if (workspace != nullptr && fused_lora_ok(w, lora, x, m, compute_dtype) &&
      (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0)
  {
    // hidden = x . A^T (bf16), Hs = hidden * (alpha/r) / epilogue scale, padded to 64 columns;
    // then one tensor-core launch computes x . W^T and Hs . Bp^T into the same accumulators.
    const LoraFwdWs ws = lora_fwd_ws(w, m);
    char *base = static_cast<char *>(workspace);
    const bool expand = may_expand && expand_ok(w, lora, x, m, compute_dtype);
    void *wb = base + ws.total;   // (expanded calls) the weight as a bf16 matrix behind the other scratch
    // the padded B factor, and with it the expansion of the weight where the call expands: one launch
    int r = expand ? launch_expand_prepare(*w, wb, lora->a, lora->b, base + ws.bp, nullptr, nullptr, lora->rank, s)
                   : launch_lora_pad_b(lora->b, base + ws.bp, w->out_dim, lora->rank, s);
    if (r == CAIFQ_OK)
    {
      r = launch_skinny_nt(x, lora->a, hidden, base + ws.hs, 1.0f, scale, epilogue_scale_ptr(w), m, w->in_dim,
                           lora->rank, s);
    }
    if (r != CAIFQ_OK)
    {
      return r;
    }
    if (expand)
    {
      const caifq_weight wbf = float_weight(wb, CAIFQ_BF16, w->out_dim, w->in_dim);
      return linear_any(&wbf, false, x, sd, 1.0f, m, y, sd, false, compute_dtype, s, who, base + ws.hs, base + ws.bp,
                        epilogue_scale_ptr(w));
    }
    return linear_any(w, false, x, sd, 1.0f, m, y, sd, false, compute_dtype, s, who, base + ws.hs, base + ws.bp);
  }
  // hidden = x . A^T, rounded to the storage dtype as the reference materialises it
  const caifq_weight wa = float_weight(lora->a, sd, lora->rank, w->in_dim);
  int r = linear_any(&wa, false, x, sd, 1.0f, m, hidden, sd, false, compute_dtype, s, who);
  if (r != CAIFQ_OK)
  {
    return r;
  }
  // y = hidden . B^T, then y *= alpha/r (two roundings in the reference)
  const caifq_weight wb = float_weight(lora->b, sd, w->out_dim, lora->rank);
  r = linear_any(&wb, false, hidden, sd, 1.0f, m, y, sd, false, compute_dtype, s, who);
  if (r != CAIFQ_OK)
  {
    return r;
  }
  r = launch_scale(y, y, sd, scale, m * static_cast<int64_t>(w->out_dim), s);
  if (r != CAIFQ_OK)
  {
    return r;
  }
  // frozen base on top: y = round(round(x . W^T) + y)
  return linear_any(w, false, x, sd, 1.0f, m, y, sd, true, compute_dtype, s, who);
}
}  // namespace

extern "C" {

int caifq_lora_linear_fwd(const caifq_weight *w, const caifq_lora *lora, const void *x, int64_t m, void *y,
                          void *hidden, void *workspace, int32_t compute_dtype, void *stream)
{
  return lora_fwd_impl(w, lora, x, m, y, hidden, workspace, compute_dtype, stream, false, "caifq_lora_linear_fwd");
}

size_t caifq_lora_fwd_workspace_bytes_expanded(const caifq_weight *w, const caifq_lora *lora, int64_t m,
                                               int32_t compute_dtype)
{
  if (w == nullptr || lora == nullptr || m <= 0)
  {
    return 0;
  }
  const size_t plain = lora_fwd_ws(w, m).total;
  return expand_ok(w, lora, kAlignedProbe, m, compute_dtype) ? plain + expanded_weight_bytes(w) : plain;
}

int caifq_lora_linear_fwd_expanded(const caifq_weight *w, const caifq_lora *lora, const void *x, int64_t m, void *y,
                                   void *hidden, void *workspace, int32_t compute_dtype, void *stream)
{
  return lora_fwd_impl(w, lora, x, m, y, hidden, workspace, compute_dtype, stream, true,
                       "caifq_lora_linear_fwd_expanded");
}

size_t caifq_lora_bwd_workspace_bytes(const caifq_weight *w, const caifq_lora *lora, int64_t m)
{
  if (w == nullptr || lora == nullptr || m <= 0 || lora->rank <= 0)
  {
    return 0;
  }
  return lora_bwd_ws(w, lora, m).total;
}

}  // extern "C"

namespace
{
int lora_bwd_impl(const caifq_weight *w, const caifq_lora *lora, const void *dy, const void *x, const void *hidden,
                  int64_t m, void *dx, void *d_a, void *d_b, void *workspace, int32_t compute_dtype, void *stream,
                  bool may_expand, const char *who)
{
  const int rc = check_lora(w, lora, who);
  if (rc != CAIFQ_OK)
  {
    return rc;
  }
  CAIFQ_CHECK_ARG(m >= 0, "%s: negative m", who);
  if (m == 0)
  {
    return CAIFQ_OK;
  }
  CAIFQ_CHECK_ARG(dy && x && hidden && dx && d_a && d_b && workspace, "%s: null pointer", who);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int sd = lora->dtype;
  const float scale = lora->alpha / static_cast<float>(lora->rank);
  const LoraBwdWs ws = lora_bwd_ws(w, lora, m);
  char *wbase = static_cast<char *>(workspace);
  void *d_hidden = wbase + ws.d_hidden;
  float *scratch = reinterpret_cast<float *>(wbase + ws.scratch);
  if (fused_lora_ok(w, lora, dy, m, compute_dtype) && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0)
  {
    // dH = (scale . dy) . B through the transposed copy of B; dHs = dH / epilogue scale, padded
    const bool expand = may_expand && expand_ok(w, lora, dy, m, compute_dtype);
    void *wb = wbase + ws.total;
    int r = CAIFQ_OK;
    if (expand)
    {
      // transposed B, padded A and the expansion of the weight in one launch
      r = launch_expand_prepare(*w, wb, lora->a, lora->b, nullptr, wbase + ws.bt, wbase + ws.ap, lora->rank, s);
    }
    else
    {
      r = launch_lora_transpose_b(lora->b, wbase + ws.bt, w->out_dim, lora->rank, s);
      if (r == CAIFQ_OK)
      {
        r = launch_lora_pad_a(lora->a, wbase + ws.ap, w->in_dim, lora->rank, s);
      }
    }
    if (r == CAIFQ_OK)
    {
      r = launch_skinny_nt(dy, wbase + ws.bt, d_hidden, wbase + ws.dhs, scale, 1.0f, epilogue_scale_ptr(w), m,
                           w->out_dim, lora->rank, s);
    }
    // dB[out, r] = (scale . dy)^T . hidden;  dA[r, in] = dH^T . x
    if (r == CAIFQ_OK)
    {
      r = launch_skinny_tn(dy, hidden, d_b, scratch, scale, m, w->out_dim, lora->rank, false, s);
    }
    if (r == CAIFQ_OK)
    {
      r = launch_skinny_tn(x, d_hidden, d_a, scratch, 1.0f, m, w->in_dim, lora->rank, true, s);
    }
    if (r != CAIFQ_OK)
    {
      return r;
    }
    // dx = dy . W + dHs . Ap in one tensor-core launch
    if (expand)
    {
      const caifq_weight wbf = float_weight(wb, CAIFQ_BF16, w->out_dim, w->in_dim);
      return linear_any(&wbf, true, dy, sd, 1.0f, m, dx, sd, false, compute_dtype, s, who, wbase + ws.dhs,
                        wbase + ws.ap, epilogue_scale_ptr(w));
    }
    return linear_any(w, true, dy, sd, 1.0f, m, dx, sd, false, compute_dtype, s, who, wbase + ws.dhs, wbase + ws.ap);
  }
  // dB[out, r] = (scale . dy)^T . hidden
  int r = launch_gemm_tn(dy, hidden, d_b, scratch, sd, compute_dtype, scale, m, w->out_dim, lora->rank, s);
  if (r != CAIFQ_OK)
  {
    return r;
  }
  // dH[m, r] = (scale . dy) . B
  const caifq_weight wb = float_weight(lora->b, sd, w->out_dim, lora->rank);
  r = linear_any(&wb, true, dy, sd, scale, m, d_hidden, sd, false, compute_dtype, s, who);
  if (r != CAIFQ_OK)
  {
    return r;
  }
  // dA[r, in] = dH^T . x
  r = launch_gemm_tn(d_hidden, x, d_a, scratch, sd, compute_dtype, 1.0f, m, lora->rank, w->in_dim, s);
  if (r != CAIFQ_OK)
  {
    return r;
  }
  // dx = dH . A, then the frozen base on top: dx = round(round(dy . W) + dx)
  const caifq_weight wa = float_weight(lora->a, sd, lora->rank, w->in_dim);
  r = linear_any(&wa, true, d_hidden, sd, 1.0f, m, dx, sd, false, compute_dtype, s, who);
  if (r != CAIFQ_OK)
  {
    return r;
  }
  return linear_any(w, true, dy, sd, 1.0f, m, dx, sd, true, compute_dtype, s, who);
}
}  // namespace

extern "C" {

int caifq_lora_linear_bwd(const caifq_weight *w, const caifq_lora *lora, const void *dy, const void *x,
                          const void *hidden, int64_t m, void *dx, void *d_a, void *d_b, void *workspace,
                          int32_t compute_dtype, void *stream)
{
  return lora_bwd_impl(w, lora, dy, x, hidden, m, dx, d_a, d_b, workspace, compute_dtype, stream, false,
                       "caifq_lora_linear_bwd");
}

size_t caifq_lora_bwd_workspace_bytes_expanded(const caifq_weight *w, const caifq_lora *lora, int64_t m,
                                               int32_t compute_dtype)
{
  if (w == nullptr || lora == nullptr || m <= 0 || lora->rank <= 0)
  {
    return 0;
  }
  const size_t plain = lora_bwd_ws(w, lora, m).total;
  return expand_ok(w, lora, kAlignedProbe, m, compute_dtype) ? plain + expanded_weight_bytes(w) : plain;
}

int caifq_lora_linear_bwd_expanded(const caifq_weight *w, const caifq_lora *lora, const void *dy, const void *x,
                                   const void *hidden, int64_t m, void *dx, void *d_a, void *d_b, void *workspace,
                                   int32_t compute_dtype, void *stream)
{
  return lora_bwd_impl(w, lora, dy, x, hidden, m, dx, d_a, d_b, workspace, compute_dtype, stream, true,
                       "caifq_lora_linear_bwd_expanded");
}

// ------------------------------------------------- LoRA backward, no allocation
//
// Scratch for caifq_lora_linear_bwd_noalloc.  It lives in the library image, so
// every GPU that loads libcaifq.so carries these 8 MiB until the process exits.
// The name below is a host-side stand-in for the array, NOT a device address:
// the device address is fetched once per device with cudaGetSymbolAddress.
#define CAIFQ_NOALLOC_SCRATCH_BYTES (8u << 20)
static __device__ __align__(256) unsigned char g_noalloc_scratch[CAIFQ_NOALLOC_SCRATCH_BYTES];

namespace
{
void *g_noalloc_ptr[kMaxDevices] = {};
std::mutex g_noalloc_mutex;
}  // namespace

size_t caifq_lora_bwd_noalloc_max_bytes(void) { return CAIFQ_NOALLOC_SCRATCH_BYTES; }

int caifq_lora_linear_bwd_noalloc(const caifq_weight *w, const caifq_lora *lora, const void *dy, const void *x,
                                  const void *hidden, int64_t m, void *dx, void *d_a, void *d_b,
                                  int32_t compute_dtype, void *stream)
{
  const char *who = "caifq_lora_linear_bwd_noalloc";
  const int rc = check_lora(w, lora, who);
  if (rc != CAIFQ_OK)
  {
    return rc;
  }
  CAIFQ_CHECK_ARG(m >= 0, "%s: negative m", who);
  const size_t need = caifq_lora_bwd_workspace_bytes(w, lora, m);
  if (need > CAIFQ_NOALLOC_SCRATCH_BYTES)
  {
    set_error("%s: this call needs %zu bytes of scratch but the built-in buffer holds %u; "
              "use caifq_lora_linear_bwd with a caller-provided workspace (m=%lld rank=%d in=%d out=%d)",
              who, need, CAIFQ_NOALLOC_SCRATCH_BYTES, static_cast<long long>(m), lora->rank, w->in_dim, w->out_dim);
    return CAIFQ_ERR_UNSUPPORTED;
  }
  int dev = 0;
  CAIFQ_CHECK_CUDA(cudaGetDevice(&dev));
  CAIFQ_CHECK_ARG(dev >= 0 && dev < kMaxDevices, "%s: device index %d out of range", who, dev);
  void *scratch = nullptr;
  {
    // one-time set-up per device, with that device current: resolve the array's device address
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_ptr[dev] == nullptr)
    {
      void *ptr = nullptr;
      CAIFQ_CHECK_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
      g_noalloc_ptr[dev] = ptr;
    }
    scratch = g_noalloc_ptr[dev];
  }
  // Nothing in the buffer is assumed: the token reductions clear their fp32
  // accumulator with a memset on `stream` before every use, and dH is fully
  // overwritten before it is read.
  return caifq_lora_linear_bwd(w, lora, dy, x, hidden, m, dx, d_a, d_b, scratch, compute_dtype, stream);
}

// ----------------------------------------------------------------------- MoE

int caifq_moe_topk(const void *probs, int32_t dtype, int32_t *indices, void *values, int32_t batch, int32_t dim,
                   int32_t k, void *stream)
{
  CAIFQ_CHECK_ARG(batch >= 0 && dim > 0 && k > 0, "caifq_moe_topk: bad shape");
  CAIFQ_CHECK_ARG(k <= dim, "caifq_moe_topk: k=%d exceeds dim=%d", k, dim);
  CAIFQ_CHECK_ARG(batch == 0 || (probs && indices && values), "caifq_moe_topk: null pointer");
  return launch_moe_topk(probs, dtype, indices, values, batch, dim, k, static_cast<cudaStream_t>(stream));
}

int caifq_moe_normalize_rows(const void *input, void *output, int32_t dtype, int32_t batch, int32_t dim, void *stream)
{
  CAIFQ_CHECK_ARG(batch >= 0 && dim > 0, "caifq_moe_normalize_rows: bad shape");
  CAIFQ_CHECK_ARG(batch == 0 || (input && output), "caifq_moe_normalize_rows: null pointer");
  return launch_moe_normalize_rows(input, output, dtype, batch, dim, static_cast<cudaStream_t>(stream));
}

int caifq_moe_router_softmax(const void *logits, const void *bias, void *probs, int32_t dtype, int32_t rows,
                             int32_t cols, void *stream)
{
  CAIFQ_CHECK_ARG(rows >= 0 && cols > 0, "caifq_moe_router_softmax: bad shape");
  CAIFQ_CHECK_ARG(is_float_dtype(dtype), "caifq_moe_router_softmax: dtype must be F32, F16 or BF16");
  CAIFQ_CHECK_ARG(rows == 0 || (logits && probs), "caifq_moe_router_softmax: null pointer");
  return launch_moe_router_softmax(logits, bias, probs, dtype, rows, cols, static_cast<cudaStream_t>(stream));
}

int caifq_moe_route_grouped(const void *input, int32_t input_is_logits, const void *selection_bias, void *scores_out,
                            int32_t *indices, void *weights, int32_t dtype, int32_t batch, int32_t dim, int32_t k,
                            int32_t n_group, int32_t topk_group, void *stream)
{
  const char *who = "caifq_moe_route_grouped";
  CAIFQ_CHECK_ARG(batch >= 0 && dim > 0 && k > 0 && k <= dim, "%s: bad shape", who);
  CAIFQ_CHECK_ARG(is_float_dtype(dtype), "%s: dtype must be F32, F16 or BF16", who);
  CAIFQ_CHECK_ARG(n_group >= 1 && n_group <= 1024 && (dim % n_group) == 0 && topk_group >= 1 && topk_group <= n_group,
                  "%s: n_group must divide the expert count and topk_group lie in 1..n_group", who);
  CAIFQ_CHECK_ARG(batch == 0 || (input && indices && weights), "%s: null pointer", who);
  CAIFQ_CHECK_ARG(n_group <= 32, "%s: at most 32 groups", who);
  return launch_moe_route_grouped(input, selection_bias, scores_out, indices, weights, dtype, batch, dim, k, n_group,
                                  topk_group, input_is_logits ? 1 : 0, static_cast<cudaStream_t>(stream));
}

int caifq_moe_router_bwd(const void *grad_weights, const void *probs, const int32_t *indices, const void *balance_bias,
                         const void *z_lse_scaled, void *grad_topk, void *grad_logits, int32_t dtype, int32_t tokens,
                         int32_t experts, int32_t top_k, int32_t sigmoid_gate, int32_t normalize,
                         float routed_scaling_factor, int32_t exact_jacobian, void *stream)
{
  const char *who = "caifq_moe_router_bwd";
  CAIFQ_CHECK_ARG(tokens >= 0 && experts > 0 && top_k > 0 && top_k <= 32 && top_k <= experts,
                  "%s: bad shape tokens=%d experts=%d top_k=%d (top_k <= 32)", who, tokens, experts, top_k);
  CAIFQ_CHECK_ARG(is_float_dtype(dtype), "%s: dtype must be F32, F16 or BF16", who);
  CAIFQ_CHECK_ARG(tokens == 0 || (grad_weights && probs && indices && grad_logits), "%s: null pointer", who);
  CAIFQ_CHECK_ARG(!(sigmoid_gate && (balance_bias || z_lse_scaled)),
                  "%s: sigmoid gating takes no load-balance or z-loss operand", who);
  return launch_moe_router_bwd(grad_weights, probs, indices, balance_bias, z_lse_scaled, grad_topk, grad_logits,
                               dtype, tokens, experts, top_k, sigmoid_gate ? 1 : 0, normalize ? 1 : 0,
                               routed_scaling_factor, exact_jacobian ? 1 : 0, static_cast<cudaStream_t>(stream));
}

// ---- several layers that share their input as one product over the concatenated weights ----
namespace
{
int concat_check(const caifq_weight *ws, int32_t count, int64_t *rows_out, const char *who)
{
  CAIFQ_CHECK_ARG(ws != nullptr && count >= 1 && count <= 8, "%s: 1 to 8 weights", who);
  int64_t rows = 0;
  for (int i = 0; i < count; ++i)
  {
    const int rc = check_weight(&ws[i], who);
    if (rc != CAIFQ_OK)
    {
      return rc;
    }
    CAIFQ_CHECK_ARG(ws[i].in_dim == ws[0].in_dim, "%s: weight %d has in_dim %d, weight 0 has %d", who, i,
                    ws[i].in_dim, ws[0].in_dim);
    CAIFQ_CHECK_ARG((ws[i].out_dim % 8) == 0, "%s: out_dim of weight %d must be a multiple of 8", who, i);
    rows += ws[i].out_dim;
  }
  CAIFQ_CHECK_ARG(rows <= 0x7FFFFFFF, "%s: too many output features", who);
  *rows_out = rows;
  return CAIFQ_OK;
}

int concat_run(const caifq_weight *ws, int32_t count, bool backward, const void *a, int a_dtype, int64_t m,
               void *c, int c_dtype, int compute_dtype, void *workspace, size_t workspace_bytes, cudaStream_t s,
               const char *who)
{
  int64_t rows = 0;
  int rc = concat_check(ws, count, &rows, who);
  if (rc != CAIFQ_OK)
  {
    return rc;
  }
  CAIFQ_CHECK_ARG(compute_dtype == CAIFQ_BF16, "%s: the concatenated operand is bf16: compute dtype must be BF16", who);
  const size_t need = align256(static_cast<size_t>(rows) * static_cast<size_t>(ws[0].in_dim) * 2);
  CAIFQ_CHECK_ARG(workspace != nullptr && workspace_bytes >= need, "%s: workspace of %zu bytes needed, %zu given", who,
                  need, workspace_bytes);
  CAIFQ_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, "%s: workspace must be 256-byte aligned", who);
  if (m == 0)
  {
    return CAIFQ_OK;
  }
  caifq_weight cat = float_weight(workspace, CAIFQ_BF16, static_cast<int>(rows), ws[0].in_dim);
  LinearArgs probe{};
  probe.w = cat;
  probe.backward = backward;
  probe.a = a;
  probe.a_dtype = a_dtype;
  probe.a_prescale = 1.0f;
  probe.m = m;
  probe.c = c;
  probe.c_dtype = c_dtype;
  probe.compute_dtype = compute_dtype;
  if (!umma_supported(probe))
  {
    set_error("%s: needs the tensor-core path (bf16 activations, at least 32 rows, aligned buffers); call the layers "
              "one by one, or caifq_linear_fwd_multi for up to 16 rows",
              who);
    return CAIFQ_ERR_UNSUPPORTED;
  }
  uint8_t *dst = static_cast<uint8_t *>(workspace);
  for (int i = 0; i < count; ++i)
  {
    rc = launch_weight_to_bf16_scaled(ws[i], dst, s);
    if (rc != CAIFQ_OK)
    {
      return rc;
    }
    dst += static_cast<size_t>(ws[i].out_dim) * static_cast<size_t>(ws[i].in_dim) * 2;
  }
  return linear_any(&cat, backward, a, a_dtype, 1.0f, m, c, c_dtype, false, compute_dtype, s, who);
}
}  // namespace

size_t caifq_linear_concat_workspace_bytes(const caifq_weight *ws, int32_t count)
{
  if (ws == nullptr || count < 1)
  {
    return 0;
  }
  size_t rows = 0;
  for (int i = 0; i < count; ++i)
  {
    rows += static_cast<size_t>(ws[i].out_dim);
  }
  return align256(rows * static_cast<size_t>(ws[0].in_dim) * 2);
}

int caifq_linear_fwd_concat(const caifq_weight *ws, int32_t count, const void *x, int32_t x_dtype, int64_t m,
                            void *y, int32_t y_dtype, int32_t compute_dtype, void *workspace, size_t workspace_bytes,
                            void *stream)
{
  return concat_run(ws, count, false, x, x_dtype, m, y, y_dtype, compute_dtype, workspace, workspace_bytes,
                    static_cast<cudaStream_t>(stream), "caifq_linear_fwd_concat");
}

int caifq_linear_dx_concat(const caifq_weight *ws, int32_t count, const void *dy, int32_t dy_dtype, int64_t m,
                           void *dx, int32_t dx_dtype, int32_t compute_dtype, void *workspace, size_t workspace_bytes,
                           void *stream)
{
  return concat_run(ws, count, true, dy, dy_dtype, m, dx, dx_dtype, compute_dtype, workspace, workspace_bytes,
                    static_cast<cudaStream_t>(stream), "caifq_linear_dx_concat");
}

int caifq_rmsnorm_fwd(const void *x, const float *gamma, void *y, float *rms_cache, float epsilon, int32_t dtype,
                      int32_t rows, int32_t dim, void *stream)
{
  const char *who = "caifq_rmsnorm_fwd";
  CAIFQ_CHECK_ARG(rows >= 0 && dim > 0, "%s: bad shape rows=%d dim=%d", who, rows, dim);
  CAIFQ_CHECK_ARG(is_float_dtype(dtype), "%s: dtype must be F32, F16 or BF16", who);
  CAIFQ_CHECK_ARG(rows == 0 || (x && gamma && y), "%s: null pointer", who);
  return launch_rmsnorm_fwd(x, gamma, y, rms_cache, epsilon, dtype, rows, dim, static_cast<cudaStream_t>(stream));
}

int caifq_rmsnorm_bwd(const void *dy, const void *x, const float *gamma, const float *rms_cache, void *dx,
                      float *grad_gamma, int32_t dtype, int32_t rows, int32_t dim, void *stream)
{
  const char *who = "caifq_rmsnorm_bwd";
  CAIFQ_CHECK_ARG(rows >= 0 && dim > 0, "%s: bad shape rows=%d dim=%d", who, rows, dim);
  CAIFQ_CHECK_ARG(is_float_dtype(dtype), "%s: dtype must be F32, F16 or BF16", who);
  CAIFQ_CHECK_ARG(rows == 0 || (dy && x && gamma && rms_cache && dx), "%s: null pointer", who);
  return launch_rmsnorm_bwd(dy, x, gamma, rms_cache, dx, grad_gamma, dtype, rows, dim,
                            static_cast<cudaStream_t>(stream));
}

int caifq_moe_bias_update(void *bias, const int32_t *counts, int32_t from_offsets, int32_t dtype, int32_t experts,
                          float rate, void *stream)
{
  const char *who = "caifq_moe_bias_update";
  CAIFQ_CHECK_ARG(experts > 0, "%s: bad expert count %d", who, experts);
  CAIFQ_CHECK_ARG(is_float_dtype(dtype), "%s: dtype must be F32, F16 or BF16", who);
  CAIFQ_CHECK_ARG(bias != nullptr && counts != nullptr, "%s: null pointer", who);
  return launch_moe_bias_update(bias, counts, dtype, experts, rate, from_offsets ? 1 : 0,
                                static_cast<cudaStream_t>(stream));
}

int caifq_moe_aux_losses(const void *logits, const void *probs, const int32_t *expert_offsets, void *balance_bias,
                         void *lse, void *z_lse_scaled, float *sums, int32_t dtype, int32_t tokens, int32_t experts,
                         int32_t top_k, float balance_weight, float z_weight, void *stream)
{
  const char *who = "caifq_moe_aux_losses";
  CAIFQ_CHECK_ARG(tokens > 0 && experts > 0 && top_k > 0, "%s: bad shape tokens=%d experts=%d top_k=%d", who, tokens,
                  experts, top_k);
  CAIFQ_CHECK_ARG(is_float_dtype(dtype), "%s: dtype must be F32, F16 or BF16", who);
  CAIFQ_CHECK_ARG(sums != nullptr, "%s: sums is null", who);
  CAIFQ_CHECK_ARG(expert_offsets != nullptr || (probs == nullptr && balance_bias == nullptr),
                  "%s: the load-balance terms need expert_offsets", who);
  CAIFQ_CHECK_ARG(logits != nullptr || (lse == nullptr && z_lse_scaled == nullptr),
                  "%s: the z-loss terms need logits", who);
  return launch_moe_aux_losses(logits, probs, expert_offsets, balance_bias, lse, z_lse_scaled, sums, dtype, tokens,
                               experts, top_k, balance_weight, z_weight, static_cast<cudaStream_t>(stream));
}

int caifq_lora_adamw_step(void *a, void *b, const void *d_a, const void *d_b, float *m_a, float *v_a, float *m_b,
                          float *v_b, int32_t rank, int32_t in_dim, int32_t out_dim, int32_t dtype, float lr,
                          float beta1, float beta2, float epsilon, float weight_decay, float bias_correction1,
                          float bias_correction2, void *stream)
{
  const char *who = "caifq_lora_adamw_step";
  CAIFQ_CHECK_ARG(rank > 0 && in_dim > 0 && out_dim > 0, "%s: bad shape", who);
  CAIFQ_CHECK_ARG(is_float_dtype(dtype), "%s: dtype must be F32, F16 or BF16", who);
  CAIFQ_CHECK_ARG(a && b && d_a && d_b && m_a && v_a && m_b && v_b, "%s: null pointer", who);
  CAIFQ_CHECK_ARG(bias_correction1 != 0.0f && bias_correction2 != 0.0f, "%s: zero bias correction", who);
  return launch_lora_adamw(a, b, d_a, d_b, m_a, v_a, m_b, v_b, static_cast<int64_t>(rank) * in_dim,
                           static_cast<int64_t>(out_dim) * rank, dtype, lr, beta1, beta2, epsilon, weight_decay,
                           bias_correction1, bias_correction2, static_cast<cudaStream_t>(stream));
}

int caifq_scale(const void *src, void *dst, int32_t dtype, float factor, int64_t n, void *stream)
{
  CAIFQ_CHECK_ARG(n >= 0, "caifq_scale: negative n");
  CAIFQ_CHECK_ARG(is_float_dtype(dtype), "caifq_scale: dtype must be F32, F16 or BF16");
  CAIFQ_CHECK_ARG(n == 0 || (src && dst), "caifq_scale: null pointer");
  if (n == 0)
  {
    return CAIFQ_OK;
  }
  return launch_scale(src, dst, dtype, factor, n, static_cast<cudaStream_t>(stream));
}

int caifq_moe_build_dispatch(const int32_t *expert_indices, int32_t num_tokens, int32_t top_k, int32_t num_experts,
                             int32_t capacity, int32_t *dispatch_map, int32_t *expert_offsets, void *stream)
{
  CAIFQ_CHECK_ARG(num_tokens >= 0 && top_k > 0 && num_experts > 0, "caifq_moe_build_dispatch: bad shape");
  CAIFQ_CHECK_ARG(expert_offsets != nullptr, "caifq_moe_build_dispatch: null expert_offsets");
  CAIFQ_CHECK_ARG(num_tokens == 0 || (expert_indices && dispatch_map), "caifq_moe_build_dispatch: null pointer");
  return launch_moe_build_dispatch(expert_indices, num_tokens, top_k, num_experts, capacity, dispatch_map,
                                   expert_offsets, static_cast<cudaStream_t>(stream));
}

int caifq_moe_dispatch(const void *input, int32_t dtype, const int32_t *expert_indices, const int32_t *dispatch_map,
                       const int32_t *expert_offsets, void *expert_buffer, int32_t num_tokens, int32_t dim,
                       int32_t top_k, void *stream)
{
  CAIFQ_CHECK_ARG(num_tokens >= 0 && dim > 0 && top_k > 0, "caifq_moe_dispatch: bad shape");
  CAIFQ_CHECK_ARG(num_tokens == 0 || (input && expert_indices && dispatch_map && expert_offsets && expert_buffer),
                  "caifq_moe_dispatch: null pointer");
  return launch_moe_dispatch(input, dtype, expert_indices, dispatch_map, expert_offsets, expert_buffer, num_tokens,
                             dim, top_k, static_cast<cudaStream_t>(stream));
}

int caifq_moe_combine(const void *expert_buffer, int32_t dtype, const int32_t *expert_indices,
                      const void *expert_weights, const int32_t *dispatch_map, const int32_t *expert_offsets,
                      void *output, int32_t num_tokens, int32_t dim, int32_t top_k, void *stream)
{
  CAIFQ_CHECK_ARG(num_tokens >= 0 && dim > 0 && top_k > 0, "caifq_moe_combine: bad shape");
  CAIFQ_CHECK_ARG(num_tokens == 0 ||
                      (expert_buffer && expert_indices && expert_weights && dispatch_map && expert_offsets && output),
                  "caifq_moe_combine: null pointer");
  return launch_moe_combine(expert_buffer, dtype, expert_indices, expert_weights, dispatch_map, expert_offsets,
                            output, num_tokens, dim, top_k, static_cast<cudaStream_t>(stream));
}

int caifq_moe_combine_bwd_grad_expert(const void *grad_output, int32_t dtype, const int32_t *expert_indices,
                                      const void *expert_weights, const int32_t *dispatch_map,
                                      const int32_t *expert_offsets, void *grad_expert_buffer, int32_t num_tokens,
                                      int32_t dim, int32_t top_k, void *stream)
{
  CAIFQ_CHECK_ARG(num_tokens >= 0 && dim > 0 && top_k > 0, "caifq_moe_combine_bwd_grad_expert: bad shape");
  CAIFQ_CHECK_ARG(num_tokens == 0 || (grad_output && expert_indices && expert_weights && dispatch_map &&
                                      expert_offsets && grad_expert_buffer),
                  "caifq_moe_combine_bwd_grad_expert: null pointer");
  return launch_moe_combine_bwd_grad_expert(grad_output, dtype, expert_indices, expert_weights, dispatch_map,
                                            expert_offsets, grad_expert_buffer, num_tokens, dim, top_k,
                                            static_cast<cudaStream_t>(stream));
}

int caifq_moe_combine_bwd_grad_weights(const void *grad_output, const void *expert_buffer, int32_t dtype,
                                       const int32_t *expert_indices, const int32_t *dispatch_map,
                                       const int32_t *expert_offsets, void *grad_weights, int32_t num_tokens,
                                       int32_t dim, int32_t top_k, void *stream)
{
  CAIFQ_CHECK_ARG(num_tokens >= 0 && dim > 0 && top_k > 0, "caifq_moe_combine_bwd_grad_weights: bad shape");
  CAIFQ_CHECK_ARG(num_tokens == 0 || (grad_output && expert_buffer && expert_indices && dispatch_map &&
                                      expert_offsets && grad_weights),
                  "caifq_moe_combine_bwd_grad_weights: null pointer");
  return launch_moe_combine_bwd_grad_weights(grad_output, expert_buffer, dtype, expert_indices, dispatch_map,
                                             expert_offsets, grad_weights, num_tokens, dim, top_k,
                                             static_cast<cudaStream_t>(stream));
}

int caifq_moe_dispatch_bwd(const void *grad_expert_buffer, int32_t dtype, const int32_t *expert_indices,
                           const int32_t *dispatch_map, const int32_t *expert_offsets, void *grad_input,
                           int32_t num_tokens, int32_t dim, int32_t top_k, void *stream)
{
  CAIFQ_CHECK_ARG(num_tokens >= 0 && dim > 0 && top_k > 0, "caifq_moe_dispatch_bwd: bad shape");
  CAIFQ_CHECK_ARG(num_tokens == 0 ||
                      (grad_expert_buffer && expert_indices && dispatch_map && expert_offsets && grad_input),
                  "caifq_moe_dispatch_bwd: null pointer");
  return launch_moe_dispatch_bwd(grad_expert_buffer, dtype, expert_indices, dispatch_map, expert_offsets, grad_input,
                                 num_tokens, dim, top_k, static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------ grouped experts

static int check_experts(const caifq_weight *gate, const caifq_weight *up, const caifq_weight *down,
                         int32_t num_experts, const int32_t *offsets, const char *who)
{
  // gate == nullptr: experts without a gate projection (the reference's UseGated() == false)
  CAIFQ_CHECK_ARG(up && down && offsets, "%s: null expert table", who);
  CAIFQ_CHECK_ARG(num_experts > 0, "%s: num_experts must be positive", who);
  const int in_dim = up[0].in_dim;
  const int hidden = up[0].out_dim;
  for (int e = 0; e < num_experts; ++e)
  {
    int rc = (gate != nullptr) ? check_weight(&gate[e], who) : CAIFQ_OK;
    if (rc == CAIFQ_OK)
    {
      rc = check_weight(&up[e], who);
    }
    if (rc == CAIFQ_OK)
    {
      rc = check_weight(&down[e], who);
    }
    if (rc != CAIFQ_OK)
    {
      return rc;
    }
    CAIFQ_CHECK_ARG(up[e].in_dim == in_dim && down[e].out_dim == in_dim && up[e].out_dim == hidden &&
                        down[e].in_dim == hidden &&
                        (gate == nullptr || (gate[e].in_dim == in_dim && gate[e].out_dim == hidden)),
                    "%s: expert %d has inconsistent dims", who, e);
    CAIFQ_CHECK_ARG(offsets[e + 1] >= offsets[e], "%s: expert offsets must be non-decreasing", who);
  }
  return CAIFQ_OK;
}

// One product for every expert of a run: a single grouped tensor-core launch when the kernel takes
// the experts (same quantized shape, bf16 rows), else one call per expert - the reference's loop
// (src/caif_device_moe_layer.cpp:534-557).
int grouped_linear(const caifq_weight *ws, int num_experts, const int32_t *offsets, bool backward, const void *a,
                   void *c, int dtype, bool accumulate, int compute_dtype, cudaStream_t s, const char *who)
{
  GroupedLinearArgs g{};
  g.weights = ws;
  g.num_experts = num_experts;
  g.offsets = offsets;
  g.backward = backward;
  g.a = a;
  g.a_dtype = dtype;
  g.c = c;
  g.c_dtype = dtype;
  g.accumulate = accumulate;
  g.compute_dtype = compute_dtype;
  const Force force = forced_path();
  static const bool grouping = []() {
    const char *e = std::getenv("CAIFQ_GROUPED");   // "0": always loop over the experts
    return e == nullptr || e[0] != '0';
  }();
  if (grouping && (force == Force::None || force == Force::Umma) && umma_grouped_supported(g))
  {
    set_path("umma-grouped");
    return launch_linear_umma_grouped(g, s);
  }
  const size_t es = dtype_bytes(dtype);
  const int64_t a_cols = backward ? ws[0].out_dim : ws[0].in_dim;
  const int64_t c_cols = backward ? ws[0].in_dim : ws[0].out_dim;
  for (int e = 0; e < num_experts; ++e)
  {
    const int64_t off = offsets[e];
    const int64_t cnt = offsets[e + 1] - off;
    if (cnt == 0)
    {
      continue;
    }
    const int r = linear_any(&ws[e], backward, static_cast<const char *>(a) + off * a_cols * es, dtype, 1.0f, cnt,
                             static_cast<char *>(c) + off * c_cols * es, dtype, accumulate, compute_dtype, s, who);
    if (r != CAIFQ_OK)
    {
      return r;
    }
  }
  return CAIFQ_OK;
}

int caifq_grouped_expert_fwd(const caifq_weight *gate, const caifq_weight *up, const caifq_weight *down,
                             int32_t num_experts, const int32_t *expert_offsets_host, const void *x, void *out,
                             void *gate_out, void *up_out, void *hidden_ws, int32_t dtype, int32_t compute_dtype,
                             void *stream)
{
  const char *who = "caifq_grouped_expert_fwd";
  const int rc = check_experts(gate, up, down, num_experts, expert_offsets_host, who);
  if (rc != CAIFQ_OK)
  {
    return rc;
  }
  CAIFQ_CHECK_ARG(is_float_dtype(dtype), "%s: dtype must be F32, F16 or BF16", who);
  const int64_t total = expert_offsets_host[num_experts];
  if (total == 0)
  {
    return CAIFQ_OK;
  }
  CAIFQ_CHECK_ARG(x && out && up_out && hidden_ws && (gate == nullptr || gate_out), "%s: null pointer", who);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t hid = up[0].out_dim;
  int r = CAIFQ_OK;
  if (gate == nullptr)
  {
    // hidden = SiLU(up(x)), src/caif_device_moe_frozen_expert.cpp:158-162
    r = grouped_linear(up, num_experts, expert_offsets_host, false, x, up_out, dtype, false, compute_dtype, s, who);
    if (r == CAIFQ_OK)
    {
      r = launch_silu_fwd(up_out, hidden_ws, dtype, total * hid, s);
    }
    if (r != CAIFQ_OK)
    {
      return r;
    }
    return grouped_linear(down, num_experts, expert_offsets_host, false, hidden_ws, out, dtype, false, compute_dtype,
                          s, who);
  }
  GroupedSwigluArgs fused{};
  fused.gate = gate;
  fused.up = up;
  fused.num_experts = num_experts;
  fused.offsets = expert_offsets_host;
  fused.x = x;
  fused.gate_out = gate_out;
  fused.up_out = up_out;
  fused.hidden = hidden_ws;
  fused.dtype = dtype;
  fused.compute_dtype = compute_dtype;
  static const bool fuse_swiglu = []() {
    const char *e = std::getenv("CAIFQ_FUSED_SWIGLU");   // "0": separate gate, up and SwiGLU launches
    return e == nullptr || e[0] != '0';
  }();
  if (fuse_swiglu && forced_path() == Force::None && umma_swiglu_supported(fused))
  {
    // gate, up and the SwiGLU in one pass over the packed rows
    r = launch_linear_umma_swiglu(fused, s);
    if (r != CAIFQ_OK)
    {
      return r;
    }
  }
  else
  {
    r = grouped_linear(up, num_experts, expert_offsets_host, false, x, up_out, dtype, false, compute_dtype, s, who);
    if (r == CAIFQ_OK)
    {
      r = grouped_linear(gate, num_experts, expert_offsets_host, false, x, gate_out, dtype, false, compute_dtype, s,
                         who);
    }
    if (r != CAIFQ_OK)
    {
      return r;
    }
    r = launch_swiglu_fwd(gate_out, up_out, hidden_ws, dtype, total * hid, s);
    if (r != CAIFQ_OK)
    {
      return r;
    }
  }
  return grouped_linear(down, num_experts, expert_offsets_host, false, hidden_ws, out, dtype, false, compute_dtype, s,
                        who);
}

int caifq_grouped_expert_bwd(const caifq_weight *gate, const caifq_weight *up, const caifq_weight *down,
                             int32_t num_experts, const int32_t *expert_offsets_host, const void *dy,
                             const void *gate_out, const void *up_out, void *dx, void *ws, int32_t dtype,
                             int32_t compute_dtype, void *stream)
{
  const char *who = "caifq_grouped_expert_bwd";
  const int rc = check_experts(gate, up, down, num_experts, expert_offsets_host, who);
  if (rc != CAIFQ_OK)
  {
    return rc;
  }
  CAIFQ_CHECK_ARG(is_float_dtype(dtype), "%s: dtype must be F32, F16 or BF16", who);
  const int64_t total = expert_offsets_host[num_experts];
  if (total == 0)
  {
    return CAIFQ_OK;
  }
  CAIFQ_CHECK_ARG(dy && up_out && dx && ws && (gate == nullptr || gate_out), "%s: null pointer", who);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t es = dtype_bytes(dtype);
  const int64_t hid = up[0].out_dim;
  char *g_hidden = static_cast<char *>(ws);
  char *g_gate = g_hidden + total * hid * es;
  char *g_up = g_gate + total * hid * es;
  int r = CAIFQ_OK;
  bool swiglu_done = false;
  if (gate != nullptr && dtype == CAIFQ_BF16 && forced_path() == Force::None)
  {
    // down^T with the SwiGLU backward in its epilogue: g_gate and g_up leave the launch, g_hidden is never stored
    GroupedLinearArgs g{};
    g.weights = down;
    g.num_experts = num_experts;
    g.offsets = expert_offsets_host;
    g.backward = true;
    g.a = dy;
    g.a_dtype = dtype;
    g.c = g_gate;
    g.c_dtype = dtype;
    g.accumulate = false;
    g.compute_dtype = compute_dtype;
    static const bool grouping = []() {
      const char *e = std::getenv("CAIFQ_GROUPED");
      return e == nullptr || e[0] != '0';
    }();
    static const bool fuse = []() {
      const char *e = std::getenv("CAIFQ_FUSED_SWIGLU");
      return e == nullptr || e[0] != '0';
    }();
    if (grouping && fuse && umma_grouped_supported(g) && (reinterpret_cast<uintptr_t>(gate_out) & 15u) == 0 &&
        (reinterpret_cast<uintptr_t>(up_out) & 15u) == 0 && (reinterpret_cast<uintptr_t>(g_up) & 15u) == 0)
    {
      g.sb_gate = gate_out;
      g.sb_up = up_out;
      g.sb_g_up = g_up;
      set_path("umma-grouped");
      r = launch_linear_umma_grouped(g, s);
      if (r != CAIFQ_OK)
      {
        return r;
      }
      swiglu_done = true;
    }
  }
  if (!swiglu_done)
  {
    r = grouped_linear(down, num_experts, expert_offsets_host, true, dy, g_hidden, dtype, false, compute_dtype, s,
                       who);
    if (r != CAIFQ_OK)
    {
      return r;
    }
  }
  if (gate == nullptr)
  {
    // g_up = SiLUBackward(up_out, g_hidden); dx = up.Bwd(g_up), src/caif_device_moe_frozen_expert.cpp:318-331
    r = launch_silu_bwd(up_out, g_hidden, g_up, dtype, total * hid, s);
    if (r != CAIFQ_OK)
    {
      return r;
    }
    return grouped_linear(up, num_experts, expert_offsets_host, true, g_up, dx, dtype, false, compute_dtype, s, who);
  }
  if (!swiglu_done)
  {
    r = launch_swiglu_bwd(g_hidden, gate_out, up_out, g_gate, g_up, dtype, total * hid, s);
    if (r != CAIFQ_OK)
    {
      return r;
    }
  }
  if (up[0].storage == CAIFQ_BF16 && gate[0].storage == CAIFQ_BF16 && up[0].scales == nullptr &&
      gate[0].scales == nullptr && forced_path() == Force::None)
  {
    // (expanded int8 experts carry a per-expert scale for the epilogue, which differs between the two
    // projections: they keep the two launches)
    // Stacked bf16 experts (the expanded copies): dx = g_up . W_up + g_gate . W_gate as ONE launch whose
    // reduction runs over both operand pairs, accumulated in fp32 and rounded once (the reference rounds each
    // product to the storage dtype and adds them: one more rounding, same bound).  No read-modify-write of dx.
    GroupedLinearArgs g{};
    g.weights = up;
    g.num_experts = num_experts;
    g.offsets = expert_offsets_host;
    g.backward = true;
    g.a = g_up;
    g.a_dtype = dtype;
    g.c = dx;
    g.c_dtype = dtype;
    g.accumulate = false;
    g.compute_dtype = compute_dtype;
    GroupedLinearArgs g2 = g;
    g2.weights = gate;
    g2.a = g_gate;
    if (umma_grouped_supported(g) && umma_grouped_supported(g2) && num_experts <= 80)
    {
      g.weights2 = gate;
      g.a2 = g_gate;
      set_path("umma-grouped");
      return launch_linear_umma_grouped(g, s);
    }
  }
  // dx = round(up.Bwd(g_up)); dx = round(round(gate.Bwd(g_gate)) + dx): the reference's Add(gi_up, gi_gate)
  r = grouped_linear(up, num_experts, expert_offsets_host, true, g_up, dx, dtype, false, compute_dtype, s, who);
  if (r != CAIFQ_OK)
  {
    return r;
  }
  return grouped_linear(gate, num_experts, expert_offsets_host, true, g_gate, dx, dtype, true, compute_dtype, s, who);
}

}  // extern "C"

// ---- frozen experts on bf16 copies of their weights, expanded once per step -----------------------

namespace
{
struct ExpandedExperts
{
  bool ok;
  size_t up_off, down_off, gate_off, total;
};

// Experts of one quantized shape on bf16 rows whose products the grouped tensor-core launches take.
ExpandedExperts expanded_layout(const caifq_weight *gate, const caifq_weight *up, const caifq_weight *down,
                                int num_experts, int dtype, int compute_dtype)
{
  ExpandedExperts l{};
  l.ok = false;
  if (up == nullptr || down == nullptr || num_experts < 1 || dtype != CAIFQ_BF16)
  {
    return l;
  }
  const caifq_weight &u0 = up[0];
  const caifq_weight &d0 = down[0];
  const bool i8 = (u0.storage == CAIFQ_I8);
  if (!(i8 && (compute_dtype == CAIFQ_BF16 || compute_dtype == CAIFQ_F32)) &&
      !(u0.storage == CAIFQ_I4 && compute_dtype == CAIFQ_BF16))
  {
    return l;
  }
  if ((u0.in_dim % 128) != 0 || (u0.out_dim % 128) != 0)
  {
    return l;
  }
  for (int e = 0; e < num_experts; ++e)
  {
    const caifq_weight *set[3] = {&up[e], &down[e], gate != nullptr ? &gate[e] : nullptr};
    for (int k = 0; k < 3; ++k)
    {
      const caifq_weight *w = set[k];
      if (w == nullptr)
      {
        continue;
      }
      const caifq_weight &r = (k == 1) ? d0 : u0;
      if (w->storage != u0.storage || w->scheme != u0.scheme || w->group_size != u0.group_size ||
          w->in_dim != r.in_dim || w->out_dim != r.out_dim || (reinterpret_cast<uintptr_t>(w->codes) & 15u) != 0 ||
          (i8 && w->scales != nullptr && w->scheme != CAIFQ_PER_TENSOR) || (!i8 && w->scales == nullptr) ||
          (!i8 && (w->group_size % 32 != 0 || w->in_dim % w->group_size != 0)))
      {
        return l;
      }
    }
  }
  const size_t one = align256(static_cast<size_t>(u0.in_dim) * static_cast<size_t>(u0.out_dim) * 2 * num_experts);
  l.up_off = 0;
  l.down_off = one;
  l.gate_off = 2 * one;
  l.total = (gate != nullptr ? 3 : 2) * one;
  l.ok = true;
  return l;
}

// bf16 views of the expanded copies; an int8 expert's per-tensor scale rides in `scales` for the epilogue
void expanded_views(const caifq_weight *src, int num_experts, const char *base, std::vector<caifq_weight> &out)
{
  out.resize(static_cast<size_t>(num_experts));
  const size_t stride = static_cast<size_t>(src[0].in_dim) * static_cast<size_t>(src[0].out_dim) * 2;
  for (int e = 0; e < num_experts; ++e)
  {
    caifq_weight w{};
    w.codes = base + static_cast<size_t>(e) * stride;
    w.scales = (src[e].storage == CAIFQ_I8) ? src[e].scales : nullptr;
    w.storage = CAIFQ_BF16;
    w.scheme = CAIFQ_PER_TENSOR;
    w.group_size = src[e].group_size;
    w.in_dim = src[e].in_dim;
    w.out_dim = src[e].out_dim;
    out[static_cast<size_t>(e)] = w;
  }
}

// every product of the step must be a grouped tensor-core launch on the views (the per-expert loop would not
// know about the scale riding in `scales`)
bool views_supported(const std::vector<caifq_weight> &ws, int num_experts, const int32_t *offsets, bool backward,
                     const void *a, void *c, bool accumulate, int compute_dtype)
{
  GroupedLinearArgs g{};
  g.weights = ws.data();
  g.num_experts = num_experts;
  g.offsets = offsets;
  g.backward = backward;
  g.a = a;
  g.a_dtype = CAIFQ_BF16;
  g.c = c;
  g.c_dtype = CAIFQ_BF16;
  g.accumulate = accumulate;
  g.compute_dtype = compute_dtype;
  return forced_path() == Force::None && umma_grouped_supported(g);
}
}  // namespace

extern "C" {

size_t caifq_grouped_expert_expanded_bytes(const caifq_weight *gate, const caifq_weight *up, const caifq_weight *down,
                                           int32_t num_experts, int32_t dtype, int32_t compute_dtype)
{
  const ExpandedExperts l = expanded_layout(gate, up, down, num_experts, dtype, compute_dtype);
  return l.ok ? l.total : 0;
}

int caifq_grouped_expert_expand(const caifq_weight *gate, const caifq_weight *up, const caifq_weight *down,
                                int32_t num_experts, void *expanded, int32_t dtype, int32_t compute_dtype, void *stream)
{
  const char *who = "caifq_grouped_expert_expand";
  const ExpandedExperts l = expanded_layout(gate, up, down, num_experts, dtype, compute_dtype);
  if (!l.ok)
  {
    set_error("%s: these experts are not expanded (caifq_grouped_expert_expanded_bytes is 0)", who);
    return CAIFQ_ERR_UNSUPPORTED;
  }
  CAIFQ_CHECK_ARG(expanded != nullptr && (reinterpret_cast<uintptr_t>(expanded) & 255u) == 0,
                  "%s: the buffer must be 256-byte aligned", who);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  char *base = static_cast<char *>(expanded);
  int r = launch_expand_grouped_to_bf16(up, num_experts, base + l.up_off, s);
  if (r == CAIFQ_OK)
  {
    r = launch_expand_grouped_to_bf16(down, num_experts, base + l.down_off, s);
  }
  if (r == CAIFQ_OK && gate != nullptr)
  {
    r = launch_expand_grouped_to_bf16(gate, num_experts, base + l.gate_off, s);
  }
  return r;
}

int caifq_grouped_expert_fwd_expanded(const caifq_weight *gate, const caifq_weight *up, const caifq_weight *down,
                                      int32_t num_experts, const int32_t *expert_offsets_host, const void *x, void *out,
                                      void *gate_out, void *up_out, void *hidden_ws, const void *expanded,
                                      int32_t dtype, int32_t compute_dtype, void *stream)
{
  const char *who = "caifq_grouped_expert_fwd_expanded";
  const int rc = check_experts(gate, up, down, num_experts, expert_offsets_host, who);
  if (rc != CAIFQ_OK)
  {
    return rc;
  }
  const ExpandedExperts l = expanded_layout(gate, up, down, num_experts, dtype, compute_dtype);
  if (l.ok && expanded != nullptr && x != nullptr && out != nullptr && hidden_ws != nullptr && up_out != nullptr)
  {
    const char *base = static_cast<const char *>(expanded);
    std::vector<caifq_weight> vu, vd, vg;
    expanded_views(up, num_experts, base + l.up_off, vu);
    expanded_views(down, num_experts, base + l.down_off, vd);
    if (gate != nullptr)
    {
      expanded_views(gate, num_experts, base + l.gate_off, vg);
    }
    bool ok = views_supported(vu, num_experts, expert_offsets_host, false, x, up_out, false, compute_dtype) &&
              views_supported(vd, num_experts, expert_offsets_host, false, hidden_ws, out, false, compute_dtype);
    if (ok && gate != nullptr)
    {
      ok = gate_out != nullptr &&
           views_supported(vg, num_experts, expert_offsets_host, false, x, gate_out, false, compute_dtype);
    }
    if (ok)
    {
      return caifq_grouped_expert_fwd(gate != nullptr ? vg.data() : nullptr, vu.data(), vd.data(), num_experts,
                                      expert_offsets_host, x, out, gate_out, up_out, hidden_ws, dtype, compute_dtype,
                                      stream);
    }
  }
  return caifq_grouped_expert_fwd(gate, up, down, num_experts, expert_offsets_host, x, out, gate_out, up_out, hidden_ws,
                                  dtype, compute_dtype, stream);
}

int caifq_grouped_expert_bwd_expanded(const caifq_weight *gate, const caifq_weight *up, const caifq_weight *down,
                                      int32_t num_experts, const int32_t *expert_offsets_host, const void *dy,
                                      const void *gate_out, const void *up_out, void *dx, void *ws,
                                      const void *expanded, int32_t dtype, int32_t compute_dtype, void *stream)
{
  const char *who = "caifq_grouped_expert_bwd_expanded";
  const int rc = check_experts(gate, up, down, num_experts, expert_offsets_host, who);
  if (rc != CAIFQ_OK)
  {
    return rc;
  }
  const ExpandedExperts l = expanded_layout(gate, up, down, num_experts, dtype, compute_dtype);
  if (l.ok && expanded != nullptr && dy != nullptr && dx != nullptr && ws != nullptr)
  {
    const char *base = static_cast<const char *>(expanded);
    std::vector<caifq_weight> vu, vd, vg;
    expanded_views(up, num_experts, base + l.up_off, vu);
    expanded_views(down, num_experts, base + l.down_off, vd);
    if (gate != nullptr)
    {
      expanded_views(gate, num_experts, base + l.gate_off, vg);
    }
    bool ok = views_supported(vd, num_experts, expert_offsets_host, true, dy, ws, false, compute_dtype) &&
              views_supported(vu, num_experts, expert_offsets_host, true, ws, dx, false, compute_dtype);
    if (ok && gate != nullptr)
    {
      ok = views_supported(vg, num_experts, expert_offsets_host, true, ws, dx, true, compute_dtype);
    }
    if (ok)
    {
      return caifq_grouped_expert_bwd(gate != nullptr ? vg.data() : nullptr, vu.data(), vd.data(), num_experts,
                                      expert_offsets_host, dy, gate_out, up_out, dx, ws, dtype, compute_dtype, stream);
    }
  }
  return caifq_grouped_expert_bwd(gate, up, down, num_experts, expert_offsets_host, dy, gate_out, up_out, dx, ws, dtype,
                                  compute_dtype, stream);
}

}  // extern "C"
