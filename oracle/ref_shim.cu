// C-linkage doorway onto the reference's own device kernels.
//
// TEST INFRASTRUCTURE ONLY.  oracle/build.py compiles this file together with
// the reference's unmodified src/caif_cuda_kernels_quant.cu, src/caif_cuda_kernels_moe.cu,
// src/caif_cuda_kernels_attention_support.cu (the router's softmax),
// src/caif_cuda_kernels_elementwise.cu and src/caif_cuda_kernels_optimizers.cu (the AdamW step of
// the LoRA factors) (read in place from the reference checkout,
// never copied) into oracle/_ref/libcaif_ref_kernels.so.  The GPU tests load
// that library to check the CPU oracle and the product kernels bit for bit
// against what the reference itself computes.  Every pointer is a device
// pointer; every call is asynchronous on `stream`.
#define USE_CAIF_CUDA 1
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cstdint>

#include "caif_cuda_kernels_quant.cuh"
#include "caif_cuda_kernels_moe.cuh"
#include "caif_cuda_kernels_attention_support.cuh"
#include "caif_cuda_kernels_elementwise.cuh"
#include "caif_cuda_kernels_optimizers.cuh"
#include "caif_cuda_kernels_activations.cuh"
#include "caif_cuda_kernels_normalization.cuh"

// The launches of CAIF_DeviceMoERouter::BackwardRoutingAuxAware (src/caif_device_moe_router.cpp:529-733) up to
// grad_logits, in its order and with its operand order: the normalize Jacobian over the chosen scores,
// Scale by routed_scaling_factor, Zeros + ScatterAdd into [tokens, experts], AddBias of the load-balance
// column term, then SoftmaxBackward called as (probs, grad_probs, grad_logits) -- the reference passes
// the cached probabilities in the grad_output slot and grad_probs in the output slot -- and the z-loss
// term; for sigmoid gating SigmoidBackward instead.  grad_topk [tokens, k] and grad_probs
// [tokens, experts] are scratch the caller provides.
template <typename T>
static void router_backward_chain(const T *grad_w, const T *probs, const int *indices, const T *balance_bias,
                                  const T *z_lse_scaled, T *grad_topk, T *grad_probs, T *grad_logits, int tokens,
                                  int experts, int k, int sigmoid_gate, int normalize, float scaling, cudaStream_t s)
{
  if (normalize != 0)
  {
    launch_normalize_rows_backward_topk_gather<T>(grad_w, probs, indices, grad_topk, tokens, experts, k, s);
  }
  else
  {
    cudaMemcpyAsync(grad_topk, grad_w, sizeof(T) * static_cast<size_t>(tokens) * k, cudaMemcpyDeviceToDevice, s);
  }
  if (scaling != 1.0f)
  {
    launch_elementwise_mul_scalar<T>(grad_topk, scaling, grad_topk, static_cast<int64_t>(tokens) * k, s);
  }
  cudaMemsetAsync(grad_probs, 0, sizeof(T) * static_cast<size_t>(tokens) * experts, s);
  launch_scatter_add<T>(grad_topk, indices, grad_probs, tokens, k, experts, s);
  if (sigmoid_gate != 0)
  {
    launch_sigmoid_backward<T>(grad_probs, probs, grad_logits, static_cast<int64_t>(tokens) * experts, s);
    return;
  }
  if (balance_bias != nullptr)
  {
    launch_bias_add_2d<T>(grad_probs, balance_bias, grad_probs, tokens, experts, s);
  }
  launch_attention_softmax_backward<T>(probs, grad_probs, grad_logits, tokens, experts, s);
  if (z_lse_scaled != nullptr)
  {
    launch_moe_z_loss_grad<T>(z_lse_scaled, probs, grad_logits, tokens, experts, s);
  }
}

extern "C" {

void ref_quantize_int8_per_tensor(const float *x, void *q, void *scale, int64_t n, void *stream)
{
  launch_quantize_int8_per_tensor(x, q, scale, n, static_cast<cudaStream_t>(stream));
}

void ref_dequantize_int8_per_tensor(const void *q, float *out, const void *scale, int64_t n, void *stream)
{
  launch_dequantize_int8_per_tensor(q, out, scale, n, static_cast<cudaStream_t>(stream));
}

void ref_quantize_int8_per_channel(const float *x, void *q, void *scales, int rows, int cols, void *stream)
{
  launch_quantize_int8_per_channel(x, q, scales, rows, cols, static_cast<cudaStream_t>(stream));
}

void ref_dequantize_int8_per_channel(const void *q, float *out, const void *scales, int rows, int cols, void *stream)
{
  launch_dequantize_int8_per_channel(q, out, scales, rows, cols, static_cast<cudaStream_t>(stream));
}

void ref_quantize_int4(const float *x, void *packed, void *scales, int64_t n, int group, void *stream)
{
  launch_quantize_to_int4(x, packed, scales, n, group, static_cast<cudaStream_t>(stream));
}

void ref_dequantize_int4(const void *packed, const void *scales, float *out, int64_t n, int group, void *stream)
{
  launch_dequantize_int4(packed, scales, out, n, group, static_cast<cudaStream_t>(stream));
}

void ref_fp32_to_bf16(const float *x, void *y, int64_t n, void *stream)
{
  launch_convert_fp32_to_bf16(x, y, n, static_cast<cudaStream_t>(stream));
}

void ref_fp32_to_fp16(const float *x, void *y, int64_t n, void *stream)
{
  launch_convert_fp32_to_fp16(x, y, n, static_cast<cudaStream_t>(stream));
}

void ref_topk_f32(const float *input, int *indices, float *values, int batch, int dim, int k, void *stream)
{
  launch_topk<float>(input, indices, values, batch, dim, k, static_cast<cudaStream_t>(stream));
}

void ref_normalize_rows_f32(const float *input, float *output, int batch, int dim, void *stream)
{
  launch_normalize_rows<float>(input, output, batch, dim, static_cast<cudaStream_t>(stream));
}

void ref_moe_dispatch_f32(const float *input, float *buffer, int num_tokens, int dim, int top_k,
                          const int *expert_indices, const int *dispatch_map, const int *expert_offsets, void *stream)
{
  launch_moe_dispatch<float>(input, expert_indices, dispatch_map, buffer, expert_offsets, num_tokens, dim, top_k,
                             static_cast<cudaStream_t>(stream));
}

void ref_moe_combine_f32(const float *buffer, float *output, int num_tokens, int dim, int top_k,
                         const int *expert_indices, const float *expert_weights, const int *dispatch_map,
                         const int *expert_offsets, void *stream)
{
  launch_moe_combine<float>(buffer, expert_indices, expert_weights, dispatch_map, expert_offsets, output, num_tokens,
                            dim, top_k, static_cast<cudaStream_t>(stream));
}

void ref_moe_combine_bwd_grad_expert_f32(const float *grad_output, float *grad_buffer, int num_tokens, int dim,
                                         int top_k, const int *expert_indices, const float *expert_weights,
                                         const int *dispatch_map, const int *expert_offsets, void *stream)
{
  launch_moe_combine_backward_grad_expert<float>(grad_output, expert_indices, expert_weights, dispatch_map,
                                                 expert_offsets, grad_buffer, num_tokens, dim, top_k,
                                                 static_cast<cudaStream_t>(stream));
}

void ref_moe_combine_bwd_grad_weights_f32(const float *grad_output, const float *buffer, float *grad_weights,
                                          int num_tokens, int dim, int top_k, const int *expert_indices,
                                          const int *dispatch_map, const int *expert_offsets, void *stream)
{
  launch_moe_combine_backward_grad_weights<float>(grad_output, buffer, expert_indices, dispatch_map, expert_offsets,
                                                  grad_weights, num_tokens, dim, top_k,
                                                  static_cast<cudaStream_t>(stream));
}

void ref_moe_dispatch_bwd_f32(const float *grad_buffer, float *grad_input, int num_tokens, int dim, int top_k,
                              const int *expert_indices, const int *dispatch_map, const int *expert_offsets,
                              void *stream)
{
  launch_moe_dispatch_backward<float>(grad_buffer, expert_indices, dispatch_map, expert_offsets, grad_input, num_tokens,
                                      dim, top_k, static_cast<cudaStream_t>(stream));
}

// the router's score path: AddBias, Softmax, Scale
void ref_softmax_f32(const float *input, float *output, int rows, int cols, void *stream)
{
  launch_attention_softmax<float>(input, output, rows, cols, static_cast<cudaStream_t>(stream));
}

void ref_softmax_bf16(const void *input, void *output, int rows, int cols, void *stream)
{
  launch_attention_softmax<__nv_bfloat16>(static_cast<const __nv_bfloat16 *>(input),
                                          static_cast<__nv_bfloat16 *>(output), rows, cols,
                                          static_cast<cudaStream_t>(stream));
}

void ref_bias_add_f32(const float *input, const float *bias, float *output, int batch, int units, void *stream)
{
  launch_bias_add_2d<float>(input, bias, output, batch, units, static_cast<cudaStream_t>(stream));
}

void ref_bias_add_bf16(const void *input, const void *bias, void *output, int batch, int units, void *stream)
{
  launch_bias_add_2d<__nv_bfloat16>(static_cast<const __nv_bfloat16 *>(input),
                                    static_cast<const __nv_bfloat16 *>(bias), static_cast<__nv_bfloat16 *>(output),
                                    batch, units, static_cast<cudaStream_t>(stream));
}

void ref_scale_bf16(const void *input, void *output, float factor, int64_t n, void *stream)
{
  launch_elementwise_mul_scalar<__nv_bfloat16>(static_cast<const __nv_bfloat16 *>(input), factor,
                                               static_cast<__nv_bfloat16 *>(output), n,
                                               static_cast<cudaStream_t>(stream));
}

void ref_fused_adam_f32(float *param, const float *grad, float *m, float *v, float lr, float beta1, float beta2,
                        float epsilon, float weight_decay, float bc1, float bc2, int64_t n, void *stream)
{
  launch_fused_adam<float>(param, grad, m, v, lr, beta1, beta2, epsilon, weight_decay, bc1, bc2, n,
                           static_cast<cudaStream_t>(stream));
}

void ref_fused_adam_bf16(void *param, const void *grad, float *m, float *v, float lr, float beta1, float beta2,
                         float epsilon, float weight_decay, float bc1, float bc2, int64_t n, void *stream)
{
  launch_fused_adam<__nv_bfloat16>(static_cast<__nv_bfloat16 *>(param), static_cast<const __nv_bfloat16 *>(grad), m, v,
                                   lr, beta1, beta2, epsilon, weight_decay, bc1, bc2, n,
                                   static_cast<cudaStream_t>(stream));
}

void ref_sigmoid_f32(const float *in, float *out, int64_t n, void *stream)
{
  launch_sigmoid_forward<float>(in, out, n, static_cast<cudaStream_t>(stream));
}

void ref_sigmoid_bf16(const void *in, void *out, int64_t n, void *stream)
{
  launch_sigmoid_forward<__nv_bfloat16>(static_cast<const __nv_bfloat16 *>(in), static_cast<__nv_bfloat16 *>(out), n,
                                        static_cast<cudaStream_t>(stream));
}

void ref_group_mask_f32(float *sel, int tokens, int experts, int n_group, int topk_group, void *stream)
{
  launch_moe_group_mask<float>(sel, tokens, experts, n_group, topk_group, static_cast<cudaStream_t>(stream));
}

void ref_group_mask_bf16(void *sel, int tokens, int experts, int n_group, int topk_group, void *stream)
{
  launch_moe_group_mask<__nv_bfloat16>(static_cast<__nv_bfloat16 *>(sel), tokens, experts, n_group, topk_group,
                                       static_cast<cudaStream_t>(stream));
}

void ref_gather_topk_f32(const float *scores, const int *indices, float *out, int tokens, int experts, int k,
                         void *stream)
{
  launch_gather_topk_values<float>(scores, indices, out, tokens, experts, k, static_cast<cudaStream_t>(stream));
}

void ref_gather_topk_bf16(const void *scores, const int *indices, void *out, int tokens, int experts, int k,
                          void *stream)
{
  launch_gather_topk_values<__nv_bfloat16>(static_cast<const __nv_bfloat16 *>(scores), indices,
                                           static_cast<__nv_bfloat16 *>(out), tokens, experts, k,
                                           static_cast<cudaStream_t>(stream));
}

void ref_topk_bf16(const void *input, int *indices, void *values, int batch, int dim, int k, void *stream)
{
  launch_topk<__nv_bfloat16>(static_cast<const __nv_bfloat16 *>(input), indices, static_cast<__nv_bfloat16 *>(values),
                             batch, dim, k, static_cast<cudaStream_t>(stream));
}

void ref_router_backward_f32(const float *grad_w, const float *probs, const int *indices, const float *balance_bias,
                             const float *z_lse_scaled, float *grad_topk, float *grad_probs, float *grad_logits,
                             int tokens, int experts, int k, int sigmoid_gate, int normalize, float scaling,
                             void *stream)
{
  router_backward_chain<float>(grad_w, probs, indices, balance_bias, z_lse_scaled, grad_topk, grad_probs, grad_logits,
                               tokens, experts, k, sigmoid_gate, normalize, scaling,
                               static_cast<cudaStream_t>(stream));
}

void ref_router_backward_bf16(const void *grad_w, const void *probs, const int *indices, const void *balance_bias,
                              const void *z_lse_scaled, void *grad_topk, void *grad_probs, void *grad_logits,
                              int tokens, int experts, int k, int sigmoid_gate, int normalize, float scaling,
                              void *stream)
{
  using B = __nv_bfloat16;
  router_backward_chain<B>(static_cast<const B *>(grad_w), static_cast<const B *>(probs), indices,
                           static_cast<const B *>(balance_bias), static_cast<const B *>(z_lse_scaled),
                           static_cast<B *>(grad_topk), static_cast<B *>(grad_probs), static_cast<B *>(grad_logits),
                           tokens, experts, k, sigmoid_gate, normalize, scaling, static_cast<cudaStream_t>(stream));
}

// the pieces of CAIF_DeviceMoELayer::ComputeZLoss / ComputeBalanceLoss (src/caif_device_moe_layer.cpp:853-925)
void ref_logsumexp_f32(const float *input, float *out, int rows, int cols, void *stream)
{
  launch_logsumexp<float>(input, out, rows, cols, static_cast<cudaStream_t>(stream));
}

void ref_logsumexp_bf16(const void *input, float *out, int rows, int cols, void *stream)
{
  launch_logsumexp<__nv_bfloat16>(static_cast<const __nv_bfloat16 *>(input), out, rows, cols,
                                  static_cast<cudaStream_t>(stream));
}

void ref_sum_axis0_f32(const float *input, float *out, int rows, int cols, void *stream)
{
  launch_sum_axis0<float>(input, out, rows, cols, static_cast<cudaStream_t>(stream));
}

void ref_sum_axis0_bf16(const void *input, float *out, int rows, int cols, void *stream)
{
  launch_sum_axis0<__nv_bfloat16>(static_cast<const __nv_bfloat16 *>(input), out, rows, cols,
                                  static_cast<cudaStream_t>(stream));
}

void ref_bias_update_f32(float *bias, const int *counts, int experts, float rate, void *stream)
{
  launch_moe_bias_update<float>(bias, counts, experts, rate, static_cast<cudaStream_t>(stream));
}

void ref_bias_update_bf16(void *bias, const int *counts, int experts, float rate, void *stream)
{
  launch_moe_bias_update<__nv_bfloat16>(static_cast<__nv_bfloat16 *>(bias), counts, experts, rate,
                                        static_cast<cudaStream_t>(stream));
}

void ref_rmsnorm_fwd_f32(const float *x, const float *gamma, float *y, float *rms, float eps, int rows, int dim, void *stream)
{
  launch_rmsnorm_forward<float>(x, gamma, y, rms, eps, rows, dim, static_cast<cudaStream_t>(stream));
}

void ref_rmsnorm_fwd_bf16(const void *x, const float *gamma, void *y, float *rms, float eps, int rows, int dim, void *stream)
{
  launch_rmsnorm_forward<__nv_bfloat16>(static_cast<const __nv_bfloat16 *>(x), gamma, static_cast<__nv_bfloat16 *>(y), rms,
                                        eps, rows, dim, static_cast<cudaStream_t>(stream));
}

void ref_rmsnorm_bwd_f32(const float *dy, const float *x, const float *gamma, const float *rms, float *dx, float *gg,
                         float eps, int rows, int dim, void *stream)
{
  launch_rmsnorm_backward<float>(dy, x, gamma, rms, dx, gg, eps, rows, dim, static_cast<cudaStream_t>(stream));
}

void ref_rmsnorm_bwd_bf16(const void *dy, const void *x, const float *gamma, const float *rms, void *dx, float *gg,
                          float eps, int rows, int dim, void *stream)
{
  launch_rmsnorm_backward<__nv_bfloat16>(static_cast<const __nv_bfloat16 *>(dy), static_cast<const __nv_bfloat16 *>(x),
                                         gamma, rms, static_cast<__nv_bfloat16 *>(dx), gg, eps, rows, dim,
                                         static_cast<cudaStream_t>(stream));
}

}  // extern "C"
