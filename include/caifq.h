/*
 * caifq -- C ABI of the B200-native quantized frozen-linear path.
 *
 * One shared library (libcaifq.so, sm_100a only) replaces the device work
 * behind the reference's CAIF_DeviceFrozenLinear / CAIF_DeviceLoRAAdapter /
 * CAIF_DeviceMoEFrozenExpert / CAIF_DeviceMoELayer hot path.  The reference has
 * no C ABI of its own: each entry point below names the reference function
 * whose device work it takes over (paths are relative to the reference
 * checkout).
 *
 * Conventions
 *   - every data pointer is a DEVICE pointer unless the name ends in _host;
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it
 *     and no entry point synchronises unless it says so;
 *   - return value 0 = success, anything else = failure; the text of the last
 *     failure on the calling thread is available from caifq_last_error();
 *   - dtype codes equal the reference's CAIF_DataType_e
 *     (include/caif/caif_data_type.h:32-48) so a binding can pass them through;
 *   - there is no CPU fallback: without a CUDA device every compute entry
 *     point fails.
 */
#ifndef CAIFQ_H
#define CAIFQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define CAIFQ_API __attribute__((visibility("default")))
#else
#define CAIFQ_API
#endif

#define CAIFQ_OK 0
#define CAIFQ_ERR_INVALID 1  /* bad argument (shape, dtype, null pointer) */
#define CAIFQ_ERR_CUDA 2     /* a CUDA runtime call or launch failed */
#define CAIFQ_ERR_UNSUPPORTED 3

typedef enum caifq_dtype
{
  CAIFQ_F32 = 0,
  CAIFQ_F16 = 2,
  CAIFQ_BF16 = 3,
  CAIFQ_I4 = 4, /* two codes per byte, even flat index in the low nibble */
  CAIFQ_I8 = 5
} caifq_dtype;

/* CAIF_Ops::QuantScheme_e, include/caif/caif_ops.h:365-369 */
typedef enum caifq_scheme
{
  CAIFQ_PER_TENSOR = 0,
  CAIFQ_PER_CHANNEL = 1
} caifq_scheme;

/*
 * A frozen weight exactly as CAIF_DeviceFrozenLinear holds it
 * (src/caif_device_frozen_linear.cpp:126-142, 234-276): `codes` is the flat
 * row-major [out_dim, in_dim] buffer in `storage` dtype; `scales` is
 *   I4: fp16 [ceil(in*out/group_size)], groups over the flat index;
 *   I8: fp32 [1] (per-tensor) or fp32 [out_dim] (per-channel, indexed by
 *       flat index % out_dim), or NULL = plain integer-to-float cast;
 *   float storage: NULL.
 */
typedef struct caifq_weight
{
  const void *codes;
  const void *scales;
  int32_t storage;    /* caifq_dtype */
  int32_t scheme;     /* caifq_scheme, I8 only */
  int32_t group_size; /* I4 only */
  int32_t in_dim;
  int32_t out_dim;
} caifq_weight;

/* LoRA factors as CAIF_DeviceLoRAAdapter holds them
 * (src/caif_device_lora_adapter.cpp:53-60): A [rank, in], B [out, rank]. */
typedef struct caifq_lora
{
  const void *a;
  const void *b;
  int32_t dtype; /* F32, F16 or BF16: dtype of A, B and of every LoRA intermediate */
  int32_t rank;
  float alpha;
} caifq_lora;

CAIFQ_API const char *caifq_last_error(void);
/* 1 when a CUDA device of compute capability 10.x is current, else 0. */
CAIFQ_API int caifq_device_ok(void);
CAIFQ_API const char *caifq_version(void);
/*
 * Waits inside the kernels (on copies, on other warps) are bounded.  A wait that
 * runs out lets its kernel finish with wrong results and raises a flag.  This
 * call synchronises the current device, returns the flags (bit 0: weight-
 * streaming kernel, bit 1: tensor-core kernel; 0 = healthy; -1 = the query
 * itself failed) and clears them.
 */
CAIFQ_API int caifq_device_status(void);
/*
 * Self-test of that give-up path (no counterpart in the reference): the next few-token
 * caifq_linear_fwd / caifq_linear_fwd_gather call of the calling thread is launched with a short
 * wait limit and announces 16 bytes for its first copy that never arrive.  The kernel returns
 * within milliseconds without writing its outputs, the GPU context stays usable, and
 * caifq_device_status() then reports bit 0.  Nothing faults and nothing hangs.
 */
CAIFQ_API void caifq_selftest_stall_next_decode(void);
/* The same for the tensor-core kernel: the next many-token caifq_linear_fwd / caifq_linear_dx call of the
 * calling thread announces 16 bytes for its first activation tile that never arrive.  The kernel returns
 * (its output is garbage), its tensor memory is released, caifq_device_status() reports bit 1. */
CAIFQ_API void caifq_selftest_stall_next_umma(void);
/*
 * The weight-streaming and tensor-core kernels are persistent: one CTA per SM.  A host that runs
 * collectives (NCCL) beside them on another stream caps their grids with this call so that the
 * collective's CTAs find SMs of their own; a persistent CTA that finds its SM taken would wait for
 * the whole collective.  max_ctas <= 0 restores one CTA per SM.  Process-wide; applies to launches
 * made after the call.  (No counterpart in the reference, which is single-device.)
 */
CAIFQ_API void caifq_set_cta_limit(int32_t max_ctas);
/* The tensor-core kernel runs 256-wide tiles on pairs of CTAs (two SMs of one cluster).  Returns how many
 * pairs the current device keeps resident at a time, as reported by the occupancy query of the launches made
 * so far on it (0 before the first such launch).  Diagnostic; no counterpart in the reference. */
CAIFQ_API int32_t caifq_umma_pair_capacity(void);

/* ---- quantize / dequantize (bit-exact with the reference kernels) -------- */

/* launch_quantize_int8_per_tensor, src/caif_cuda_kernels_quant.cu:458-483 */
CAIFQ_API int caifq_quantize_int8_per_tensor(const float *x, int8_t *q, float *scale, int64_t n, void *stream);
/* launch_quantize_int8_per_channel, src/caif_cuda_kernels_quant.cu:576-600 */
CAIFQ_API int caifq_quantize_int8_per_channel(const float *x, int8_t *q, float *scales, int32_t rows, int32_t cols,
                                    void *stream);
/* launch_quantize_to_int4, src/caif_cuda_kernels_quant.cu:344-362 */
CAIFQ_API int caifq_quantize_int4_per_group(const float *x, uint8_t *packed, uint16_t *scales_f16, int64_t n,
                                  int32_t group_size, void *stream);
/* launch_dequantize_int8_per_tensor, src/caif_cuda_kernels_quant.cu:485-500 */
CAIFQ_API int caifq_dequantize_int8_per_tensor(const int8_t *q, float *out, const float *scale, int64_t n, void *stream);
/* launch_dequantize_int8_per_channel, src/caif_cuda_kernels_quant.cu:602-620 */
CAIFQ_API int caifq_dequantize_int8_per_channel(const int8_t *q, float *out, const float *scales, int32_t rows, int32_t cols,
                                      void *stream);
/* launch_dequantize_int4, src/caif_cuda_kernels_quant.cu:239-256 */
CAIFQ_API int caifq_dequantize_int4(const uint8_t *packed, const uint16_t *scales_f16, float *out, int64_t n,
                          int32_t group_size, void *stream);
/* CAIF_DeviceTensor::To between F32/F16/BF16/I8, src/caif_device_tensor.cpp:604-706
 * (kernels src/caif_cuda_kernels_quant.cu:38-199) */
CAIFQ_API int caifq_cast(const void *src, int32_t src_dtype, void *dst, int32_t dst_dtype, int64_t n, void *stream);

/* CAIF_DeviceFrozenLinear::FrozenTensorFP32 / ConvertToComputeDtype,
 * src/caif_device_frozen_linear.cpp:288-378, 759-826: the [out,in] weight in
 * `dst_dtype` (F32/F16/BF16), reduced dtypes by way of fp32 as the reference does. */
CAIFQ_API int caifq_weight_materialize(const caifq_weight *w, void *dst, int32_t dst_dtype, void *stream);

/* ---- frozen linear ------------------------------------------------------- */

/*
 * CAIF_DeviceFrozenLinear::ForwardImpl, src/caif_device_frozen_linear.cpp:381-524.
 *   y[m, out] = x[m, in] . W_deq[out, in]^T, fp32 accumulate.
 * x_dtype in {F32,F16,BF16}; compute_dtype in {F32,F16,BF16} selects the
 * operand precision (the reference's ComputeT); y_dtype F32 (what the reference
 * returns), or F16/BF16 for callers that cast straight after.
 * The weight is dequantized on the fly inside the kernel: no [out,in] float
 * copy is ever written to memory.
 * Few-token calls (m <= 16) are launched with the programmatic-dependent-launch attribute: the
 * kernel starts copying codes and scales as soon as the previous kernel in the stream lets go of
 * the SMs, and waits for that kernel only before it touches x and y.  Codes and scales are frozen:
 * a kernel of another library that writes them must not be the one enqueued directly ahead of this
 * call in the same stream (the first few-token call after one of this library's own quantize calls
 * is a plain launch and needs no care); CAIFQ_PDL=0 turns the attribute off.
 */
CAIFQ_API int caifq_linear_fwd(const caifq_weight *w, const void *x, int32_t x_dtype, int64_t m, void *y, int32_t y_dtype,
                     int32_t compute_dtype, void *stream);

/*
 * CAIF_DeviceFrozenLinear::BackwardImpl, src/caif_device_frozen_linear.cpp:526-660.
 *   dx[m, in] = dy[m, out] . W_deq[out, in], fp32 accumulate.  No weight gradient.
 */
CAIFQ_API int caifq_linear_dx(const caifq_weight *w, const void *dy, int32_t dy_dtype, int64_t m, void *dx, int32_t dx_dtype,
                    int32_t compute_dtype, void *stream);

/*
 * Column-parallel forward with the all-gather of Y fused into the kernel's stores, for layers
 * sharded by output features over the GPUs of one box (the reference itself has no multi-GPU
 * linear; this replaces ForwardImpl followed by an NCCL all-gather of the slices).
 * This rank holds rows [y_col0, y_col0 + w->out_dim) of a wider layer.  Every output element
 * y[t, y_col0 + j] is written into y_peers[r] for r = 0 .. num_peers-1 (row pitch y_ld elements):
 * this GPU's own result buffer and the peers' buffers mapped into this process (CUDA IPC or
 * symmetric memory with peer access enabled).  Plain stores over NVLink, complete when the kernel
 * is; the caller orders the consumers behind all ranks' kernels (stream-ordered barrier or event).
 * Few-token calls only (m <= 16, bf16 x, int4 / per-tensor int8): other calls are refused with
 * CAIFQ_ERR_UNSUPPORTED and should use caifq_linear_fwd plus a collective.
 */
CAIFQ_API int caifq_linear_fwd_gather(const caifq_weight *w, const void *x, int32_t x_dtype, int64_t m,
                                      void *const *y_peers, int32_t num_peers, int64_t y_ld, int64_t y_col0,
                                      int32_t y_dtype, int32_t compute_dtype, void *stream);

/*
 * ForwardImpl followed by the residual Add of the block that owns the layer
 * (CAIF_DevicePreNormBlock::ForwardLoop, src/caif_device_pre_norm_block.cpp:116-124: x = x + sub_out) for the
 * projection that ends a sub-layer (attention's o, the FFN's down): y_inout [m, out] holds the residual
 * stream on entry and, on return, round(round(x . W_deq^T) + residual), both roundings to y_dtype -- the
 * value the reference's cast of the projection output followed by CAIF_Ops::Add gives.  The add runs in the
 * epilogue of the product, so the residual stream is read and written once and no sub_out tensor exists.
 */
CAIFQ_API int caifq_linear_fwd_residual(const caifq_weight *w, const void *x, int32_t x_dtype, int64_t m,
                                        void *y_inout, int32_t y_dtype, int32_t compute_dtype, void *stream);

/*
 * Several frozen linears that share their input, few tokens: the q/k/v projections of an attention
 * block (src/caif_device_multi_head_attention.cpp:544-546) or gate/up of an FFN
 * (src/caif_device_ffn.cpp:324,335), which the reference runs as separate ForwardImpl calls.  One
 * persistent launch streams all the code matrices, so the per-launch latency is paid once:
 *   y[m, sum_i out_i] = x[m, in] . [W_0; W_1; ...]_deq^T      (weight i's outputs at columns sum_{j<i} out_j)
 * Every output element has the bits caifq_linear_fwd gives for its own layer.  1 to 4 weights of one
 * storage (int4 or per-tensor int8), in_dim, scheme and group size, each but the last with a multiple of 8
 * rows; m <= 16, bf16 x.  Other calls are refused with CAIFQ_ERR_UNSUPPORTED (use caifq_linear_fwd per layer).
 */
CAIFQ_API int caifq_linear_fwd_multi(const caifq_weight *ws, int32_t num_weights, const void *x, int32_t x_dtype,
                                     int64_t m, void *y, int32_t y_dtype, int32_t compute_dtype, void *stream);

/* Name of the kernel family the last caifq_linear_fwd / caifq_linear_dx call
 * on this thread chose ("decode", "umma", "generic"); for tests and reports. */
CAIFQ_API const char *caifq_last_path(void);

/* ---- LoRA on a frozen linear --------------------------------------------- */

/*
 * CAIF_DeviceLoRAAdapter::ForwardImpl over a frozen base,
 * src/caif_device_lora_adapter.cpp:119-203:
 *   hidden[m, r] = x . A^T;  y = W-path(x) + (alpha/r) . hidden . B^T
 * x, y, hidden are in lora->dtype.  `hidden` [m, r] is required: it is the
 * tensor the reference caches for backward, and the up-projection reads it.
 * `workspace` (caifq_lora_fwd_workspace_bytes(w, lora, m) bytes, 256-byte
 * aligned; may be NULL) enables the fused path for bf16 adapters of rank
 * 8/16/32/64 on int8/int4 bases: the LoRA product rides in the tensor-core
 * kernel as one extra k-block instead of separate launches.  There the LoRA
 * term is rounded once with the sum (the reference rounds hidden.B^T, its
 * scaling and the sum separately); both stay inside the bf16 tolerance.
 */
CAIFQ_API size_t caifq_lora_fwd_workspace_bytes(const caifq_weight *w, const caifq_lora *lora, int64_t m);
CAIFQ_API int caifq_lora_linear_fwd(const caifq_weight *w, const caifq_lora *lora, const void *x, int64_t m, void *y,
                                    void *hidden, void *workspace, int32_t compute_dtype, void *stream);

/*
 * CAIF_DeviceLoRAAdapter::BackwardImpl, src/caif_device_lora_adapter.cpp:205-281:
 *   g = (alpha/r) dy;  dB = g^T hidden;  dH = g B;  dA = dH^T x;
 *   dx = dy . W_deq + dH . A
 * dA [r,in] and dB [out,r] are OVERWRITTEN (the reference's GEMMs run with
 * beta = 0).  All tensors in lora->dtype.  `workspace` must hold
 * caifq_lora_bwd_workspace_bytes(w, lora, m) bytes of device memory (dH plus
 * the fp32 scratch of the two reductions over tokens).
 */
CAIFQ_API size_t caifq_lora_bwd_workspace_bytes(const caifq_weight *w, const caifq_lora *lora, int64_t m);
CAIFQ_API int caifq_lora_linear_bwd(const caifq_weight *w, const caifq_lora *lora, const void *dy, const void *x,
                          const void *hidden, int64_t m, void *dx, void *d_a, void *d_b, void *workspace,
                          int32_t compute_dtype, void *stream);

/*
 * The same two calls for hosts that can spare a larger workspace (no counterpart in the reference, whose
 * cache_fp32 keeps an fp32 copy of every weight for good).  From a few thousand tokens on (m >= 4096, bf16
 * adapter on an int8 base, or on an int4 base under bf16 compute, in_dim and out_dim multiples of 256) the
 * weight is expanded ONCE per call into a bf16 [out, in] matrix behind the other scratch -- int8 codes as
 * exact integers with the per-tensor scale left to the epilogue, int4 as bf16(scale * code), the value the
 * reference's dequantize-then-cast gives -- and the tensor core is fed from it by plain tile copies on CTA
 * pairs, instead of every CTA converting every weight tile again for each 256 rows of tokens.  Results: int8
 * bit-equal to caifq_lora_linear_fwd / _bwd; int4 the reference's own operand (closer to it than the
 * unexpanded form).  The workspace must hold caifq_lora_*_workspace_bytes_expanded(...) bytes (equal to the
 * plain size for calls that are not expanded), 256-byte aligned.
 */
CAIFQ_API size_t caifq_lora_fwd_workspace_bytes_expanded(const caifq_weight *w, const caifq_lora *lora, int64_t m,
                                                         int32_t compute_dtype);
CAIFQ_API int caifq_lora_linear_fwd_expanded(const caifq_weight *w, const caifq_lora *lora, const void *x, int64_t m,
                                             void *y, void *hidden, void *workspace, int32_t compute_dtype,
                                             void *stream);
CAIFQ_API size_t caifq_lora_bwd_workspace_bytes_expanded(const caifq_weight *w, const caifq_lora *lora, int64_t m,
                                                         int32_t compute_dtype);
CAIFQ_API int caifq_lora_linear_bwd_expanded(const caifq_weight *w, const caifq_lora *lora, const void *dy,
                                             const void *x, const void *hidden, int64_t m, void *dx, void *d_a,
                                             void *d_b, void *workspace, int32_t compute_dtype, void *stream);

/*
 * The optimizer step of the adapter: AdamW with decoupled weight decay on A [rank, in] and B [out, rank] in
 * ONE launch (the reference steps each parameter tensor with its own launch_fused_adam,
 * src/caif_cuda_kernels_optimizers.cu:49-92,217-245).  Same arithmetic in the same order, fp32 math and fp32
 * moments m, v per factor; A, B, dA, dB in `dtype`.  bias_correction1/2 are 1 - beta^t, computed by the
 * caller as the reference's optimizer does.  Results are bit-identical to the reference kernel.  After the
 * step the host calls nothing else: no cached copy of the factors exists in this library.
 */
CAIFQ_API int caifq_lora_adamw_step(void *a, void *b, const void *d_a, const void *d_b, float *m_a, float *v_a,
                                    float *m_b, float *v_b, int32_t rank, int32_t in_dim, int32_t out_dim,
                                    int32_t dtype, float lr, float beta1, float beta2, float epsilon,
                                    float weight_decay, float bias_correction1, float bias_correction2, void *stream);

/*
 * caifq_lora_linear_bwd for callers that cannot hand over a workspace.
 * (No counterpart in the reference: its layers always own their scratch as
 * CAIF_DeviceTensor objects.)
 *
 * Some hosts of this library hold nothing but the pointers they pass in: a
 * plugin loaded into another runtime has no access to that runtime's caching
 * allocator, and a serving or training step that must not stall cannot call
 * cudaMalloc itself, because the driver synchronises the whole device around
 * it.  For them the scratch of the backward pass (dH and the fp32 accumulator
 * of the dA/dB reductions) comes from an 8 MiB buffer built into the library
 * image; each GPU that loads the library holds it until the process exits.
 *
 *   - Same arguments and results as caifq_lora_linear_bwd, minus `workspace`.
 *   - Calls whose scratch need (caifq_lora_bwd_workspace_bytes) exceeds
 *     caifq_lora_bwd_noalloc_max_bytes() are rejected with CAIFQ_ERR_UNSUPPORTED
 *     and a message naming both sizes; nothing is launched.
 *   - No cudaMalloc / cudaFree and no allocating library routine is called.
 *   - The first call on a device looks up the buffer's device address
 *     (cudaGetSymbolAddress, with that device current).  Make that first call
 *     outside any stream capture.
 *   - All calls on a device share the one buffer and find in it whatever the
 *     previous call left; the entry point clears what has to start at zero.
 *     Two calls that can overlap on the GPU (different streams, no dependency)
 *     race on it: serialise them, or use caifq_lora_linear_bwd with separate
 *     workspaces.
 */
CAIFQ_API size_t caifq_lora_bwd_noalloc_max_bytes(void);
CAIFQ_API int caifq_lora_linear_bwd_noalloc(const caifq_weight *w, const caifq_lora *lora, const void *dy,
                                            const void *x, const void *hidden, int64_t m, void *dx, void *d_a,
                                            void *d_b, int32_t compute_dtype, void *stream);

/*
 * Several frozen linears that share their input (q / k / v of an attention block, gate / up of an FFN) as ONE
 * tensor-core product over their weights laid one under the other -- the fusion the reference applies to its
 * own non-projection attention path (CHANGES.md:183-187), here for the frozen projections:
 *   fwd:  y [m, sum out_i] = x . [W_0; W_1; ...]^T     (columns of layer i start at sum_{j<i} out_j)
 *   dx:   dx [m, in] = dy [m, sum out_i] . [W_0; W_1; ...]   one reduction over all layers' features instead of
 *         one launch per layer accumulating into dx
 * Each call first writes the layers' weights into `workspace` as the bf16 matrix the reference's
 * ConvertToComputeDtype holds for bf16 compute (src/caif_device_frozen_linear.cpp:288-378: int4
 * bf16(scale * code), int8 per-tensor bf16(float(code) * scale), floats rounded to bf16), then runs one launch
 * on CTA pairs.  compute_dtype must be CAIFQ_BF16; activations bf16, m >= 32; all layers one in_dim; up to 8
 * layers; workspace >= caifq_linear_concat_workspace_bytes, 256-byte aligned, free again when the call's work
 * on `stream` is done.  Other calls are refused with CAIFQ_ERR_UNSUPPORTED (run the layers one by one, or
 * caifq_linear_fwd_multi for up to 16 rows).
 */
CAIFQ_API size_t caifq_linear_concat_workspace_bytes(const caifq_weight *ws, int32_t count);
CAIFQ_API int caifq_linear_fwd_concat(const caifq_weight *ws, int32_t count, const void *x, int32_t x_dtype,
                                      int64_t m, void *y, int32_t y_dtype, int32_t compute_dtype, void *workspace,
                                      size_t workspace_bytes, void *stream);
CAIFQ_API int caifq_linear_dx_concat(const caifq_weight *ws, int32_t count, const void *dy, int32_t dy_dtype,
                                     int64_t m, void *dx, int32_t dx_dtype, int32_t compute_dtype, void *workspace,
                                     size_t workspace_bytes, void *stream);

/* ---- the norm in front of the frozen projections --------------------------- */

/*
 * RMSNorm as CAIF_DevicePreNormBlock applies it before a frozen linear
 * (src/caif_device_pre_norm_block.cpp:97-135; kernels src/caif_cuda_kernels_normalization.cu:46-119, 129-203):
 *   fwd: rms[r] = sqrt(mean_c x[r,c]^2 + epsilon); y[r,c] = T(x[r,c] / rms[r] * gamma[c]); rms_cache [rows] fp32
 *        (may be NULL when no backward follows)
 *   bwd: dx[r,c] = T(rstd * (dy * gamma - x_hat * mean_c(dy * gamma * x_hat))), x_hat = x * rstd, rstd = 1 / rms;
 *        grad_gamma[c] += sum_r dy[r,c] * x_hat[r,c]  (fp32 [dim], accumulated onto what is there: zero it first,
 *        as the reference does; may be NULL)
 * x, y, dy, dx in `dtype`; gamma, rms_cache, grad_gamma fp32.  y, rms_cache and dx are bit-identical to the
 * reference kernels (same per-thread column order, reduction trees and roundings); grad_gamma is a sum over
 * rows whose order the reference leaves to its atomics and agrees to rounding.  Rows up to 96 KB (forward) /
 * 8192 elements (backward).  In place (y == x, dx == dy) is allowed.
 */
CAIFQ_API int caifq_rmsnorm_fwd(const void *x, const float *gamma, void *y, float *rms_cache, float epsilon,
                                int32_t dtype, int32_t rows, int32_t dim, void *stream);
CAIFQ_API int caifq_rmsnorm_bwd(const void *dy, const void *x, const float *gamma, const float *rms_cache, void *dx,
                                float *grad_gamma, int32_t dtype, int32_t rows, int32_t dim, void *stream);

/* ---- MoE routing and dispatch -------------------------------------------- */

/* launch_topk, src/caif_cuda_kernels_moe.cu:280-345: descending values, ties to
 * the lowest index; `dtype` is the dtype of probs and values. */
CAIFQ_API int caifq_moe_topk(const void *probs, int32_t dtype, int32_t *indices, void *values, int32_t batch, int32_t dim,
                   int32_t k, void *stream);
/* launch_normalize_rows, src/caif_cuda_kernels_moe.cu:43-97 */
CAIFQ_API int caifq_moe_normalize_rows(const void *input, void *output, int32_t dtype, int32_t batch, int32_t dim,
                             void *stream);
/*
 * The score function of CAIF_DeviceMoERouter::Route for SoftmaxTopK gating,
 * src/caif_device_moe_router.cpp:233-303: probs = softmax(logits [+ bias]) over the experts of each
 * row, with the operation order of launch_attention_softmax
 * (src/caif_cuda_kernels_attention_support.cu:350-460, 866-884) so that the probabilities, and with
 * them the top-k indices, come out bit-identical.  `bias` [cols] may be NULL; when given it is added
 * first and the sum rounded to `dtype`, as the reference's separate AddBias kernel stores it
 * (src/caif_cuda_kernels_elementwise.cu:124-137).  In place (probs == logits) is allowed.
 */
CAIFQ_API int caifq_moe_router_softmax(const void *logits, const void *bias, void *probs, int32_t dtype, int32_t rows,
                             int32_t cols, void *stream);

/*
 * CAIF_DeviceMoERouter::Route for SigmoidNoauxTc gating and for DeepSeek group-limited routing
 * (src/caif_device_moe_router.cpp:286-376) in one launch instead of the reference's Sigmoid, AddBias,
 * MoEGroupMask, TopK and GatherTopKValues kernels:
 *   scores    = sigmoid(input) when input_is_logits != 0 (launch_sigmoid_forward), else input as given
 *               (softmax probabilities from caifq_moe_router_softmax); written to scores_out when non-NULL
 *   selection = scores (+ selection_bias [dim], may be NULL: the aux-loss-free bias, for selection only)
 *   n_group > 1: the experts of a token form n_group equal groups scored by the sum of their two largest
 *               selection entries; all but the topk_group best groups are masked (launch_moe_group_mask)
 *   indices   = top-k of the selection (largest first, ties to the lowest index)
 *   weights   = the ORIGINAL scores at the chosen experts when a bias was given (launch_gather_topk_values),
 *               else the selection values themselves
 * Bit-identical to the reference kernels.  The caller applies norm_topk_prob and routed_scaling_factor with
 * caifq_moe_normalize_rows and caifq_scale, as the router does.  At most 32 groups.
 */
CAIFQ_API int caifq_moe_route_grouped(const void *input, int32_t input_is_logits, const void *selection_bias,
                                      void *scores_out, int32_t *indices, void *weights, int32_t dtype, int32_t batch,
                                      int32_t dim, int32_t k, int32_t n_group, int32_t topk_group, void *stream);
/*
 * CAIF_DeviceMoERouter::BackwardRoutingAuxAware up to grad_logits (src/caif_device_moe_router.cpp:529-733) in
 * one launch instead of NormalizeRowsBackwardTopKGather, Scale, Zeros, ScatterAdd, AddBias, SoftmaxBackward
 * and MoEZLossGradAdd (SigmoidBackward for sigmoid gating), bit-identical to that chain:
 *   grad_topk   = normalize != 0 ? (grad_weights - dot(w, grad_weights)) / s : grad_weights, with
 *                 p = probs at the chosen experts, s = max(sum p, 1e-12), w = p / s
 *                 (src/caif_cuda_kernels_moe.cu:128-171); then * routed_scaling_factor when it is not 1.
 *                 Written to grad_topk [tokens, top_k] when non-NULL (the router's GradTopkPreview).
 *   grad_probs  = scatter of grad_topk to [tokens, experts] (+ balance_bias [experts] per column, may be NULL)
 *   sigmoid_gate != 0: grad_logits = grad_probs * probs * (1 - probs); balance_bias and z_lse_scaled must be
 *                 NULL (the reference refuses them for SigmoidNoauxTc).
 *   else        grad_logits = softmax backward of grad_probs (+ z_lse_scaled[t] * probs, may be NULL).
 * exact_jacobian selects how the softmax backward is evaluated.  The reference calls
 * SoftmaxBackward(CachedProbs(), grad_probs, grad_logits) (src/caif_device_moe_router.cpp:702) against the
 * signature (grad_output, output, grad_input) (include/caif/caif_ops.h:650), so its kernel computes
 * grad_probs * (probs - dot(probs, grad_probs)); 0 reproduces that bit for bit, 1 computes
 * probs * (grad_probs - dot(probs, grad_probs)).  The two linear-layer products that follow in the reference
 * (grad_w_router += x^T grad_logits, grad_input = grad_logits w_router^T) are caifq_linear_* calls of the host.
 * top_k <= 32.  indices are int32, [tokens, top_k]; entries outside [0, experts) are skipped.
 */
CAIFQ_API int caifq_moe_router_bwd(const void *grad_weights, const void *probs, const int32_t *indices,
                                   const void *balance_bias, const void *z_lse_scaled, void *grad_topk,
                                   void *grad_logits, int32_t dtype, int32_t tokens, int32_t experts, int32_t top_k,
                                   int32_t sigmoid_gate, int32_t normalize, float routed_scaling_factor,
                                   int32_t exact_jacobian, void *stream);
/*
 * CAIF_Ops::MoEBiasUpdate (src/caif_ops_device.cpp:4644-4672, launch_moe_bias_update,
 * src/caif_cuda_kernels_moe.cu:481-537), the aux-loss-free balancing step of SigmoidNoauxTc routers
 * (src/caif_device_moe_router.cpp:942): bias[e] += rate where the expert's load is under the mean load,
 * -= rate where over, in place, rounded to `dtype`.  counts is device int32 [experts], or the
 * [experts + 1] offsets caifq_moe_build_dispatch wrote when from_offsets != 0.  Bit-identical.
 */
CAIFQ_API int caifq_moe_bias_update(void *bias, const int32_t *counts, int32_t from_offsets, int32_t dtype,
                                    int32_t experts, float rate, void *stream);
/*
 * The auxiliary losses of CAIF_DeviceMoELayer and the operands their gradients enter the router backward
 * with (src/caif_device_moe_layer.cpp:792-835 and 853-925), on the device, with no host round trip:
 *   sums[0] = balance_weight * experts * sum_e (count_e / (tokens * top_k)) * (sum_t probs[t, e] / tokens)
 *   sums[1] = z_weight * sum_t lse_t^2 / tokens,  lse_t = logsumexp(logits[t, :]) rounded to `dtype`
 *   sums[2 + e] = sum_t probs[t, e]                              (sums: device float [2 + experts])
 *   balance_bias[e] = balance_weight * experts / (tokens^2 * top_k) * count_e     ([experts], may be NULL)
 *   lse[t], z_lse_scaled[t] = lse_t, lse_t * 2 * z_weight / tokens               ([tokens], may be NULL)
 * count_e = expert_offsets[e + 1] - expert_offsets[e] (the offsets caifq_moe_build_dispatch wrote).
 * logits may be NULL (no z-loss: sums[1] = 0) and probs may be NULL (no balance loss: sums[0] = 0).
 * lse, z_lse_scaled and balance_bias are bit-identical to the reference's tensors (its logsumexp tree order,
 * src/caif_cuda_kernels_elementwise.cu:930-990); the two loss values add their terms in another order
 * than the reference's sequential column sums and agree to rounding.  One deliberate difference: the reference
 * sums the squared logsumexp with launch_reduction_sum, whose kernel stores one partial per 256-element block
 * (src/caif_cuda_kernels_elementwise.cu:450-493) into a one-element tensor (src/caif_device_moe_layer.cpp:911-913),
 * so beyond 256 tokens its z loss holds the first block's partial only (and the other partials land past the
 * tensor); sums[1] here is the sum over all tokens.  The z-loss GRADIENT operand is unaffected in both.
 */
CAIFQ_API int caifq_moe_aux_losses(const void *logits, const void *probs, const int32_t *expert_offsets,
                                   void *balance_bias, void *lse, void *z_lse_scaled, float *sums, int32_t dtype,
                                   int32_t tokens, int32_t experts, int32_t top_k, float balance_weight,
                                   float z_weight, void *stream);
/* CAIF_Ops::Scale, src/caif_ops_device.cpp:3142-3160 (the router's routed_scaling_factor on the top-k
 * weights, src/caif_device_moe_router.cpp:394-407; LoRA's alpha/r): dst = T(float(src) * factor).
 * In place is allowed. */
CAIFQ_API int caifq_scale(const void *src, void *dst, int32_t dtype, float factor, int64_t n, void *stream);
/*
 * CAIF_Ops::MoEBuildDispatchMap, src/caif_ops_device.cpp:4876-4950, computed on
 * the device with the identical result: expert_offsets[E+1] (exclusive prefix
 * sum of the capacity-clamped counts) and dispatch_map[T,k] (arrival order
 * within the expert scanning tokens then k; -1 = dropped).  The total assigned
 * is expert_offsets[E]; no host copy is made.  capacity 0 = unlimited.
 */
CAIFQ_API int caifq_moe_build_dispatch(const int32_t *expert_indices, int32_t num_tokens, int32_t top_k, int32_t num_experts,
                             int32_t capacity, int32_t *dispatch_map, int32_t *expert_offsets, void *stream);
/* launch_moe_dispatch, src/caif_cuda_kernels_moe.cu:616-680 */
CAIFQ_API int caifq_moe_dispatch(const void *input, int32_t dtype, const int32_t *expert_indices, const int32_t *dispatch_map,
                       const int32_t *expert_offsets, void *expert_buffer, int32_t num_tokens, int32_t dim,
                       int32_t top_k, void *stream);
/* launch_moe_combine, src/caif_cuda_kernels_moe.cu:705-790 */
CAIFQ_API int caifq_moe_combine(const void *expert_buffer, int32_t dtype, const int32_t *expert_indices,
                      const void *expert_weights, const int32_t *dispatch_map, const int32_t *expert_offsets,
                      void *output, int32_t num_tokens, int32_t dim, int32_t top_k, void *stream);

/* launch_moe_combine_backward_grad_expert, src/caif_cuda_kernels_moe.cu:816-875:
 * grad_expert_buffer[slot(t,k), :] = w[t,k] * grad_output[t, :] for every assigned (t,k);
 * other rows of the buffer are left as they are. */
CAIFQ_API int caifq_moe_combine_bwd_grad_expert(const void *grad_output, int32_t dtype, const int32_t *expert_indices,
                      const void *expert_weights, const int32_t *dispatch_map, const int32_t *expert_offsets,
                      void *grad_expert_buffer, int32_t num_tokens, int32_t dim, int32_t top_k, void *stream);
/* launch_moe_combine_backward_grad_weights, src/caif_cuda_kernels_moe.cu:925-990:
 * grad_weights[t,k] = <grad_output[t,:], expert_buffer[slot(t,k),:]> (0 for dropped picks), summed in
 * the reference's order (256 strided partial sums, halving tree). */
CAIFQ_API int caifq_moe_combine_bwd_grad_weights(const void *grad_output, const void *expert_buffer, int32_t dtype,
                      const int32_t *expert_indices, const int32_t *dispatch_map, const int32_t *expert_offsets,
                      void *grad_weights, int32_t num_tokens, int32_t dim, int32_t top_k, void *stream);
/* launch_moe_dispatch_backward, src/caif_cuda_kernels_moe.cu:1040-1085:
 * grad_input[t, :] = sum over k, in order, of grad_expert_buffer[slot(t,k), :]. */
CAIFQ_API int caifq_moe_dispatch_bwd(const void *grad_expert_buffer, int32_t dtype, const int32_t *expert_indices,
                      const int32_t *dispatch_map, const int32_t *expert_offsets, void *grad_input,
                      int32_t num_tokens, int32_t dim, int32_t top_k, void *stream);

/* ---- grouped frozen experts ---------------------------------------------- */

/*
 * The per-expert loop of CAIF_DeviceMoELayer::ForwardImpl over
 * CAIF_DeviceMoEFrozenExpert::ForwardInto (src/caif_device_moe_layer.cpp:534-557,
 * src/caif_device_moe_frozen_expert.cpp:91-229) as ONE grouped call:
 * for every expert e, rows [offsets[e], offsets[e+1]) of the packed buffer go
 * through  down_e( silu(gate_e(x)) * up_e(x) ).
 * gate/up/down are arrays of num_experts weights (host array of structs whose
 * pointers are device pointers).  gate == NULL selects experts without a gate
 * projection (the reference's UseGated() == false, :158-162, 318-331):
 * down_e( silu(up_e(x)) ); gate_out is then unused and may be NULL.  x, out, and the saved gate_out / up_out
 * (each [total, hidden], may be NULL when not training) are in `dtype`.
 * expert_offsets_host is the host copy of the offsets (E+1 ints).
 */
CAIFQ_API int caifq_grouped_expert_fwd(const caifq_weight *gate, const caifq_weight *up, const caifq_weight *down,
                             int32_t num_experts, const int32_t *expert_offsets_host, const void *x, void *out,
                             void *gate_out, void *up_out, void *hidden_ws, int32_t dtype, int32_t compute_dtype,
                             void *stream);
/* Backward of the same loop (src/caif_device_moe_layer.cpp:754-778,
 * src/caif_device_moe_frozen_expert.cpp:232-332): dX only.
 * ws must hold 3 * total * hidden elements of `dtype`. */
CAIFQ_API int caifq_grouped_expert_bwd(const caifq_weight *gate, const caifq_weight *up, const caifq_weight *down,
                             int32_t num_experts, const int32_t *expert_offsets_host, const void *dy,
                             const void *gate_out, const void *up_out, void *dx, void *ws, int32_t dtype,
                             int32_t compute_dtype, void *stream);

/*
 * The same two calls on bf16 copies of the experts' weights that the host expands once per step (no
 * counterpart in the reference, whose cache_fp32 keeps fp32 copies of every expert for good: 2.2 GB for the
 * 64 experts of the MoE config, against 1.1 GB of scratch here that the host may reuse for anything else
 * between steps).  With quantized experts of one shape on bf16 rows (int8, or int4 under bf16 compute; in and
 * hidden multiples of 128):
 *   caifq_grouped_expert_expanded_bytes   size of the scratch, 0 when these experts are not expanded
 *   caifq_grouped_expert_expand           one launch per projection writes all experts' matrices, stacked, as
 *                                         bf16: int8 codes as exact integers (scale left to the epilogue), int4
 *                                         as bf16(scale * code), the reference's dequantize-then-cast value
 *   caifq_grouped_expert_fwd_expanded /   the grouped launches read their weight tiles from the copies with
 *   caifq_grouped_expert_bwd_expanded     plain tile copies (on CTA pairs where the width allows) instead of
 *                                         converting every tile in every CTA; `expanded` is the buffer that
 *                                         caifq_grouped_expert_expand filled for the same tables.  With
 *                                         expanded == NULL, or experts that are not expanded, they are the
 *                                         plain calls.
 * Results: int8 bit-equal to the plain calls; int4 the reference's own operand values.
 */
CAIFQ_API size_t caifq_grouped_expert_expanded_bytes(const caifq_weight *gate, const caifq_weight *up,
                                                     const caifq_weight *down, int32_t num_experts, int32_t dtype,
                                                     int32_t compute_dtype);
CAIFQ_API int caifq_grouped_expert_expand(const caifq_weight *gate, const caifq_weight *up, const caifq_weight *down,
                                          int32_t num_experts, void *expanded, int32_t dtype, int32_t compute_dtype,
                                          void *stream);
CAIFQ_API int caifq_grouped_expert_fwd_expanded(const caifq_weight *gate, const caifq_weight *up,
                                                const caifq_weight *down, int32_t num_experts,
                                                const int32_t *expert_offsets_host, const void *x, void *out,
                                                void *gate_out, void *up_out, void *hidden_ws, const void *expanded,
                                                int32_t dtype, int32_t compute_dtype, void *stream);
CAIFQ_API int caifq_grouped_expert_bwd_expanded(const caifq_weight *gate, const caifq_weight *up,
                                                const caifq_weight *down, int32_t num_experts,
                                                const int32_t *expert_offsets_host, const void *dy,
                                                const void *gate_out, const void *up_out, void *dx, void *ws,
                                                const void *expanded, int32_t dtype, int32_t compute_dtype,
                                                void *stream);

/* ---- sharded over the GPUs of one box ------------------------------------- */
/*
 * The reference is single-device; these entry points have no counterpart in it.  They run the
 * entry point named in each comment and enqueue the NCCL collective a sharded layer needs behind it
 * on the same stream.  `nccl_comm` is the host's ncclComm_t (passed as void*); NCCL is not linked into
 * the library: its functions are looked up among the libraries loaded into the process (the host's
 * own NCCL), then in libnccl.so.2.  One process per GPU; every rank of the communicator makes the
 * same call.  No kernel of the library reads peer memory here: remote data lands in local buffers
 * through the collective.
 */

/* Column-parallel forward: this rank holds output features [r*out/N, (r+1)*out/N) (a contiguous
 * slice of codes and scales, w_shard->out_dim = out/N).  caifq_linear_fwd into y_local [m, out/N],
 * then ncclAllGather into y_gathered [N, m, out/N] (rank r's slice at index r). */
CAIFQ_API int caifq_linear_fwd_sharded(const caifq_weight *w_shard, const void *x, int32_t x_dtype, int64_t m,
                             void *y_local, void *y_gathered, int32_t y_dtype, int32_t compute_dtype,
                             void *nccl_comm, void *stream);
/* Column-parallel dX: caifq_linear_dx on this rank's slice of dY [m, out/N] gives a partial sum
 * dx_partial [m, in]; reduce_scatter != 0: ncclReduceScatter into dx_out [m/N, in] (rank r keeps rows
 * [r*m/N, (r+1)*m/N)); reduce_scatter == 0: ncclAllReduce into dx_out [m, in] (may equal dx_partial). */
CAIFQ_API int caifq_linear_dx_sharded(const caifq_weight *w_shard, const void *dy_local, int32_t dy_dtype, int64_t m,
                            void *dx_partial, void *dx_out, int32_t reduce_scatter, int32_t dx_dtype,
                            int32_t compute_dtype, void *nccl_comm, void *stream);
/* The exchange of expert-parallel frozen experts: rows of `row_bytes` bytes, send_rows_host[r] of them
 * for rank r lying back to back in `send` (rank order), recv_rows_host[r] arriving from rank r back to
 * back in `recv`: an all-to-all with per-pair counts as one group of ncclSend / ncclRecv; a rank's own
 * rows are copied.  With the packed buffer of caifq_moe_dispatch (ordered by expert, experts owned in
 * rank order) this delivers every row to its expert's owner; the mirror call returns the results. */
CAIFQ_API int caifq_rows_all_to_all(const void *send, const int64_t *send_rows_host, void *recv,
                          const int64_t *recv_rows_host, int64_t row_bytes, void *nccl_comm, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* CAIFQ_H */
