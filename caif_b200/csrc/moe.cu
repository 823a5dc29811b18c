// Routing, dispatch and expert elementwise kernels of the frozen-MoE path.
//
// Integer results (top-k indices, dispatch map, offsets) are bit-identical to
// the reference (src/caif_cuda_kernels_moe.cu:280-334 top-k,
// src/caif_ops_device.cpp:4876-4950 dispatch map); float results follow the
// same fp32 operation order per element (normalize :43-85, combine :705-745,
// SiLU src/caif_cuda_kernels_activations.cu:499-566).
#include "common.cuh"

namespace caifq
{

namespace
{

constexpr float kNegSentinel = -1e30f;
constexpr float kRowSumEps = 1e-10f;

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f<__half>(float v) { return __float2half(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

// ------------------------------------------------------------------------ top-k
// One warp per row.  The reference lets thread 0 scan the row k times with a
// strict '>' from index 0 against a -1e30 sentinel: the winner of each round is
// the largest value, lowest index among equals, and (-1e30, index 0) when
// nothing exceeds the sentinel.  The warp version keeps exactly that order.
template <typename T>
__global__ void topk_kernel(const T *__restrict__ input, int *__restrict__ indices, T *__restrict__ values,
                            int batch, int dim, int k)
{
  extern __shared__ float s_rows[];
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * warps_per_block + warp;
  if (row >= batch)
  {
    return;
  }
  float *temp = s_rows + static_cast<size_t>(warp) * dim;
  const T *src = input + static_cast<size_t>(row) * dim;
  for (int d = lane; d < dim; d += 32)
  {
    temp[d] = to_f<T>(src[d]);
  }
  __syncwarp();
  for (int i = 0; i < k; ++i)
  {
    float best = kNegSentinel;
    int best_idx = 0;
    for (int d = lane; d < dim; d += 32)
    {
      const float v = temp[d];
      if (v > best)
      {
        best = v;
        best_idx = d;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
    {
      const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
      const int oi = __shfl_xor_sync(0xFFFFFFFFu, best_idx, o);
      if (ov > best || (ov == best && oi < best_idx))
      {
        best = ov;
        best_idx = oi;
      }
    }
    if (lane == 0)
    {
      indices[static_cast<size_t>(row) * k + i] = best_idx;
      values[static_cast<size_t>(row) * k + i] = from_f<T>(best);
      temp[best_idx] = kNegSentinel;
    }
    __syncwarp();
  }
}

// ------------------------------------------- sigmoid / group-limited top-k routing
// CAIF_DeviceMoERouter::Route for SigmoidNoauxTc gating and for group-limited routing
// (src/caif_device_moe_router.cpp:286-376): scores = sigmoid(logits) (or the probabilities given), a per-token
// selection copy with the selection-only bias added (bias_add_2d: T(float + float)), the DeepSeek group mask
// (moe_group_mask_kernel: a group's score is the sum of its two largest entries, the topk_group best groups
// stay, ties to the lowest group, everything else becomes T(-1e30)), top-k on the selection with the
// reference's order, and combine weights gathered from the ORIGINAL scores when a bias was used.  The
// reference runs five kernels with thread 0 of a block doing the scans; here one warp does a token in one
// pass with the same comparisons in the same order, so indices and weights are bit-identical.
template <typename T>
__global__ void route_grouped_kernel(const T *__restrict__ input, const T *__restrict__ bias, T *__restrict__ scores_out,
                                     int *__restrict__ indices, T *__restrict__ weights, int batch, int dim, int k,
                                     int n_group, int topk_group, int apply_sigmoid)
{
  extern __shared__ float s_route[];
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * warps_per_block + warp;
  if (row >= batch)
  {
    return;
  }
  float *sel = s_route + static_cast<size_t>(warp) * (2 * dim + 64);   // selection scores
  float *orig = sel + dim;                                              // original scores
  float *grp = orig + dim;                                              // group scores, then keep flags
  float *keep = grp + 32;
  const T *src = input + static_cast<size_t>(row) * dim;
  for (int d = lane; d < dim; d += 32)
  {
    T score = src[d];
    if (apply_sigmoid)
    {
      const float x = to_f<T>(src[d]);
      score = from_f<T>(1.0f / (1.0f + expf(-x)));
    }
    if (scores_out != nullptr)
    {
      scores_out[static_cast<size_t>(row) * dim + d] = score;
    }
    const float sf = to_f<T>(score);
    orig[d] = sf;
    sel[d] = (bias != nullptr) ? to_f<T>(from_f<T>(sf + to_f<T>(bias[d]))) : sf;
  }
  __syncwarp();
  if (n_group > 1)
  {
    const int per_group = dim / n_group;
    // lane g scores group g: the two largest entries in the reference's scan order
    for (int g0 = 0; g0 < n_group; g0 += 32)
    {
      const int g = g0 + lane;
      if (g < n_group)
      {
        float top1 = kNegSentinel;
        float top2 = kNegSentinel;
        for (int j = 0; j < per_group; ++j)
        {
          const float v = sel[g * per_group + j];
          if (v > top1)
          {
            top2 = top1;
            top1 = v;
          }
          else if (v > top2)
          {
            top2 = v;
          }
        }
        grp[g] = top1 + top2;
        keep[g] = 0.0f;
      }
    }
    __syncwarp();
    for (int r = 0; r < topk_group; ++r)
    {
      // the first strictly largest group score from group 0 upwards; (sentinel, group 0) when none exceeds it
      float best = kNegSentinel;
      int best_g = 0;
      for (int g = lane; g < n_group; g += 32)
      {
        if (grp[g] > best)
        {
          best = grp[g];
          best_g = g;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
      {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const int og = __shfl_xor_sync(0xFFFFFFFFu, best_g, o);
        if (ov > best || (ov == best && og < best_g))
        {
          best = ov;
          best_g = og;
        }
      }
      if (lane == 0)
      {
        keep[best_g] = 1.0f;
        grp[best_g] = kNegSentinel;
      }
      __syncwarp();
    }
    const float masked = to_f<T>(from_f<T>(kNegSentinel));
    for (int d = lane; d < dim; d += 32)
    {
      if (keep[d / per_group] == 0.0f)
      {
        sel[d] = masked;
      }
    }
    __syncwarp();
  }
  for (int i = 0; i < k; ++i)
  {
    float best = kNegSentinel;
    int best_idx = 0;
    for (int d = lane; d < dim; d += 32)
    {
      const float v = sel[d];
      if (v > best)
      {
        best = v;
        best_idx = d;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
    {
      const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
      const int oi = __shfl_xor_sync(0xFFFFFFFFu, best_idx, o);
      if (ov > best || (ov == best && oi < best_idx))
      {
        best = ov;
        best_idx = oi;
      }
    }
    if (lane == 0)
    {
      indices[static_cast<size_t>(row) * k + i] = best_idx;
      // with a selection-only bias the combine weight is the original score at the chosen expert
      weights[static_cast<size_t>(row) * k + i] = (bias != nullptr) ? from_f<T>(orig[best_idx]) : from_f<T>(best);
      sel[best_idx] = kNegSentinel;
    }
    __syncwarp();
  }
}

// -------------------------------------------------------------- normalize rows
// The reference uses a block of 256 threads: thread t sums elements t, t+256,
// ... and a shared-memory tree (stride 128..1) adds the 256 partials.  A warp
// reproduces that order: lane l owns partials l, l+32, ..., l+224.
template <typename T>
__global__ void normalize_rows_kernel(const T *__restrict__ input, T *__restrict__ output, int batch, int dim)
{
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (row >= batch)
  {
    return;
  }
  const T *src = input + static_cast<size_t>(row) * dim;
  T *dst = output + static_cast<size_t>(row) * dim;
  float part[8];
#pragma unroll
  for (int j = 0; j < 8; ++j)
  {
    float acc = 0.0f;
    for (int d = lane + 32 * j; d < dim; d += 256)
    {
      acc += to_f<T>(src[d]);
    }
    part[j] = acc;
  }
  // strides 128, 64, 32 stay inside the lane
  part[0] += part[4];
  part[1] += part[5];
  part[2] += part[6];
  part[3] += part[7];
  part[0] += part[2];
  part[1] += part[3];
  float v = part[0] + part[1];
  // strides 16..1 cross lanes: slot t takes slot t+stride
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
  {
    const float other = __shfl_down_sync(0xFFFFFFFFu, v, o);
    if (lane < o)
    {
      v += other;
    }
  }
  v = __shfl_sync(0xFFFFFFFFu, v, 0);
  const float sum = fmaxf(v, kRowSumEps);
  const float inv = __fdiv_rn(1.0f, sum);
  for (int d = lane; d < dim; d += 32)
  {
    dst[d] = from_f<T>(__fmul_rn(to_f<T>(src[d]), inv));
  }
}

// ---------------------------------------------------------------- router softmax
// CAIF_DeviceMoERouter::Route turns logits into probabilities with the attention softmax kernel
// (src/caif_cuda_kernels_attention_support.cu:350-460) after an optional AddBias
// (src/caif_cuda_kernels_elementwise.cu:124-137, which stores T(float(x) + float(bias))).  The routing
// indices depend on the exact probabilities, so the order of every operation is kept: the reference
// runs 128 threads per row, thread t scanning columns t, t+128, ... with the online (max, sum)
// update, then an xor butterfly inside each warp, then the four warp results combined in lanes 0-3
// with offsets 2 and 1.  Here one warp owns a row: lane l plays threads l, l+32, l+64, l+96 (one
// per warp of the reference), runs the same butterfly on each of the four values, and combines them
// in the reference's order.  Far fewer idle threads for rows of 64-256 experts, identical bits.
__device__ __forceinline__ void softmax_absorb(float &m, float &s, float m_other, float s_other)
{
  if (m_other > m)
  {
    s = s * expf(m - m_other) + s_other;
    m = m_other;
  }
  else
  {
    s += s_other * expf(m_other - m);
  }
}

template <typename T>
__global__ void router_softmax_kernel(const T *__restrict__ logits, const T *__restrict__ bias,
                                      T *__restrict__ probs, int rows, int cols)
{
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (row >= rows)
  {
    return;
  }
  const T *x = logits + static_cast<size_t>(row) * cols;
  T *y = probs + static_cast<size_t>(row) * cols;
  // the value the softmax sees: the logit, or the biased logit rounded to T as the separate
  // AddBias kernel would have stored it
  auto value = [&](int col) -> float
  {
    float v = to_f<T>(x[col]);
    if (bias != nullptr)
    {
      v = to_f<T>(from_f<T>(v + to_f<T>(bias[col])));
    }
    return v;
  };
  float m[4];
  float sum[4];
#pragma unroll
  for (int w = 0; w < 4; ++w)
  {
    // thread 32 w + lane of the reference's 128-thread block
    m[w] = kNegSentinel;
    sum[w] = 0.0f;
    for (int col = 32 * w + lane; col < cols; col += 128)
    {
      const float v = value(col);
      if (v > m[w])
      {
        sum[w] = sum[w] * expf(m[w] - v) + 1.0f;
        m[w] = v;
      }
      else
      {
        sum[w] += expf(v - m[w]);
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
    {
      const float m_other = __shfl_xor_sync(0xFFFFFFFFu, m[w], off);
      const float s_other = __shfl_xor_sync(0xFFFFFFFFu, sum[w], off);
      softmax_absorb(m[w], sum[w], m_other, s_other);
    }
  }
  // lanes 0..3 of the reference's warp 0 hold the four warp results; lane 0 ends with
  // absorb(absorb(v0, v2), absorb(v1, v3))
  softmax_absorb(m[0], sum[0], m[2], sum[2]);
  softmax_absorb(m[1], sum[1], m[3], sum[3]);
  softmax_absorb(m[0], sum[0], m[1], sum[1]);
  const float row_max = m[0];
  const float inv_sum = __fdiv_rn(1.0f, sum[0]);
  for (int col = lane; col < cols; col += 32)
  {
    y[col] = from_f<T>(__fmul_rn(expf(value(col) - row_max), inv_sum));
  }
}

// --------------------------------------------------------------- router backward
// CAIF_DeviceMoERouter::BackwardRoutingAuxAware (src/caif_device_moe_router.cpp:529-733) reaches
// grad_logits through up to seven launches, each rounding to the storage type: the normalize Jacobian
// over the chosen scores (src/caif_cuda_kernels_moe.cu:128-171), Scale by routed_scaling_factor, Zeros +
// ScatterAdd into [tokens, experts] (:553-572), AddBias of the load-balance column term, the softmax
// Jacobian (src/caif_cuda_kernels_attention_support.cu:464-530) and the z-loss term (_moe.cu:1376-1395);
// sigmoid gating ends with SigmoidBackward (src/caif_cuda_kernels_activations.cu:189-228) instead.  Here
// one warp owns a token and does all of it with the row of grad_probs in shared memory.  Every
// intermediate is rounded to T where the reference stores it, and every reduction adds in the reference's
// order (an xor butterfly over 32 lanes for the top-k sums; for the softmax dot 128 threads striding the
// row with fused multiply-adds, a butterfly per warp and (w0 + w2) + (w1 + w3) across the four warps), so
// the result has the reference's bits.
//
// The reference calls SoftmaxBackward(probs, grad_probs, grad_logits): the cached probabilities sit in
// the kernel's grad_output slot and grad_probs in its output slot, which evaluates
// grad_probs * (probs - dot) rather than probs * (grad_probs - dot).  `exact_jacobian` == 0 keeps that
// evaluation (parity with the reference); 1 gives the softmax Jacobian itself.
constexpr float kTopkSumEps = 1e-12f;

template <typename T>
__global__ void router_bwd_kernel(const T *__restrict__ grad_w, const T *__restrict__ probs,
                                  const int *__restrict__ indices, const T *__restrict__ balance_bias,
                                  const T *__restrict__ z_lse_scaled, T *__restrict__ grad_topk,
                                  T *__restrict__ grad_logits, int tokens, int experts, int top_k, int sigmoid_gate,
                                  int normalize, float scaling, int exact_jacobian)
{
  extern __shared__ float rb_rows[];
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int t = blockIdx.x * warps_per_block + warp;
  if (t >= tokens)
  {
    return;
  }
  float *gp = rb_rows + static_cast<size_t>(warp) * experts;
  const T *p_row = probs + static_cast<size_t>(t) * experts;
  for (int c = lane; c < experts; c += 32)
  {
    gp[c] = 0.0f;
  }
  int idx = -1;
  float p_k = 0.0f;
  float g_k = 0.0f;
  if (lane < top_k)
  {
    idx = indices[static_cast<size_t>(t) * top_k + lane];
    g_k = to_f<T>(grad_w[static_cast<size_t>(t) * top_k + lane]);
    if (idx >= 0 && idx < experts)
    {
      p_k = to_f<T>(p_row[idx]);
    }
  }
  float gt = g_k;
  if (normalize != 0)
  {
    float sum = p_k;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
    {
      sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
    }
    sum = fmaxf(sum, kTopkSumEps);
    const float inv = __fdiv_rn(1.0f, sum);
    float dot = __fmul_rn(__fmul_rn(p_k, inv), g_k);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
    {
      dot += __shfl_xor_sync(0xFFFFFFFFu, dot, off);
    }
    gt = to_f<T>(from_f<T>(__fmul_rn(__fsub_rn(g_k, dot), inv)));
  }
  if (scaling != 1.0f)
  {
    gt = to_f<T>(from_f<T>(__fmul_rn(gt, scaling)));
  }
  if (grad_topk != nullptr && lane < top_k)
  {
    grad_topk[static_cast<size_t>(t) * top_k + lane] = from_f<T>(gt);
  }
  __syncwarp();
  // the scatter: one add per chosen expert, rounded to T like the reference's atomic on T
  for (int k = 0; k < top_k; ++k)
  {
    const int ik = __shfl_sync(0xFFFFFFFFu, idx, k);
    const float vk = __shfl_sync(0xFFFFFFFFu, gt, k);
    if (lane == 0 && ik >= 0 && ik < experts)
    {
      gp[ik] = to_f<T>(from_f<T>(__fadd_rn(gp[ik], vk)));
    }
  }
  __syncwarp();
  T *out = grad_logits + static_cast<size_t>(t) * experts;
  if (sigmoid_gate != 0)
  {
    for (int c = lane; c < experts; c += 32)
    {
      const float ov = to_f<T>(p_row[c]);
      out[c] = from_f<T>(__fmul_rn(__fmul_rn(gp[c], ov), __fsub_rn(1.0f, ov)));
    }
    return;
  }
  if (balance_bias != nullptr)
  {
    for (int c = lane; c < experts; c += 32)
    {
      gp[c] = to_f<T>(from_f<T>(__fadd_rn(gp[c], to_f<T>(balance_bias[c]))));
    }
    __syncwarp();
  }
  float part[4];
#pragma unroll
  for (int w = 0; w < 4; ++w)
  {
    part[w] = 0.0f;
    for (int c = 32 * w + lane; c < experts; c += 128)
    {
      part[w] = __fmaf_rn(to_f<T>(p_row[c]), gp[c], part[w]);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
    {
      part[w] += __shfl_xor_sync(0xFFFFFFFFu, part[w], off);
    }
  }
  const float dot = __fadd_rn(__fadd_rn(part[0], part[2]), __fadd_rn(part[1], part[3]));
  const float lse = (z_lse_scaled != nullptr) ? to_f<T>(z_lse_scaled[t]) : 0.0f;
  for (int c = lane; c < experts; c += 32)
  {
    const float p = to_f<T>(p_row[c]);
    const float g = gp[c];
    const float y = exact_jacobian != 0 ? p : g;
    const float dy = exact_jacobian != 0 ? g : p;
    T v = from_f<T>(__fmul_rn(y, __fsub_rn(dy, dot)));
    if (z_lse_scaled != nullptr)
    {
      v = from_f<T>(__fmaf_rn(lse, p, to_f<T>(v)));
    }
    out[c] = v;
  }
}

// ------------------------------------------------------------------- aux losses
// CAIF_DeviceMoELayer::ComputeBalanceLoss / ComputeZLoss and the two gradient operands its backward
// builds (src/caif_device_moe_layer.cpp:792-835, 853-925).  Pass 1, one warp per token: the row's
// logsumexp in the order of the reference's 256-thread shared-memory tree (for rows up to 256 wide: pairs
// (c, c + 128), (c, c + 64), (c, c + 32), then 16 ... 1), rounded to T as the cached tensor is, its
// square rounded to T summed into sums[1], the scaled copy for the z-loss gradient, and the column sums
// of the probabilities into sums[2 ...].  Pass 2, one CTA: the two loss values and the per-expert
// load-balance term.  The reference adds each column sequentially over the tokens and its sum of squares
// with atomics; the sums here add in another order, so the two loss values agree to rounding, not bits.
template <typename T>
__global__ void aux_rows_kernel(const T *__restrict__ logits, const T *__restrict__ probs, T *__restrict__ lse_out,
                                T *__restrict__ z_lse_scaled, float *__restrict__ sums, int tokens, int experts,
                                float z_scale)
{
  extern __shared__ float aux_cols[];   // [experts] column sums of this CTA, then one slot for the squares
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warps_per_block = blockDim.x >> 5;
  for (int c = threadIdx.x; c <= experts; c += blockDim.x)
  {
    aux_cols[c] = 0.0f;
  }
  __syncthreads();
  float sq = 0.0f;
  for (int t = blockIdx.x * warps_per_block + warp; t < tokens; t += gridDim.x * warps_per_block)
  {
    if (probs != nullptr)
    {
      const T *p_row = probs + static_cast<size_t>(t) * experts;
      for (int c = lane; c < experts; c += 32)
      {
        atomicAdd(&aux_cols[c], to_f<T>(p_row[c]));
      }
    }
    if (logits != nullptr)
    {
      const T *x = logits + static_cast<size_t>(t) * experts;
      // thread tid of the reference's block holds columns tid, tid + 256, ...; lane l plays threads
      // l + 32 j, j = 0..7
      float vmax[8];
      float m = kNegSentinel;
#pragma unroll
      for (int j = 0; j < 8; ++j)
      {
        vmax[j] = kNegSentinel;
        for (int c = lane + 32 * j; c < experts; c += 256)
        {
          vmax[j] = fmaxf(vmax[j], to_f<T>(x[c]));
        }
        m = fmaxf(m, vmax[j]);
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
      {
        m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
      }
      float e[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
      {
        e[j] = 0.0f;
        for (int c = lane + 32 * j; c < experts; c += 256)
        {
          e[j] += expf(to_f<T>(x[c]) - m);
        }
      }
      // strides 128, 64, 32 of the tree fold thread t + stride into thread t
      float v = __fadd_rn(__fadd_rn(__fadd_rn(e[0], e[4]), __fadd_rn(e[2], e[6])),
                          __fadd_rn(__fadd_rn(e[1], e[5]), __fadd_rn(e[3], e[7])));
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
      {
        v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
      }
      const T lse_t = from_f<T>(m + logf(v));
      const float lse_f = to_f<T>(lse_t);
      if (lane == 0)
      {
        if (lse_out != nullptr)
        {
          lse_out[t] = lse_t;
        }
        if (z_lse_scaled != nullptr)
        {
          z_lse_scaled[t] = from_f<T>(__fmul_rn(lse_f, z_scale));
        }
        sq += to_f<T>(from_f<T>(__fmul_rn(lse_f, lse_f)));
      }
    }
  }
  if (lane == 0 && logits != nullptr)
  {
    atomicAdd(&aux_cols[experts], sq);
  }
  __syncthreads();
  for (int c = threadIdx.x; c < experts; c += blockDim.x)
  {
    if (probs != nullptr)
    {
      atomicAdd(&sums[2 + c], aux_cols[c]);
    }
  }
  if (threadIdx.x == 0 && logits != nullptr)
  {
    atomicAdd(&sums[1], aux_cols[experts]);
  }
}

template <typename T>
__global__ void aux_finish_kernel(float *__restrict__ sums, const int *__restrict__ expert_offsets,
                                  T *__restrict__ balance_bias, int tokens, int experts, int top_k,
                                  float balance_weight, float z_weight, int have_logits, int have_probs)
{
  if (balance_bias != nullptr)
  {
    // scale * count in the reference's float operations, stored as T
    const float denom = __fmul_rn(__fmul_rn(static_cast<float>(tokens), static_cast<float>(tokens)),
                                  static_cast<float>(top_k));
    const float scale = __fdiv_rn(__fmul_rn(balance_weight, static_cast<float>(experts)), denom);
    for (int e = threadIdx.x; e < experts; e += blockDim.x)
    {
      const int count = expert_offsets[e + 1] - expert_offsets[e];
      balance_bias[e] = from_f<T>(__fmul_rn(scale, static_cast<float>(count)));
    }
  }
  __syncthreads();
  if (threadIdx.x == 0)
  {
    float balance = 0.0f;
    if (have_probs != 0)
    {
      const float total = __fmul_rn(static_cast<float>(tokens), static_cast<float>(top_k));
      float loss = 0.0f;
      for (int e = 0; e < experts; ++e)
      {
        const int count = expert_offsets[e + 1] - expert_offsets[e];
        const float fraction = __fdiv_rn(static_cast<float>(count), total);
        const float mean_p = __fdiv_rn(to_f<T>(from_f<T>(sums[2 + e])), static_cast<float>(tokens));
        loss = __fadd_rn(loss, __fmul_rn(fraction, mean_p));
      }
      balance = __fmul_rn(__fmul_rn(balance_weight, static_cast<float>(experts)), loss);
    }
    float z = 0.0f;
    if (have_logits != 0)
    {
      z = __fdiv_rn(__fmul_rn(z_weight, to_f<T>(from_f<T>(sums[1]))), static_cast<float>(tokens));
    }
    sums[0] = balance;
    sums[1] = z;
  }
}

// ---------------------------------------------------------- aux-loss-free bias
// launch_moe_bias_update (src/caif_cuda_kernels_moe.cu:481-537): every expert's selection bias moves by
// `rate` towards balance, up when its load is under the mean and down when over.  The mean is the
// reference's: 256 threads striding the counts, a shared-memory tree, one division (exact for loads
// below 2^24, the same rounding beyond).  counts[e], or offsets[e + 1] - offsets[e] when `from_offsets`.
template <typename T>
__global__ void bias_update_kernel(T *__restrict__ bias, const int *__restrict__ counts, int experts, float rate,
                                   int from_offsets)
{
  __shared__ float partial[256];
  const int tid = threadIdx.x;
  auto load = [&](int e) -> float
  { return static_cast<float>(from_offsets != 0 ? counts[e + 1] - counts[e] : counts[e]); };
  float local = 0.0f;
  for (int e = tid; e < experts; e += 256)
  {
    local += load(e);
  }
  partial[tid] = local;
  __syncthreads();
  for (int stride = 128; stride > 0; stride >>= 1)
  {
    if (tid < stride)
    {
      partial[tid] += partial[tid + stride];
    }
    __syncthreads();
  }
  const float mean = __fdiv_rn(partial[0], static_cast<float>(experts));
  for (int e = tid; e < experts; e += 256)
  {
    const float err = mean - load(e);
    const float step = err > 0.0f ? rate : (err < 0.0f ? -rate : 0.0f);
    bias[e] = from_f<T>(to_f<T>(bias[e]) + step);
  }
}

// ------------------------------------------------------------------ dispatch map
// Stable counting rank on the device.  One CTA walks the [T*k] index list in
// chunks of blockDim entries; inside a chunk, warps rank equal experts with
// match_any, a per-warp histogram is scanned over warps, and a running count per
// expert carries across chunks.  The rank of an entry is the number of earlier
// entries (token-major, k-minor) with the same expert -- what the reference's
// host loop assigns.
constexpr int kMapThreads = 1024;
constexpr int kMapWarps = kMapThreads / 32;

__global__ void __launch_bounds__(kMapThreads)
build_dispatch_kernel(const int *__restrict__ expert_indices, int64_t total, int num_experts, int capacity,
                      int *__restrict__ dispatch_map, int *__restrict__ expert_offsets)
{
  extern __shared__ int s_map[];
  int *running = s_map;                      // [E]
  int *warp_hist = s_map + num_experts;      // [warps][E]
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  for (int e = tid; e < num_experts; e += kMapThreads)
  {
    running[e] = 0;
  }
  __syncthreads();
  for (int64_t base = 0; base < total; base += kMapThreads)
  {
    for (int e = lane; e < num_experts; e += 32)
    {
      warp_hist[warp * num_experts + e] = 0;
    }
    __syncwarp();
    const int64_t i = base + tid;
    int e = -1;
    if (i < total)
    {
      const int v = expert_indices[i];
      if (v >= 0 && v < num_experts)
      {
        e = v;
      }
    }
    const unsigned peers = __match_any_sync(0xFFFFFFFFu, e);
    const int lane_rank = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && lane_rank == 0)
    {
      warp_hist[warp * num_experts + e] = __popc(peers);
    }
    __syncthreads();
    // exclusive scan over warps, per expert; fold the chunk into the running count
    for (int x = tid; x < num_experts; x += kMapThreads)
    {
      int acc = running[x];
      for (int w = 0; w < kMapWarps; ++w)
      {
        const int c = warp_hist[w * num_experts + x];
        warp_hist[w * num_experts + x] = acc;
        acc += c;
      }
      running[x] = acc;
    }
    __syncthreads();
    if (i < total)
    {
      int pos = -1;
      if (e >= 0)
      {
        const int rank = warp_hist[warp * num_experts + e] + lane_rank;
        if (capacity <= 0 || rank < capacity)
        {
          pos = rank;
        }
      }
      dispatch_map[i] = pos;
    }
    __syncthreads();
  }
  if (tid == 0)
  {
    int acc = 0;
    expert_offsets[0] = 0;
    for (int e = 0; e < num_experts; ++e)
    {
      int c = running[e];
      if (capacity > 0 && c > capacity)
      {
        c = capacity;
      }
      acc += c;
      expert_offsets[e + 1] = acc;
    }
  }
}

// ------------------------------------------------------------- dispatch / combine
template <typename T>
__global__ void moe_dispatch_kernel(const T *__restrict__ input, const int *__restrict__ expert_indices,
                                    const int *__restrict__ dispatch_map, const int *__restrict__ expert_offsets,
                                    T *__restrict__ buffer, int64_t assignments, int dim, int top_k)
{
  const int lane = threadIdx.x & 31;
  const int64_t a = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (a >= assignments)
  {
    return;
  }
  const int e = expert_indices[a];
  const int pos = dispatch_map[a];
  if (e < 0 || pos < 0)
  {
    return;
  }
  const T *src = input + (a / top_k) * dim;
  T *dst = buffer + (static_cast<int64_t>(expert_offsets[e]) + pos) * dim;
  const int vec = 16 / static_cast<int>(sizeof(T));
  if ((dim % vec) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0)
  {
    const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
    uint4 *d4 = reinterpret_cast<uint4 *>(dst);
    for (int i = lane; i < dim / vec; i += 32)
    {
      d4[i] = s4[i];
    }
  }
  else
  {
    for (int i = lane; i < dim; i += 32)
    {
      dst[i] = src[i];
    }
  }
}

template <typename T>
__global__ void moe_combine_kernel(const T *__restrict__ buffer, const int *__restrict__ expert_indices,
                                   const T *__restrict__ expert_weights, const int *__restrict__ dispatch_map,
                                   const int *__restrict__ expert_offsets, T *__restrict__ output, int num_tokens,
                                   int dim, int top_k)
{
  const int64_t total = static_cast<int64_t>(num_tokens) * dim;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
  {
    const int token = static_cast<int>(i / dim);
    const int d = static_cast<int>(i % dim);
    float sum = 0.0f;
    for (int k = 0; k < top_k; ++k)
    {
      const int e = expert_indices[token * top_k + k];
      const int pos = dispatch_map[token * top_k + k];
      if (e >= 0 && pos >= 0)
      {
        const float w = to_f<T>(expert_weights[token * top_k + k]);
        const float v = to_f<T>(buffer[(static_cast<int64_t>(expert_offsets[e]) + pos) * dim + d]);
        sum = fmaf(w, v, sum);
      }
    }
    output[i] = from_f<T>(sum);
  }
}

// ------------------------------------------------------------------- SwiGLU
template <typename T>
__global__ void swiglu_fwd_kernel(const T *__restrict__ gate, const T *__restrict__ up, T *__restrict__ hidden,
                                  int64_t n)
{
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
  {
    const float x = to_f<T>(gate[i]);
    const T act = from_f<T>(x / (1.0f + expf(-x)));
    hidden[i] = from_f<T>(to_f<T>(act) * to_f<T>(up[i]));
  }
}

template <typename T>
__global__ void swiglu_bwd_kernel(const T *__restrict__ g_hidden, const T *__restrict__ gate,
                                  const T *__restrict__ up, T *__restrict__ g_gate, T *__restrict__ g_up, int64_t n)
{
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
  {
    const float x = to_f<T>(gate[i]);
    const float gh = to_f<T>(g_hidden[i]);
    const T act = from_f<T>(x / (1.0f + expf(-x)));
    g_up[i] = from_f<T>(gh * to_f<T>(act));
    const float gv = to_f<T>(from_f<T>(gh * to_f<T>(up[i])));
    const float s = 1.0f / (1.0f + expf(-x));
    g_gate[i] = from_f<T>(gv * s * (1.0f + x * (1.0f - s)));
  }
}

// Non-gated experts (CAIF_DeviceMoEFrozenExpert with UseGated() == false,
// src/caif_device_moe_frozen_expert.cpp:158-162, 318-331): hidden = SiLU(up), g_up = SiLUBackward(up, g_hidden)
// with the reference's formulas (src/caif_cuda_kernels_activations.cu:513-514, 558-561).
template <typename T>
__global__ void silu_fwd_kernel(const T *__restrict__ x_in, T *__restrict__ out, int64_t n)
{
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
  {
    const float x = to_f<T>(x_in[i]);
    out[i] = from_f<T>(x / (1.0f + expf(-x)));
  }
}

template <typename T>
__global__ void silu_bwd_kernel(const T *__restrict__ x_in, const T *__restrict__ grad, T *__restrict__ out, int64_t n)
{
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
  {
    const float x = to_f<T>(x_in[i]);
    const float s = 1.0f / (1.0f + expf(-x));
    out[i] = from_f<T>(to_f<T>(grad[i]) * s * (1.0f + x * (1.0f - s)));
  }
}

template <typename T>
__global__ void add_kernel(const T *__restrict__ a, const T *__restrict__ b, T *__restrict__ out, int64_t n)
{
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
  {
    out[i] = from_f<T>(to_f<T>(a[i]) + to_f<T>(b[i]));
  }
}

// ---- 16-byte vector forms of the elementwise kernels (same arithmetic per element) ----
template <typename T>
struct Vec16
{
  static constexpr int N = 16 / static_cast<int>(sizeof(T));
};

template <typename T>
__device__ __forceinline__ void load_vec(const T *p, float (&v)[Vec16<T>::N])
{
  const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(p));
  const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
  for (int i = 0; i < Vec16<T>::N; ++i)
  {
    v[i] = to_f<T>(e[i]);
  }
}

template <typename T>
__device__ __forceinline__ void store_vec(T *p, const float (&v)[Vec16<T>::N])
{
  uint4 raw;
  T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
  for (int i = 0; i < Vec16<T>::N; ++i)
  {
    e[i] = from_f<T>(v[i]);
  }
  *reinterpret_cast<uint4 *>(p) = raw;
}

template <typename T>
__global__ void swiglu_fwd_vec_kernel(const T *__restrict__ gate, const T *__restrict__ up, T *__restrict__ hidden,
                                      int64_t n_vec)
{
  constexpr int N = Vec16<T>::N;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += stride)
  {
    float g[N], u[N], h[N];
    load_vec<T>(gate + i * N, g);
    load_vec<T>(up + i * N, u);
#pragma unroll
    for (int j = 0; j < N; ++j)
    {
      const T act = from_f<T>(g[j] / (1.0f + expf(-g[j])));
      h[j] = to_f<T>(act) * u[j];
    }
    store_vec<T>(hidden + i * N, h);
  }
}

template <typename T>
__global__ void swiglu_bwd_vec_kernel(const T *__restrict__ g_hidden, const T *__restrict__ gate,
                                      const T *__restrict__ up, T *__restrict__ g_gate, T *__restrict__ g_up,
                                      int64_t n_vec)
{
  constexpr int N = Vec16<T>::N;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += stride)
  {
    float x[N], gh[N], u[N], gg[N], gu[N];
    load_vec<T>(gate + i * N, x);
    load_vec<T>(g_hidden + i * N, gh);
    load_vec<T>(up + i * N, u);
#pragma unroll
    for (int j = 0; j < N; ++j)
    {
      const T act = from_f<T>(x[j] / (1.0f + expf(-x[j])));
      gu[j] = gh[j] * to_f<T>(act);
      const float gv = to_f<T>(from_f<T>(gh[j] * u[j]));
      const float sg = 1.0f / (1.0f + expf(-x[j]));
      gg[j] = gv * sg * (1.0f + x[j] * (1.0f - sg));
    }
    store_vec<T>(g_up + i * N, gu);
    store_vec<T>(g_gate + i * N, gg);
  }
}

template <typename T>
__global__ void moe_combine_vec_kernel(const T *__restrict__ buffer, const int *__restrict__ expert_indices,
                                       const T *__restrict__ expert_weights, const int *__restrict__ dispatch_map,
                                       const int *__restrict__ expert_offsets, T *__restrict__ output,
                                       int num_tokens, int dim, int top_k)
{
  constexpr int N = Vec16<T>::N;
  const int dim_vec = dim / N;
  const int64_t total = static_cast<int64_t>(num_tokens) * dim_vec;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
  {
    const int token = static_cast<int>(i / dim_vec);
    const int d = static_cast<int>(i % dim_vec) * N;
    float sum[N];
#pragma unroll
    for (int j = 0; j < N; ++j)
    {
      sum[j] = 0.0f;
    }
    for (int k = 0; k < top_k; ++k)
    {
      const int e = expert_indices[token * top_k + k];
      const int pos = dispatch_map[token * top_k + k];
      if (e >= 0 && pos >= 0)
      {
        const float w = to_f<T>(expert_weights[token * top_k + k]);
        float v[N];
        load_vec<T>(buffer + (static_cast<int64_t>(expert_offsets[e]) + pos) * dim + d, v);
#pragma unroll
        for (int j = 0; j < N; ++j)
        {
          sum[j] = fmaf(w, v[j], sum[j]);
        }
      }
    }
    store_vec<T>(output + static_cast<int64_t>(token) * dim + d, sum);
  }
}

// ---- backward of combine and dispatch (src/caif_cuda_kernels_moe.cu:816-1067) ----
// grad_buffer[slot(t,k), d] = w[t,k] * grad_output[t,d]; one warp per (t,k), 16-byte pieces when possible
template <typename T>
__global__ void moe_combine_bwd_grad_expert_kernel(const T *__restrict__ grad_output,
                                                   const int *__restrict__ expert_indices,
                                                   const T *__restrict__ expert_weights,
                                                   const int *__restrict__ dispatch_map,
                                                   const int *__restrict__ expert_offsets,
                                                   T *__restrict__ grad_buffer, int64_t assignments, int dim,
                                                   int top_k, int vec_ok)
{
  constexpr int N = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t a = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (a >= assignments)
  {
    return;
  }
  const int e = expert_indices[a];
  const int pos = dispatch_map[a];
  if (e < 0 || pos < 0)
  {
    return;
  }
  const float w = to_f<T>(expert_weights[a]);
  const T *src = grad_output + (a / top_k) * dim;
  T *dst = grad_buffer + (static_cast<int64_t>(expert_offsets[e]) + pos) * dim;
  if (vec_ok)
  {
    for (int i = lane * N; i < dim; i += 32 * N)
    {
      float v[N];
      load_vec<T>(src + i, v);
#pragma unroll
      for (int j = 0; j < N; ++j)
      {
        v[j] = __fmul_rn(w, v[j]);
      }
      store_vec<T>(dst + i, v);
    }
  }
  else
  {
    for (int i = lane; i < dim; i += 32)
    {
      dst[i] = from_f<T>(__fmul_rn(w, to_f<T>(src[i])));
    }
  }
}

// grad_weights[t,k] = <grad_output[t,:], buffer[slot(t,k),:]>: the reference's summation order -
// 256 threads, thread i takes d = i, i+256, ... with fused multiply-adds, then a halving tree
constexpr int kGradWeightsThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kGradWeightsThreads)
moe_combine_bwd_grad_weights_kernel(const T *__restrict__ grad_output, const T *__restrict__ buffer,
                                    const int *__restrict__ expert_indices, const int *__restrict__ dispatch_map,
                                    const int *__restrict__ expert_offsets, T *__restrict__ grad_weights, int dim,
                                    int top_k)
{
  const int64_t a = blockIdx.x;
  const int e = expert_indices[a];
  const int pos = dispatch_map[a];
  float partial = 0.0f;
  if (e >= 0 && pos >= 0)
  {
    const T *src = buffer + (static_cast<int64_t>(expert_offsets[e]) + pos) * dim;
    const T *g = grad_output + (a / top_k) * dim;
    for (int d = threadIdx.x; d < dim; d += kGradWeightsThreads)
    {
      partial = fmaf(to_f<T>(g[d]), to_f<T>(src[d]), partial);
    }
  }
  __shared__ float sdata[kGradWeightsThreads];
  sdata[threadIdx.x] = partial;
  __syncthreads();
  for (int stride = kGradWeightsThreads / 2; stride > 0; stride >>= 1)
  {
    if (threadIdx.x < stride)
    {
      sdata[threadIdx.x] = __fadd_rn(sdata[threadIdx.x], sdata[threadIdx.x + stride]);
    }
    __syncthreads();
  }
  if (threadIdx.x == 0)
  {
    grad_weights[a] = from_f<T>(sdata[0]);
  }
}

// grad_input[t,d] = sum over k (in order) of grad_buffer[slot(t,k), d]
template <typename T>
__global__ void moe_dispatch_bwd_kernel(const T *__restrict__ grad_buffer, const int *__restrict__ expert_indices,
                                        const int *__restrict__ dispatch_map,
                                        const int *__restrict__ expert_offsets, T *__restrict__ grad_input,
                                        int num_tokens, int dim, int top_k, int vec_ok)
{
  constexpr int N = Vec16<T>::N;
  const int step = vec_ok ? N : 1;
  const int dim_steps = dim / step;
  const int64_t total = static_cast<int64_t>(num_tokens) * dim_steps;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
  {
    const int token = static_cast<int>(i / dim_steps);
    const int d = static_cast<int>(i % dim_steps) * step;
    float sum[N];
#pragma unroll
    for (int j = 0; j < N; ++j)
    {
      sum[j] = 0.0f;
    }
    for (int k = 0; k < top_k; ++k)
    {
      const int e = expert_indices[token * top_k + k];
      const int pos = dispatch_map[token * top_k + k];
      if (e >= 0 && pos >= 0)
      {
        const T *src = grad_buffer + (static_cast<int64_t>(expert_offsets[e]) + pos) * dim + d;
        if (vec_ok)
        {
          float v[N];
          load_vec<T>(src, v);
#pragma unroll
          for (int j = 0; j < N; ++j)
          {
            sum[j] = __fadd_rn(sum[j], v[j]);
          }
        }
        else
        {
          sum[0] = __fadd_rn(sum[0], to_f<T>(src[0]));
        }
      }
    }
    T *dst = grad_input + static_cast<int64_t>(token) * dim + d;
    if (vec_ok)
    {
      store_vec<T>(dst, sum);
    }
    else
    {
      dst[0] = from_f<T>(sum[0]);
    }
  }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int ew_grid(int64_t n)
{
  int64_t g = (n + 255) / 256;
  if (g > 148 * 16)
  {
    g = 148 * 16;
  }
  return static_cast<int>(g < 1 ? 1 : g);
}

}  // namespace

#define CAIFQ_DISPATCH_FLOAT(dtype, CALL)          \
  switch (dtype)                                   \
  {                                                \
    case CAIFQ_F32:                                \
    {                                              \
      using T = float;                             \
      CALL;                                        \
      break;                                       \
    }                                              \
    case CAIFQ_F16:                                \
    {                                              \
      using T = __half;                            \
      CALL;                                        \
      break;                                       \
    }                                              \
    case CAIFQ_BF16:                               \
    {                                              \
      using T = __nv_bfloat16;                     \
      CALL;                                        \
      break;                                       \
    }                                              \
    default:                                       \
      set_error("unsupported dtype %d", dtype);    \
      return CAIFQ_ERR_INVALID;                    \
  }

int launch_moe_topk(const void *probs, int dtype, int *indices, void *values, int batch, int dim, int k,
                    cudaStream_t s)
{
  if (batch <= 0)
  {
    return CAIFQ_OK;
  }
  int warps = 8;
  while (warps > 1 && static_cast<size_t>(warps) * dim * sizeof(float) > 40 * 1024)
  {
    warps >>= 1;
  }
  const size_t smem = static_cast<size_t>(warps) * dim * sizeof(float);
  if (smem > 48 * 1024)
  {
    set_error("moe_topk: dim=%d too large", dim);
    return CAIFQ_ERR_UNSUPPORTED;
  }
  const int grid = (batch + warps - 1) / warps;
  CAIFQ_DISPATCH_FLOAT(dtype, (topk_kernel<T><<<grid, warps * 32, smem, s>>>(
                                  static_cast<const T *>(probs), indices, static_cast<T *>(values), batch, dim, k)));
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_moe_route_grouped(const void *input, const void *bias, void *scores_out, int *indices, void *weights,
                             int dtype, int batch, int dim, int k, int n_group, int topk_group, int apply_sigmoid,
                             cudaStream_t s)
{
  if (batch <= 0)
  {
    return CAIFQ_OK;
  }
  const size_t per_warp = (static_cast<size_t>(2) * dim + 64) * sizeof(float);
  int warps = 8;
  while (warps > 1 && warps * per_warp > 40 * 1024)
  {
    warps >>= 1;
  }
  if (warps * per_warp > 48 * 1024)
  {
    set_error("moe_route_grouped: dim=%d too large", dim);
    return CAIFQ_ERR_UNSUPPORTED;
  }
  const int grid = (batch + warps - 1) / warps;
  CAIFQ_DISPATCH_FLOAT(dtype, (route_grouped_kernel<T><<<grid, warps * 32, warps * per_warp, s>>>(
                                  static_cast<const T *>(input), static_cast<const T *>(bias),
                                  static_cast<T *>(scores_out), indices, static_cast<T *>(weights), batch, dim, k,
                                  n_group, topk_group, apply_sigmoid)));
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_moe_normalize_rows(const void *input, void *output, int dtype, int batch, int dim, cudaStream_t s)
{
  if (batch <= 0)
  {
    return CAIFQ_OK;
  }
  const int warps = 8;
  const int grid = (batch + warps - 1) / warps;
  CAIFQ_DISPATCH_FLOAT(dtype, (normalize_rows_kernel<T><<<grid, warps * 32, 0, s>>>(
                                  static_cast<const T *>(input), static_cast<T *>(output), batch, dim)));
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_moe_router_softmax(const void *logits, const void *bias, void *probs, int dtype, int rows, int cols,
                              cudaStream_t s)
{
  if (rows <= 0)
  {
    return CAIFQ_OK;
  }
  const int warps = 8;
  const int grid = (rows + warps - 1) / warps;
  CAIFQ_DISPATCH_FLOAT(dtype, (router_softmax_kernel<T><<<grid, warps * 32, 0, s>>>(
                                  static_cast<const T *>(logits), static_cast<const T *>(bias),
                                  static_cast<T *>(probs), rows, cols)));
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_moe_router_bwd(const void *grad_w, const void *probs, const int *indices, const void *balance_bias,
                          const void *z_lse_scaled, void *grad_topk, void *grad_logits, int dtype, int tokens,
                          int experts, int top_k, int sigmoid_gate, int normalize, float scaling, int exact_jacobian,
                          cudaStream_t s)
{
  if (tokens <= 0)
  {
    return CAIFQ_OK;
  }
  const size_t per_warp = static_cast<size_t>(experts) * sizeof(float);
  int warps = 8;
  while (warps > 1 && warps * per_warp > 40 * 1024)
  {
    warps >>= 1;
  }
  if (warps * per_warp > 48 * 1024)
  {
    set_error("moe_router_bwd: experts=%d too many", experts);
    return CAIFQ_ERR_UNSUPPORTED;
  }
  const int grid = (tokens + warps - 1) / warps;
  CAIFQ_DISPATCH_FLOAT(dtype, (router_bwd_kernel<T><<<grid, warps * 32, warps * per_warp, s>>>(
                                  static_cast<const T *>(grad_w), static_cast<const T *>(probs), indices,
                                  static_cast<const T *>(balance_bias), static_cast<const T *>(z_lse_scaled),
                                  static_cast<T *>(grad_topk), static_cast<T *>(grad_logits), tokens, experts, top_k,
                                  sigmoid_gate, normalize, scaling, exact_jacobian)));
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_moe_aux_losses(const void *logits, const void *probs, const int *expert_offsets, void *balance_bias,
                          void *lse, void *z_lse_scaled, float *sums, int dtype, int tokens, int experts, int top_k,
                          float balance_weight, float z_weight, cudaStream_t s)
{
  cudaError_t err = cudaMemsetAsync(sums, 0, sizeof(float) * (2 + static_cast<size_t>(experts)), s);
  if (err != cudaSuccess)
  {
    set_error("moe_aux_losses: memset failed: %s", cudaGetErrorString(err));
    return CAIFQ_ERR_CUDA;
  }
  if (tokens > 0 && (logits != nullptr || probs != nullptr))
  {
    const int warps = 8;
    int grid = (tokens + warps - 1) / warps;
    if (grid > 592)
    {
      grid = 592;   // four CTAs per SM; each adds its column sums once
    }
    const float z_scale = 2.0f * z_weight / static_cast<float>(tokens);
    const size_t smem = (static_cast<size_t>(experts) + 1) * sizeof(float);
    CAIFQ_DISPATCH_FLOAT(dtype, (aux_rows_kernel<T><<<grid, warps * 32, smem, s>>>(
                                    static_cast<const T *>(logits), static_cast<const T *>(probs),
                                    static_cast<T *>(lse), static_cast<T *>(z_lse_scaled), sums, tokens, experts,
                                    z_scale)));
    CAIFQ_CHECK_LAUNCH();
  }
  CAIFQ_DISPATCH_FLOAT(dtype, (aux_finish_kernel<T><<<1, 256, 0, s>>>(
                                  sums, expert_offsets, static_cast<T *>(balance_bias), tokens, experts, top_k,
                                  balance_weight, z_weight, logits != nullptr ? 1 : 0, probs != nullptr ? 1 : 0)));
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_moe_bias_update(void *bias, const int *counts, int dtype, int experts, float rate, int from_offsets,
                           cudaStream_t s)
{
  CAIFQ_DISPATCH_FLOAT(dtype, (bias_update_kernel<T><<<1, 256, 0, s>>>(static_cast<T *>(bias), counts, experts, rate,
                                                                       from_offsets)));
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_moe_build_dispatch(const int *expert_indices, int num_tokens, int top_k, int num_experts, int capacity,
                              int *dispatch_map, int *expert_offsets, cudaStream_t s)
{
  const size_t smem = static_cast<size_t>(num_experts) * (kMapWarps + 1) * sizeof(int);
  if (smem > 48 * 1024)
  {
    set_error("moe_build_dispatch: num_experts=%d exceeds the supported %d", num_experts,
              static_cast<int>(48 * 1024 / ((kMapWarps + 1) * sizeof(int))));
    return CAIFQ_ERR_UNSUPPORTED;
  }
  const int64_t total = static_cast<int64_t>(num_tokens) * top_k;
  build_dispatch_kernel<<<1, kMapThreads, smem, s>>>(expert_indices, total, num_experts, capacity, dispatch_map,
                                                     expert_offsets);
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_moe_dispatch(const void *input, int dtype, const int *expert_indices, const int *dispatch_map,
                        const int *expert_offsets, void *buffer, int num_tokens, int dim, int top_k, cudaStream_t s)
{
  const int64_t assignments = static_cast<int64_t>(num_tokens) * top_k;
  if (assignments <= 0)
  {
    return CAIFQ_OK;
  }
  const int64_t grid = (assignments * 32 + 255) / 256;
  CAIFQ_DISPATCH_FLOAT(dtype, (moe_dispatch_kernel<T><<<static_cast<unsigned>(grid), 256, 0, s>>>(
                                  static_cast<const T *>(input), expert_indices, dispatch_map, expert_offsets,
                                  static_cast<T *>(buffer), assignments, dim, top_k)));
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_moe_combine(const void *buffer, int dtype, const int *expert_indices, const void *expert_weights,
                       const int *dispatch_map, const int *expert_offsets, void *output, int num_tokens, int dim,
                       int top_k, cudaStream_t s)
{
  const int64_t total = static_cast<int64_t>(num_tokens) * dim;
  if (total <= 0)
  {
    return CAIFQ_OK;
  }
  const bool vec = aligned16(buffer) && aligned16(output);
  CAIFQ_DISPATCH_FLOAT(
      dtype, (vec && (dim % Vec16<T>::N) == 0
                  ? moe_combine_vec_kernel<T><<<ew_grid(total / Vec16<T>::N), 256, 0, s>>>(
                        static_cast<const T *>(buffer), expert_indices, static_cast<const T *>(expert_weights),
                        dispatch_map, expert_offsets, static_cast<T *>(output), num_tokens, dim, top_k)
                  : moe_combine_kernel<T><<<ew_grid(total), 256, 0, s>>>(
                        static_cast<const T *>(buffer), expert_indices, static_cast<const T *>(expert_weights),
                        dispatch_map, expert_offsets, static_cast<T *>(output), num_tokens, dim, top_k)));
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_moe_combine_bwd_grad_expert(const void *grad_output, int dtype, const int *expert_indices,
                                       const void *expert_weights, const int *dispatch_map, const int *expert_offsets,
                                       void *grad_buffer, int num_tokens, int dim, int top_k, cudaStream_t s)
{
  const int64_t assignments = static_cast<int64_t>(num_tokens) * top_k;
  if (assignments <= 0)
  {
    return CAIFQ_OK;
  }
  const int64_t threads = assignments * 32;
  const unsigned grid = static_cast<unsigned>((threads + 255) / 256);
  const bool al = aligned16(grad_output) && aligned16(grad_buffer);
  CAIFQ_DISPATCH_FLOAT(dtype, (moe_combine_bwd_grad_expert_kernel<T><<<grid, 256, 0, s>>>(
                                  static_cast<const T *>(grad_output), expert_indices,
                                  static_cast<const T *>(expert_weights), dispatch_map, expert_offsets,
                                  static_cast<T *>(grad_buffer), assignments, dim, top_k,
                                  (al && (dim % Vec16<T>::N) == 0) ? 1 : 0)));
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_moe_combine_bwd_grad_weights(const void *grad_output, const void *buffer, int dtype,
                                        const int *expert_indices, const int *dispatch_map,
                                        const int *expert_offsets, void *grad_weights, int num_tokens, int dim,
                                        int top_k, cudaStream_t s)
{
  const int64_t assignments = static_cast<int64_t>(num_tokens) * top_k;
  if (assignments <= 0)
  {
    return CAIFQ_OK;
  }
  CAIFQ_DISPATCH_FLOAT(dtype, (moe_combine_bwd_grad_weights_kernel<T>
                               <<<static_cast<unsigned>(assignments), kGradWeightsThreads, 0, s>>>(
                                   static_cast<const T *>(grad_output), static_cast<const T *>(buffer),
                                   expert_indices, dispatch_map, expert_offsets, static_cast<T *>(grad_weights), dim,
                                   top_k)));
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_moe_dispatch_bwd(const void *grad_buffer, int dtype, const int *expert_indices, const int *dispatch_map,
                            const int *expert_offsets, void *grad_input, int num_tokens, int dim, int top_k,
                            cudaStream_t s)
{
  const int64_t total = static_cast<int64_t>(num_tokens) * dim;
  if (total <= 0)
  {
    return CAIFQ_OK;
  }
  const bool al = aligned16(grad_buffer) && aligned16(grad_input);
  CAIFQ_DISPATCH_FLOAT(dtype, (moe_dispatch_bwd_kernel<T><<<ew_grid(total / 4), 256, 0, s>>>(
                                  static_cast<const T *>(grad_buffer), expert_indices, dispatch_map, expert_offsets,
                                  static_cast<T *>(grad_input), num_tokens, dim, top_k,
                                  (al && (dim % Vec16<T>::N) == 0) ? 1 : 0)));
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_swiglu_fwd(const void *gate, const void *up, void *hidden, int dtype, int64_t n, cudaStream_t s)
{
  if (n <= 0)
  {
    return CAIFQ_OK;
  }
  const bool vec = aligned16(gate) && aligned16(up) && aligned16(hidden);
  CAIFQ_DISPATCH_FLOAT(
      dtype, (vec && (n % Vec16<T>::N) == 0
                  ? swiglu_fwd_vec_kernel<T><<<ew_grid(n / Vec16<T>::N), 256, 0, s>>>(
                        static_cast<const T *>(gate), static_cast<const T *>(up), static_cast<T *>(hidden),
                        n / Vec16<T>::N)
                  : swiglu_fwd_kernel<T><<<ew_grid(n), 256, 0, s>>>(static_cast<const T *>(gate),
                                                                    static_cast<const T *>(up),
                                                                    static_cast<T *>(hidden), n)));
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_swiglu_bwd(const void *g_hidden, const void *gate, const void *up, void *g_gate, void *g_up, int dtype,
                      int64_t n, cudaStream_t s)
{
  if (n <= 0)
  {
    return CAIFQ_OK;
  }
  const bool vec = aligned16(g_hidden) && aligned16(gate) && aligned16(up) && aligned16(g_gate) && aligned16(g_up);
  CAIFQ_DISPATCH_FLOAT(
      dtype, (vec && (n % Vec16<T>::N) == 0
                  ? swiglu_bwd_vec_kernel<T><<<ew_grid(n / Vec16<T>::N), 256, 0, s>>>(
                        static_cast<const T *>(g_hidden), static_cast<const T *>(gate), static_cast<const T *>(up),
                        static_cast<T *>(g_gate), static_cast<T *>(g_up), n / Vec16<T>::N)
                  : swiglu_bwd_kernel<T><<<ew_grid(n), 256, 0, s>>>(
                        static_cast<const T *>(g_hidden), static_cast<const T *>(gate), static_cast<const T *>(up),
                        static_cast<T *>(g_gate), static_cast<T *>(g_up), n)));
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_silu_fwd(const void *x, void *out, int dtype, int64_t n, cudaStream_t s)
{
  if (n <= 0)
  {
    return CAIFQ_OK;
  }
  CAIFQ_DISPATCH_FLOAT(dtype, (silu_fwd_kernel<T><<<ew_grid(n), 256, 0, s>>>(static_cast<const T *>(x),
                                                                             static_cast<T *>(out), n)));
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_silu_bwd(const void *x, const void *grad, void *out, int dtype, int64_t n, cudaStream_t s)
{
  if (n <= 0)
  {
    return CAIFQ_OK;
  }
  CAIFQ_DISPATCH_FLOAT(dtype, (silu_bwd_kernel<T><<<ew_grid(n), 256, 0, s>>>(
                                  static_cast<const T *>(x), static_cast<const T *>(grad), static_cast<T *>(out), n)));
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_add(const void *a, const void *b, void *out, int dtype, int64_t n, cudaStream_t s)
{
  if (n <= 0)
  {
    return CAIFQ_OK;
  }
  CAIFQ_DISPATCH_FLOAT(dtype, (add_kernel<T><<<ew_grid(n), 256, 0, s>>>(
                                  static_cast<const T *>(a), static_cast<const T *>(b), static_cast<T *>(out), n)));
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

}  // namespace caifq
