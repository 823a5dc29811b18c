/*
 * CPU oracle for the quantized frozen-linear path of cppaif/caif.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of
 * the reference's device kernels so that the CUDA library can be checked
 * against it.  Nothing in the shipped library links, loads or calls it; it is
 * used by the tests, by the smoke check and by the benchmark's CPU-baseline
 * leg, always as the checker or the baseline and never as the product path.
 *
 * Parity pin: the restatement is compared bit for bit with the reference's own
 * kernels (src/caif_cuda_kernels_quant.cu, src/caif_cuda_kernels_moe.cu,
 * compiled unmodified into oracle/_ref/) by the GPU tests, and with golden
 * vectors captured from those kernels (tests/golden/).
 *
 * Every function cites the reference lines it follows.  All arithmetic is
 * IEEE fp32 without contraction (build with -ffp-contract=off, no fast-math).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_EXPORT __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* Scalar conversions (round to nearest even), matching __float2half,        */
/* __half2float, __float2bfloat16, __bfloat162float used at                  */
/* src/caif_cuda_kernels_quant.cu:49,97 and by the elementwise kernels.      */
/* ------------------------------------------------------------------------- */

static inline uint32_t f32_bits(float f)
{
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}

static inline float bits_f32(uint32_t u)
{
  float f;
  memcpy(&f, &u, 4);
  return f;
}

ORC_EXPORT uint16_t orc_f32_to_f16(float f)
{
  const uint32_t x = f32_bits(f);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const uint32_t abs = x & 0x7FFFFFFFu;
  if (abs > 0x7F800000u)
  {
    return 0x7FFFu; /* CUDA's canonical half NaN */
  }
  if (abs >= 0x47800000u) /* >= 65536: overflow to inf (65520 rounds up too, handled below) */
  {
    return (uint16_t)(sign | 0x7C00u);
  }
  if (abs < 0x33000001u) /* <= 2^-25: rounds to zero (exactly 2^-25 ties to even = 0) */
  {
    return (uint16_t)sign;
  }
  int32_t exp = (int32_t)(abs >> 23) - 127;
  uint32_t man = (abs & 0x007FFFFFu) | 0x00800000u;
  uint32_t shift;
  uint32_t half_exp;
  if (exp < -14)
  {
    /* subnormal half: value = man * 2^(exp-23); target unit 2^-24 */
    shift = (uint32_t)(13 + (-14 - exp));
    half_exp = 0;
  }
  else
  {
    shift = 13;
    half_exp = (uint32_t)(exp + 15);
  }
  uint32_t q = man >> shift;
  const uint32_t rem = man & ((1u << shift) - 1u);
  const uint32_t halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (q & 1u)))
  {
    ++q;
  }
  uint32_t out;
  if (half_exp == 0)
  {
    out = q; /* a carry into bit 10 lands on the smallest normal, as it should */
  }
  else
  {
    out = ((half_exp - 1u) << 10) + q; /* q carries the implicit bit (1<<10) */
  }
  if (out >= 0x7C00u)
  {
    out = 0x7C00u;
  }
  return (uint16_t)(sign | out);
}

ORC_EXPORT float orc_f16_to_f32(uint16_t h)
{
  const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1Fu;
  const uint32_t man = h & 0x3FFu;
  if (exp == 0)
  {
    if (man == 0)
    {
      return bits_f32(sign);
    }
    const float v = ldexpf((float)man, -24);
    return sign ? -v : v;
  }
  if (exp == 31)
  {
    return bits_f32(sign | 0x7F800000u | (man << 13));
  }
  return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

ORC_EXPORT uint16_t orc_f32_to_bf16(float f)
{
  uint32_t x = f32_bits(f);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u)
  {
    return 0x7FFFu; /* __float2bfloat16 canonical NaN */
  }
  const uint32_t lsb = (x >> 16) & 1u;
  x += 0x7FFFu + lsb;
  return (uint16_t)(x >> 16);
}

ORC_EXPORT float orc_bf16_to_f32(uint16_t b)
{
  return bits_f32((uint32_t)b << 16);
}

/* Array helpers: dtype codes follow CAIF_DataType_e
 * (include/caif/caif_data_type.h:32-48): Float32=0, Float16=2, BFloat16=3. */
ORC_EXPORT void orc_round_through(float *x, int64_t n, int dtype)
{
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
  {
    if (dtype == 2)
    {
      x[i] = orc_f16_to_f32(orc_f32_to_f16(x[i]));
    }
    else if (dtype == 3)
    {
      x[i] = orc_bf16_to_f32(orc_f32_to_bf16(x[i]));
    }
  }
}

ORC_EXPORT void orc_f32_to_f16_array(const float *x, uint16_t *y, int64_t n)
{
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
  {
    y[i] = orc_f32_to_f16(x[i]);
  }
}

ORC_EXPORT void orc_f32_to_bf16_array(const float *x, uint16_t *y, int64_t n)
{
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
  {
    y[i] = orc_f32_to_bf16(x[i]);
  }
}

ORC_EXPORT void orc_f16_to_f32_array(const uint16_t *x, float *y, int64_t n)
{
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
  {
    y[i] = orc_f16_to_f32(x[i]);
  }
}

ORC_EXPORT void orc_bf16_to_f32_array(const uint16_t *x, float *y, int64_t n)
{
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
  {
    y[i] = orc_bf16_to_f32(x[i]);
  }
}

/* CUDA's float->integer conversion maps NaN to 0; plain C leaves it undefined. */
static inline int rint_to_int(float v)
{
  if (v != v)
  {
    return 0;
  }
  return (int)rintf(v);
}

static inline float clamp_sym(float v, float lim)
{
  if (v > lim)
  {
    return lim;
  }
  if (v < -lim)
  {
    return -lim;
  }
  return v; /* NaN falls through both comparisons, as on the device */
}

/* ------------------------------------------------------------------------- */
/* INT8 per-tensor: src/caif_cuda_kernels_quant.cu:384-443 (scale = max|x|/127,
 * 1.0 when the tensor is all zero; q = rintf(clamp(x * (1/s), +-127))).     */
/* The device max-reduce is an atomicMax over the bit patterns of            */
/* non-negative floats, which equals the plain maximum; NaNs never win.      */
/* ------------------------------------------------------------------------- */
ORC_EXPORT void orc_quantize_int8_per_tensor(const float *x, int64_t n, int8_t *q, float *scale)
{
  if (n <= 0)
  {
    return;
  }
  float max_abs = 0.0f;
#pragma omp parallel for reduction(max : max_abs) schedule(static)
  for (int64_t i = 0; i < n; ++i)
  {
    const float v = fabsf(x[i]);
    if (v > max_abs)
    {
      max_abs = v;
    }
  }
  float s = 1.0f;
  if (max_abs > 0.0f)
  {
    s = max_abs / 127.0f;
  }
  scale[0] = s;
  float inv_s = 0.0f;
  if (s > 0.0f)
  {
    inv_s = 1.0f / s;
  }
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
  {
    const float v = clamp_sym(x[i] * inv_s, 127.0f);
    q[i] = (int8_t)rint_to_int(v);
  }
}

/* src/caif_cuda_kernels_quant.cu:446-455 */
ORC_EXPORT void orc_dequantize_int8_per_tensor(const int8_t *q, int64_t n, const float *scale, float *out)
{
  const float s = scale[0];
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
  {
    out[i] = (float)q[i] * s;
  }
}

/* ------------------------------------------------------------------------- */
/* INT8 per-channel: src/caif_cuda_kernels_quant.cu:502-574.  The channel is */
/* the LAST axis of a [rows, cols] matrix: scale index = flat index % cols.  */
/* ------------------------------------------------------------------------- */
ORC_EXPORT void orc_quantize_int8_per_channel(const float *x, int rows, int cols, int8_t *q, float *scales)
{
  if (rows <= 0 || cols <= 0)
  {
    return;
  }
#pragma omp parallel for schedule(static)
  for (int c = 0; c < cols; ++c)
  {
    float max_abs = 0.0f;
    for (int r = 0; r < rows; ++r)
    {
      const float v = fabsf(x[(int64_t)r * cols + c]);
      if (v > max_abs)
      {
        max_abs = v;
      }
    }
    scales[c] = (max_abs > 0.0f) ? (max_abs / 127.0f) : 1.0f;
  }
  const int64_t total = (int64_t)rows * cols;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < total; ++i)
  {
    const float s = scales[i % cols];
    float inv_s = 0.0f;
    if (s > 0.0f)
    {
      inv_s = 1.0f / s;
    }
    q[i] = (int8_t)rint_to_int(clamp_sym(x[i] * inv_s, 127.0f));
  }
}

ORC_EXPORT void orc_dequantize_int8_per_channel(const int8_t *q, int rows, int cols, const float *scales, float *out)
{
  const int64_t total = (int64_t)rows * cols;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < total; ++i)
  {
    out[i] = (float)q[i] * scales[i % cols];
  }
}

/* ------------------------------------------------------------------------- */
/* INT4 per-group: src/caif_cuda_kernels_quant.cu:258-342.                   */
/* Groups run over the FLAT element index.  scale = max|x|/7 in fp32 (0 for  */
/* an all-zero group), stored as fp16; the reciprocal uses the UNROUNDED     */
/* fp32 scale.  Two codes per byte, even index in the low nibble; the byte   */
/* index is i/2 with i stepping from the group start, and a lone last        */
/* element gets a zero high nibble.                                           */
/* ------------------------------------------------------------------------- */
ORC_EXPORT void orc_quantize_int4(const float *x, int64_t n, int group, uint8_t *packed, uint16_t *scales)
{
  if (n <= 0)
  {
    return;
  }
  const int64_t num_groups = (n + group - 1) / group;
  /* groups of even size write disjoint bytes and may run in parallel; an odd
   * group size makes neighbouring groups share a byte, where the device result
   * depends on thread timing -- keep that case serial (later group wins). */
#pragma omp parallel for schedule(static) if ((group & 1) == 0)
  for (int64_t g = 0; g < num_groups; ++g)
  {
    const int64_t start = g * group;
    int64_t end = start + group;
    if (end > n)
    {
      end = n;
    }
    float max_abs = 0.0f;
    for (int64_t i = start; i < end; ++i)
    {
      const float a = fabsf(x[i]);
      if (a > max_abs)
      {
        max_abs = a;
      }
    }
    float scale = 0.0f;
    if (max_abs != 0.0f)
    {
      scale = max_abs / 7.0f;
    }
    scales[g] = orc_f32_to_f16(scale);
    float inv = 0.0f;
    if (scale != 0.0f)
    {
      inv = 1.0f / scale;
    }
    for (int64_t i = start; i < end; i += 2)
    {
      const int q0 = rint_to_int(clamp_sym(x[i] * inv, 7.0f)) & 0xF;
      int q1 = 0;
      if (i + 1 < end)
      {
        q1 = rint_to_int(clamp_sym(x[i + 1] * inv, 7.0f)) & 0xF;
      }
      packed[i / 2] = (uint8_t)(q0 | (q1 << 4));
    }
  }
}

/* src/caif_cuda_kernels_quant.cu:205-237 */
ORC_EXPORT void orc_dequantize_int4(const uint8_t *packed, const uint16_t *scales, int64_t n, int group, float *out)
{
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
  {
    const uint8_t b = packed[i / 2];
    int v = (i & 1) ? ((b >> 4) & 0xF) : (b & 0xF);
    if (v & 0x8)
    {
      v |= (int)0xFFFFFFF0;
    }
    out[i] = (float)v * orc_f16_to_f32(scales[i / group]);
  }
}

/* ------------------------------------------------------------------------- */
/* Plain casts: src/caif_cuda_kernels_quant.cu:118-175 (fp32 <-> int8 with   */
/* clamp to +-127 and rintf), the path an INT8 weight without scales takes   */
/* (src/caif_device_frozen_linear.cpp:373-375).                              */
/* ------------------------------------------------------------------------- */
ORC_EXPORT void orc_cast_f32_to_int8(const float *x, int64_t n, int8_t *q)
{
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
  {
    q[i] = (int8_t)rint_to_int(clamp_sym(x[i], 127.0f));
  }
}

ORC_EXPORT void orc_cast_int8_to_f32(const int8_t *q, int64_t n, float *out)
{
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
  {
    out[i] = (float)q[i];
  }
}

/* ------------------------------------------------------------------------- */
/* Weight materialisation: CAIF_DeviceFrozenLinear::ConvertToComputeDtype,   */
/* src/caif_device_frozen_linear.cpp:288-378.  Produces the [out,in] matrix  */
/* the GEMM consumes, as fp32 values already rounded through the compute     */
/* dtype (0 fp32, 2 fp16, 3 bf16).  storage: 0 fp32, 2 fp16, 3 bf16, 4 int4, */
/* 5 int8.  scheme: 0 per-tensor, 1 per-channel (scale index = flat % out,   */
/* because the device call passes rows=in, cols=out, :356-361).              */
/* scales==NULL with int8 storage is the raw integer cast.                   */
/* ------------------------------------------------------------------------- */
ORC_EXPORT int orc_weight_to_compute(const void *codes, const void *scales, int storage, int scheme, int group,
                                     int in_dim, int out_dim, int compute, float *w)
{
  const int64_t total = (int64_t)in_dim * out_dim;
  switch (storage)
  {
    case 0:
      memcpy(w, codes, (size_t)total * 4);
      break;
    case 2:
      orc_f16_to_f32_array((const uint16_t *)codes, w, total);
      break;
    case 3:
      orc_bf16_to_f32_array((const uint16_t *)codes, w, total);
      break;
    case 4:
      if (scales == NULL)
      {
        return -1;
      }
      orc_dequantize_int4((const uint8_t *)codes, (const uint16_t *)scales, total, group, w);
      break;
    case 5:
      if (scales == NULL)
      {
        orc_cast_int8_to_f32((const int8_t *)codes, total, w);
      }
      else if (scheme == 0)
      {
        orc_dequantize_int8_per_tensor((const int8_t *)codes, total, (const float *)scales, w);
      }
      else
      {
        orc_dequantize_int8_per_channel((const int8_t *)codes, in_dim, out_dim, (const float *)scales, w);
      }
      break;
    default:
      return -2;
  }
  if (compute != storage)
  {
    orc_round_through(w, total, compute);
  }
  return 0;
}

/* ------------------------------------------------------------------------- */
/* GEMMs of the layer, fp32 operands, fp64 accumulation (a tie-breaker that  */
/* is more exact than any fp32 library order):                               */
/*   forward  Y[m,out] = X[m,in] . W[out,in]^T   (frozen_linear.cpp:445-509) */
/*   backward dX[m,in] = dY[m,out] . W[out,in]   (frozen_linear.cpp:591-641) */
/* ------------------------------------------------------------------------- */
ORC_EXPORT void orc_gemm_nt(const float *x, const float *w, float *y, int m, int n, int k)
{
#pragma omp parallel for collapse(2) schedule(static)
  for (int i = 0; i < m; ++i)
  {
    for (int j = 0; j < n; ++j)
    {
      const float *a = x + (int64_t)i * k;
      const float *b = w + (int64_t)j * k;
      double acc = 0.0;
      for (int p = 0; p < k; ++p)
      {
        acc += (double)a[p] * (double)b[p];
      }
      y[(int64_t)i * n + j] = (float)acc;
    }
  }
}

ORC_EXPORT void orc_gemm_nn(const float *a, const float *b, float *c, int m, int n, int k)
{
  /* c[m,n] = a[m,k] . b[k,n] */
#pragma omp parallel for schedule(static)
  for (int i = 0; i < m; ++i)
  {
    double *acc = (double *)calloc((size_t)n, sizeof(double));
    for (int p = 0; p < k; ++p)
    {
      const double av = (double)a[(int64_t)i * k + p];
      const float *brow = b + (int64_t)p * n;
      for (int j = 0; j < n; ++j)
      {
        acc[j] += av * (double)brow[j];
      }
    }
    for (int j = 0; j < n; ++j)
    {
      c[(int64_t)i * n + j] = (float)acc[j];
    }
    free(acc);
  }
}

ORC_EXPORT void orc_gemm_tn(const float *a, const float *b, float *c, int m, int n, int k)
{
  /* c[m,n] = a[k,m]^T . b[k,n]  (MatMulTransposeA, used for dA and dB) */
#pragma omp parallel for schedule(static)
  for (int i = 0; i < m; ++i)
  {
    double *acc = (double *)calloc((size_t)n, sizeof(double));
    for (int p = 0; p < k; ++p)
    {
      const double av = (double)a[(int64_t)p * m + i];
      const float *brow = b + (int64_t)p * n;
      for (int j = 0; j < n; ++j)
      {
        acc[j] += av * (double)brow[j];
      }
    }
    for (int j = 0; j < n; ++j)
    {
      c[(int64_t)i * n + j] = (float)acc[j];
    }
    free(acc);
  }
}

/* ------------------------------------------------------------------------- */
/* Routing.                                                                  */
/* ------------------------------------------------------------------------- */

/* Top-k per row: src/caif_cuda_kernels_moe.cu:280-334.  Values are compared */
/* as fp32 with strict '>' scanning upward from index 0 against a -1e30      */
/* sentinel, so ties go to the lowest index and a row of values <= -1e30     */
/* yields index 0 repeatedly.                                                 */
ORC_EXPORT void orc_topk(const float *input, int batch, int dim, int k, int32_t *indices, float *values)
{
#pragma omp parallel for schedule(static)
  for (int b = 0; b < batch; ++b)
  {
    float *temp = (float *)malloc((size_t)dim * sizeof(float));
    memcpy(temp, input + (int64_t)b * dim, (size_t)dim * sizeof(float));
    for (int i = 0; i < k; ++i)
    {
      float max_val = -1e30f;
      int max_idx = 0;
      for (int d = 0; d < dim; ++d)
      {
        if (temp[d] > max_val)
        {
          max_val = temp[d];
          max_idx = d;
        }
      }
      indices[(int64_t)b * k + i] = max_idx;
      values[(int64_t)b * k + i] = max_val;
      temp[max_idx] = -1e30f;
    }
    free(temp);
  }
}

/* Row normalisation: src/caif_cuda_kernels_moe.cu:43-85.  Block of 256      */
/* threads: thread t sums elements t, t+256, ... in order, then a binary     */
/* tree over shared memory (stride 128 .. 1); the divisor is max(sum,1e-10)  */
/* and each element is multiplied by its fp32 reciprocal.                    */
ORC_EXPORT void orc_normalize_rows(const float *input, int batch, int dim, float *output)
{
#pragma omp parallel for schedule(static)
  for (int b = 0; b < batch; ++b)
  {
    float s[256];
    const float *row = input + (int64_t)b * dim;
    for (int t = 0; t < 256; ++t)
    {
      float local = 0.0f;
      for (int d = t; d < dim; d += 256)
      {
        local += row[d];
      }
      s[t] = local;
    }
    for (int stride = 128; stride > 0; stride >>= 1)
    {
      for (int t = 0; t < stride; ++t)
      {
        s[t] += s[t + stride];
      }
    }
    const float sum = fmaxf(s[0], 1e-10f);
    const float inv = 1.0f / sum;
    for (int d = 0; d < dim; ++d)
    {
      output[(int64_t)b * dim + d] = row[d] * inv;
    }
  }
}

/* Router softmax: launch_attention_softmax,                                   */
/* src/caif_cuda_kernels_attention_support.cu:350-460, 866-884 (128 threads  */
/* per row on every architecture the selection table knows, :53-83).  Thread */
/* t scans columns t, t+128, ... with the online (max, sum) update; each     */
/* warp of 32 threads folds its values with an xor butterfly (offsets 16..1);*/
/* the four warp results are folded in lanes 0..3 with offsets 2 and 1; then */
/* y = expf(x - max) * (1 / sum).  With a bias (CAIF_Ops::AddBias,           */
/* src/caif_cuda_kernels_elementwise.cu:124-137, ahead of the softmax in     */
/* src/caif_device_moe_router.cpp:233-243) the value seen is the sum rounded */
/* through `dtype`.  expf here is the host libm's: the order of operations   */
/* is the kernel's, the last bits of expf need not be.                       */
static void orc_softmax_absorb(float *m, float *s, float m_other, float s_other)
{
  if (m_other > *m)
  {
    *s = *s * expf(*m - m_other) + s_other;
    *m = m_other;
  }
  else
  {
    *s += s_other * expf(m_other - *m);
  }
}

ORC_EXPORT void orc_router_softmax(const float *logits, const float *bias, int rows, int cols, int dtype, float *probs)
{
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r)
  {
    const float *x = logits + (int64_t)r * cols;
    float m[128];
    float s[128];
    float *v = (float *)malloc((size_t)cols * sizeof(float));
    for (int c = 0; c < cols; ++c)
    {
      v[c] = x[c];
      if (bias != NULL)
      {
        v[c] = x[c] + bias[c];
        orc_round_through(&v[c], 1, dtype);
      }
    }
    for (int t = 0; t < 128; ++t)
    {
      m[t] = -1e30f;
      s[t] = 0.0f;
      for (int c = t; c < cols; c += 128)
      {
        if (v[c] > m[t])
        {
          s[t] = s[t] * expf(m[t] - v[c]) + 1.0f;
          m[t] = v[c];
        }
        else
        {
          s[t] += expf(v[c] - m[t]);
        }
      }
    }
    for (int w = 0; w < 4; ++w)
    {
      for (int off = 16; off > 0; off >>= 1)
      {
        float nm[32];
        float ns[32];
        for (int l = 0; l < 32; ++l)
        {
          nm[l] = m[32 * w + l];
          ns[l] = s[32 * w + l];
          orc_softmax_absorb(&nm[l], &ns[l], m[32 * w + (l ^ off)], s[32 * w + (l ^ off)]);
        }
        for (int l = 0; l < 32; ++l)
        {
          m[32 * w + l] = nm[l];
          s[32 * w + l] = ns[l];
        }
      }
    }
    {
      float fm[4] = {m[0], m[32], m[64], m[96]};
      float fs[4] = {s[0], s[32], s[64], s[96]};
      orc_softmax_absorb(&fm[0], &fs[0], fm[2], fs[2]);
      orc_softmax_absorb(&fm[1], &fs[1], fm[3], fs[3]);
      orc_softmax_absorb(&fm[0], &fs[0], fm[1], fs[1]);
      const float inv = 1.0f / fs[0];
      for (int c = 0; c < cols; ++c)
      {
        probs[(int64_t)r * cols + c] = expf(v[c] - fm[0]) * inv;
      }
    }
    free(v);
  }
}

/* Router backward up to grad_logits: CAIF_DeviceMoERouter::BackwardRoutingAuxAware,   */
/* src/caif_device_moe_router.cpp:529-733, as the chain of kernels it launches, every   */
/* intermediate rounded through `dtype` where the reference stores a tensor:            */
/*  1. normalize Jacobian over the chosen scores (src/caif_cuda_kernels_moe.cu:128-171):*/
/*     32 lanes, lane k < top_k holding p_k and g_k, sums by xor butterfly 16..1,       */
/*     s = max(sum p, 1e-12), inv = 1/s, dot = sum (p_k inv) g_k, out = (g_k - dot) inv */
/*  2. Scale by routed_scaling_factor when it is not 1                                  */
/*  3. Zeros + ScatterAdd to [tokens, experts] (:553-572)                               */
/*  4. sigmoid gating: g * p * (1 - p) (src/caif_cuda_kernels_activations.cu:189-228)   */
/*     softmax gating: AddBias of balance_bias (src/caif_cuda_kernels_elementwise.cu:   */
/*     124-137), then attention_softmax_backward_kernel                                 */
/*     (src/caif_cuda_kernels_attention_support.cu:464-530) called with (probs,         */
/*     grad_probs) in its (grad_output, output) slots (router.cpp:702): 128 threads,    */
/*     thread t accumulating columns t, t+128, ... with a fused multiply-add, a         */
/*     butterfly per warp, (w0 + w2) + (w1 + w3) across the warps, then                 */
/*     dx = y (dy - dot) with y = grad_probs, dy = probs; exact_jacobian != 0 swaps     */
/*     them into the softmax Jacobian proper.  Then the z-loss term                     */
/*     fma(lse_scaled[t], p, dx) (src/caif_cuda_kernels_moe.cu:1376-1395).              */
static float orc_butterfly_sum(float *lanes)
{
  for (int off = 16; off > 0; off >>= 1)
  {
    float next[32];
    for (int l = 0; l < 32; ++l)
    {
      next[l] = lanes[l] + lanes[l ^ off];
    }
    memcpy(lanes, next, sizeof(next));
  }
  return lanes[0];
}

static float orc_round1(float v, int dtype)
{
  orc_round_through(&v, 1, dtype);
  return v;
}

ORC_EXPORT void orc_router_backward(const float *grad_w, const float *probs, const int32_t *indices,
                                    const float *balance_bias, const float *z_lse_scaled, int tokens, int experts,
                                    int top_k, int sigmoid_gate, int normalize, float scaling, int exact_jacobian,
                                    int dtype, float *grad_topk, float *grad_logits)
{
#pragma omp parallel for schedule(static)
  for (int t = 0; t < tokens; ++t)
  {
    const float *p_row = probs + (int64_t)t * experts;
    float *gp = (float *)calloc((size_t)experts, sizeof(float));
    float gt[32];
    float lanes[32];
    float pk[32];
    for (int k = 0; k < 32; ++k)
    {
      const int idx = k < top_k ? indices[(int64_t)t * top_k + k] : -1;
      pk[k] = (k < top_k && idx >= 0 && idx < experts) ? p_row[idx] : 0.0f;
      gt[k] = k < top_k ? grad_w[(int64_t)t * top_k + k] : 0.0f;
    }
    if (normalize)
    {
      memcpy(lanes, pk, sizeof(lanes));
      const float sum = fmaxf(orc_butterfly_sum(lanes), 1e-12f);
      const float inv = 1.0f / sum;
      for (int k = 0; k < 32; ++k)
      {
        lanes[k] = (pk[k] * inv) * gt[k];
      }
      const float dot = orc_butterfly_sum(lanes);
      for (int k = 0; k < top_k; ++k)
      {
        gt[k] = orc_round1((gt[k] - dot) * inv, dtype);
      }
    }
    for (int k = 0; k < top_k; ++k)
    {
      if (scaling != 1.0f)
      {
        gt[k] = orc_round1(gt[k] * scaling, dtype);
      }
      if (grad_topk != NULL)
      {
        grad_topk[(int64_t)t * top_k + k] = gt[k];
      }
      const int idx = indices[(int64_t)t * top_k + k];
      if (idx >= 0 && idx < experts)
      {
        gp[idx] = orc_round1(gp[idx] + gt[k], dtype);
      }
    }
    float *out = grad_logits + (int64_t)t * experts;
    if (sigmoid_gate)
    {
      for (int c = 0; c < experts; ++c)
      {
        out[c] = orc_round1((gp[c] * p_row[c]) * (1.0f - p_row[c]), dtype);
      }
      free(gp);
      continue;
    }
    if (balance_bias != NULL)
    {
      for (int c = 0; c < experts; ++c)
      {
        gp[c] = orc_round1(gp[c] + balance_bias[c], dtype);
      }
    }
    float warp_sum[4];
    for (int w = 0; w < 4; ++w)
    {
      for (int l = 0; l < 32; ++l)
      {
        float acc = 0.0f;
        for (int c = 32 * w + l; c < experts; c += 128)
        {
          acc = fmaf(p_row[c], gp[c], acc);
        }
        lanes[l] = acc;
      }
      warp_sum[w] = orc_butterfly_sum(lanes);
    }
    const float dot = (warp_sum[0] + warp_sum[2]) + (warp_sum[1] + warp_sum[3]);
    for (int c = 0; c < experts; ++c)
    {
      const float y = exact_jacobian ? p_row[c] : gp[c];
      const float dy = exact_jacobian ? gp[c] : p_row[c];
      float v = orc_round1(y * (dy - dot), dtype);
      if (z_lse_scaled != NULL)
      {
        v = orc_round1(fmaf(z_lse_scaled[t], p_row[c], v), dtype);
      }
      out[c] = v;
    }
    free(gp);
  }
}

/* Auxiliary losses of CAIF_DeviceMoELayer, src/caif_device_moe_layer.cpp:792-835 and   */
/* 853-925.  logsumexp_kernel (src/caif_cuda_kernels_elementwise.cu:930-990): 256       */
/* threads, thread t over columns t, t+256, ...; max, then sum of expf(x - max), both   */
/* through the shared-memory tree (strides 128 ... 1); lse = max + logf(sum), stored    */
/* through `dtype`.  z loss = zw * T(sum_t T(lse_t^2)) / tokens; z_lse_scaled =         */
/* T(lse * (2 zw / tokens)).  Balance loss = bw * E * sum_e (count_e / (tokens k)) *    */
/* (T(sum_t probs[t,e]) / tokens) with the column sums added sequentially over t        */
/* (sum_axis0_kernel, :800-816); balance_bias[e] = T(bw E / (tokens^2 k) * count_e).    */
/* losses[0] = balance, losses[1] = z.  logits or probs may be NULL.                    */
/* The z loss here sums over ALL tokens.  The executing reference reduces with           */
/* launch_reduction_sum, one partial per 256-element block stored into a one-element     */
/* tensor (:450-493 of the elementwise kernels, moe_layer.cpp:911-913), so for more than */
/* 256 tokens it reports the first block's partial; tests/test_moe_layer_reference.py    */
/* reproduces that figure from the first 256 rows of this function's lse.                */
ORC_EXPORT void orc_moe_aux_losses(const float *logits, const float *probs, const int32_t *counts, int tokens,
                                   int experts, int top_k, float balance_weight, float z_weight, int dtype,
                                   float *balance_bias, float *lse, float *z_lse_scaled, float *losses)
{
  losses[0] = 0.0f;
  losses[1] = 0.0f;
  if (probs != NULL)
  {
    const float total = (float)tokens * (float)top_k;
    float loss = 0.0f;
    for (int e = 0; e < experts; ++e)
    {
      float sum = 0.0f;
      for (int t = 0; t < tokens; ++t)
      {
        sum += probs[(int64_t)t * experts + e];
      }
      const float mean_p = orc_round1(sum, dtype) / (float)tokens;
      loss += ((float)counts[e] / total) * mean_p;
    }
    losses[0] = balance_weight * (float)experts * loss;
    if (balance_bias != NULL)
    {
      const float denom = (float)tokens * (float)tokens * (float)top_k;
      const float scale = balance_weight * (float)experts / denom;
      for (int e = 0; e < experts; ++e)
      {
        balance_bias[e] = orc_round1(scale * (float)counts[e], dtype);
      }
    }
  }
  if (logits != NULL)
  {
    const float z_scale = 2.0f * z_weight / (float)tokens;
    float total = 0.0f;
    for (int t = 0; t < tokens; ++t)
    {
      const float *x = logits + (int64_t)t * experts;
      float smax[256];
      float ssum[256];
      for (int i = 0; i < 256; ++i)
      {
        smax[i] = -1e30f;
        for (int c = i; c < experts; c += 256)
        {
          smax[i] = fmaxf(smax[i], x[c]);
        }
      }
      for (int stride = 128; stride > 0; stride >>= 1)
      {
        for (int i = 0; i < stride; ++i)
        {
          smax[i] = fmaxf(smax[i], smax[i + stride]);
        }
      }
      const float m = smax[0];
      for (int i = 0; i < 256; ++i)
      {
        ssum[i] = 0.0f;
        for (int c = i; c < experts; c += 256)
        {
          ssum[i] += expf(x[c] - m);
        }
      }
      for (int stride = 128; stride > 0; stride >>= 1)
      {
        for (int i = 0; i < stride; ++i)
        {
          ssum[i] += ssum[i + stride];
        }
      }
      const float l = orc_round1(m + logf(ssum[0]), dtype);
      if (lse != NULL)
      {
        lse[t] = l;
      }
      if (z_lse_scaled != NULL)
      {
        z_lse_scaled[t] = orc_round1(l * z_scale, dtype);
      }
      total += orc_round1(l * l, dtype);
    }
    losses[1] = z_weight * orc_round1(total, dtype) / (float)tokens;
  }
}

/* RMSNorm, src/caif_cuda_kernels_normalization.cu:46-119 (forward) and 129-203          */
/* (backward): one block of 256 threads per row, thread t over columns t, t+256, ...    */
/* with a fused multiply-add per step; warp_reduce_sum is a shuffle-DOWN tree (offsets  */
/* 16..1; a lane whose partner is out of range adds its own value, only lane 0 is used);*/
/* the eight warp sums sit in lanes 0..7 of warp 0 and go through the same tree.        */
/* rms = sqrtf(sum / dim + eps); y = T((x * (1 / rms)) * gamma).  Backward:             */
/* sum_term = sum((dy * gamma) * x_hat) / dim with x_hat = x * rstd;                    */
/* dx = T(rstd * (dy * gamma - x_hat * sum_term)), the inner expression fused as the    */
/* reference build fuses it (`form` 0, pinned on the GPU against its kernel:             */
/* fma(dy, gamma, -(x_hat sum_term));                                                   */
/* 1 fma(-x_hat, sum_term, dy gamma), 2 unfused); grad_gamma[c] = sum_r dy * x_hat      */
/* in row order (the reference's atomics fix no order).                                 */
static float orc_shfl_down_tree(const float *lanes32)
{
  float v[32];
  memcpy(v, lanes32, sizeof(v));
  for (int off = 16; off > 0; off >>= 1)
  {
    float n[32];
    for (int l = 0; l < 32; ++l)
    {
      n[l] = v[l] + (l + off < 32 ? v[l + off] : v[l]);
    }
    memcpy(v, n, sizeof(v));
  }
  return v[0];
}

static float orc_block256_sum(const float *thread_vals)
{
  float warp[32];
  memset(warp, 0, sizeof(warp));
  for (int w = 0; w < 8; ++w)
  {
    warp[w] = orc_shfl_down_tree(thread_vals + 32 * w);
  }
  return orc_shfl_down_tree(warp);
}

ORC_EXPORT void orc_rmsnorm_forward(const float *x, const float *gamma, int rows, int dim, float eps, int dtype,
                                    float *y, float *rms_out)
{
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r)
  {
    const float *xr = x + (int64_t)r * dim;
    float t[256];
    for (int i = 0; i < 256; ++i)
    {
      t[i] = 0.0f;
      for (int c = i; c < dim; c += 256)
      {
        t[i] = fmaf(xr[c], xr[c], t[i]);
      }
    }
    const float rms = sqrtf(orc_block256_sum(t) / (float)dim + eps);
    rms_out[r] = rms;
    const float rstd = 1.0f / rms;
    for (int c = 0; c < dim; ++c)
    {
      y[(int64_t)r * dim + c] = orc_round1((xr[c] * rstd) * gamma[c], dtype);
    }
  }
}

ORC_EXPORT void orc_rmsnorm_backward(const float *dy, const float *x, const float *gamma, const float *rms, int rows,
                                     int dim, int dtype, int form, float *dx, float *grad_gamma)
{
  memset(grad_gamma, 0, (size_t)dim * sizeof(float));
  for (int r = 0; r < rows; ++r)
  {
    const float *xr = x + (int64_t)r * dim;
    const float *gr = dy + (int64_t)r * dim;
    const float rstd = 1.0f / rms[r];
    float t[256];
    for (int i = 0; i < 256; ++i)
    {
      t[i] = 0.0f;
      for (int c = i; c < dim; c += 256)
      {
        t[i] = fmaf(gr[c] * gamma[c], xr[c] * rstd, t[i]);
      }
    }
    const float sum_term = orc_block256_sum(t) / (float)dim;
    for (int c = 0; c < dim; ++c)
    {
      const float x_hat = xr[c] * rstd;
      float inner;
      if (form == 0)
      {
        inner = fmaf(gr[c], gamma[c], -(x_hat * sum_term));
      }
      else if (form == 1)
      {
        inner = fmaf(-x_hat, sum_term, gr[c] * gamma[c]);
      }
      else
      {
        inner = gr[c] * gamma[c] - x_hat * sum_term;
      }
      dx[(int64_t)r * dim + c] = orc_round1(rstd * inner, dtype);
      grad_gamma[c] += gr[c] * x_hat;
    }
  }
}

/* Dispatch map: CAIF_Ops::MoEBuildDispatchMapDevice,                        */
/* src/caif_ops_device.cpp:4876-4950.  counts per expert (indices outside    */
/* [0,E) ignored) -> capacity clamp -> exclusive prefix sum -> position of   */
/* each (token,k) within its expert in token-major, k-minor arrival order,   */
/* -1 when the expert is already at capacity.  Returns the total assigned.   */
ORC_EXPORT int32_t orc_build_dispatch_map(const int32_t *expert_indices, int num_tokens, int top_k, int num_experts,
                                          int capacity, int32_t *dispatch_map, int32_t *expert_offsets)
{
  uint32_t *counts = (uint32_t *)calloc((size_t)num_experts, sizeof(uint32_t));
  uint32_t *positions = (uint32_t *)calloc((size_t)num_experts, sizeof(uint32_t));
  const int64_t total = (int64_t)num_tokens * top_k;
  for (int64_t i = 0; i < total; ++i)
  {
    const int32_t e = expert_indices[i];
    if (e >= 0 && e < num_experts)
    {
      ++counts[e];
    }
  }
  expert_offsets[0] = 0;
  for (int e = 0; e < num_experts; ++e)
  {
    if (capacity > 0 && counts[e] > (uint32_t)capacity)
    {
      counts[e] = (uint32_t)capacity;
    }
    expert_offsets[e + 1] = expert_offsets[e] + (int32_t)counts[e];
  }
  for (int64_t i = 0; i < total; ++i)
  {
    dispatch_map[i] = -1;
    const int32_t e = expert_indices[i];
    if (e >= 0 && e < num_experts)
    {
      if (positions[e] < counts[e])
      {
        dispatch_map[i] = (int32_t)positions[e];
        ++positions[e];
      }
    }
  }
  const int32_t assigned = expert_offsets[num_experts];
  free(counts);
  free(positions);
  return assigned;
}

/* Gather into the packed per-expert buffer: src/caif_cuda_kernels_moe.cu:616-647. */
ORC_EXPORT void orc_moe_dispatch(const float *input, const int32_t *expert_indices, const int32_t *dispatch_map,
                                 const int32_t *expert_offsets, int num_tokens, int dim, int top_k, float *buffer)
{
  for (int t = 0; t < num_tokens; ++t)
  {
    for (int k = 0; k < top_k; ++k)
    {
      const int32_t e = expert_indices[(int64_t)t * top_k + k];
      const int32_t pos = dispatch_map[(int64_t)t * top_k + k];
      if (e >= 0 && pos >= 0)
      {
        memcpy(buffer + ((int64_t)expert_offsets[e] + pos) * dim, input + (int64_t)t * dim, (size_t)dim * 4);
      }
    }
  }
}

/* Weighted combine: src/caif_cuda_kernels_moe.cu:705-745.  fp32 accumulate  */
/* over k in order (separate multiply and add are contracted to an FMA by    */
/* the device compiler: sum = fma(w, v, sum)), one rounding to the storage   */
/* dtype by the caller.                                                       */
ORC_EXPORT void orc_moe_combine(const float *buffer, const int32_t *expert_indices, const float *weights,
                                const int32_t *dispatch_map, const int32_t *expert_offsets, int num_tokens, int dim,
                                int top_k, float *output)
{
#pragma omp parallel for schedule(static)
  for (int t = 0; t < num_tokens; ++t)
  {
    for (int d = 0; d < dim; ++d)
    {
      float sum = 0.0f;
      for (int k = 0; k < top_k; ++k)
      {
        const int32_t e = expert_indices[(int64_t)t * top_k + k];
        const int32_t pos = dispatch_map[(int64_t)t * top_k + k];
        if (e >= 0 && pos >= 0)
        {
          const float v = buffer[((int64_t)expert_offsets[e] + pos) * dim + d];
          sum = fmaf(weights[(int64_t)t * top_k + k], v, sum);
        }
      }
      output[(int64_t)t * dim + d] = sum;
    }
  }
}

/* Backward of the combine, packed-buffer gradient: src/caif_cuda_kernels_moe.cu:816-847.  */
/* Every assigned slot gets w * g (one fp32 product, rounded to the storage dtype by the     */
/* caller); unassigned slots of the buffer are not written.                                   */
ORC_EXPORT void orc_moe_combine_bwd_grad_expert(const float *grad_output, const int32_t *expert_indices,
                                                const float *weights, const int32_t *dispatch_map,
                                                const int32_t *expert_offsets, int num_tokens, int dim, int top_k,
                                                float *grad_buffer)
{
  for (int t = 0; t < num_tokens; ++t)
  {
    for (int k = 0; k < top_k; ++k)
    {
      const int32_t e = expert_indices[(int64_t)t * top_k + k];
      const int32_t pos = dispatch_map[(int64_t)t * top_k + k];
      if (e >= 0 && pos >= 0)
      {
        const float w = weights[(int64_t)t * top_k + k];
        float *dst = grad_buffer + ((int64_t)expert_offsets[e] + pos) * dim;
        for (int d = 0; d < dim; ++d)
        {
          dst[d] = w * grad_output[(int64_t)t * dim + d];
        }
      }
    }
  }
}

/* Backward of the combine, routing-weight gradient: src/caif_cuda_kernels_moe.cu:925-972.   */
/* One 256-thread block per (token, k): thread i adds g*b for d = i, i+256, ... (the device    */
/* compiler contracts the multiply-add to an FMA), then a halving tree over the 256 partials. */
ORC_EXPORT void orc_moe_combine_bwd_grad_weights(const float *grad_output, const float *buffer,
                                                 const int32_t *expert_indices, const int32_t *dispatch_map,
                                                 const int32_t *expert_offsets, int num_tokens, int dim, int top_k,
                                                 float *grad_weights)
{
#pragma omp parallel for schedule(static)
  for (int a = 0; a < num_tokens * top_k; ++a)
  {
    const int t = a / top_k;
    const int32_t e = expert_indices[a];
    const int32_t pos = dispatch_map[a];
    float part[256];
    for (int i = 0; i < 256; ++i)
    {
      part[i] = 0.0f;
    }
    if (e >= 0 && pos >= 0)
    {
      const float *src = buffer + ((int64_t)expert_offsets[e] + pos) * dim;
      const float *g = grad_output + (int64_t)t * dim;
      for (int i = 0; i < 256; ++i)
      {
        for (int d = i; d < dim; d += 256)
        {
          part[i] = fmaf(g[d], src[d], part[i]);
        }
      }
    }
    for (int stride = 128; stride > 0; stride >>= 1)
    {
      for (int i = 0; i < stride; ++i)
      {
        part[i] += part[i + stride];
      }
    }
    grad_weights[a] = part[0];
  }
}

/* Backward of the dispatch: src/caif_cuda_kernels_moe.cu:1040-1067.  fp32 sum over k in order. */
ORC_EXPORT void orc_moe_dispatch_bwd(const float *grad_buffer, const int32_t *expert_indices,
                                     const int32_t *dispatch_map, const int32_t *expert_offsets, int num_tokens,
                                     int dim, int top_k, float *grad_input)
{
#pragma omp parallel for schedule(static)
  for (int t = 0; t < num_tokens; ++t)
  {
    for (int d = 0; d < dim; ++d)
    {
      float sum = 0.0f;
      for (int k = 0; k < top_k; ++k)
      {
        const int32_t e = expert_indices[(int64_t)t * top_k + k];
        const int32_t pos = dispatch_map[(int64_t)t * top_k + k];
        if (e >= 0 && pos >= 0)
        {
          sum += grad_buffer[((int64_t)expert_offsets[e] + pos) * dim + d];
        }
      }
      grad_input[(int64_t)t * dim + d] = sum;
    }
  }
}

/* SiLU and its derivative: src/caif_cuda_kernels_activations.cu:513-514,558-561. */
ORC_EXPORT void orc_silu(const float *x, int64_t n, float *y)
{
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
  {
    y[i] = x[i] / (1.0f + expf(-x[i]));
  }
}

ORC_EXPORT void orc_silu_backward(const float *grad, const float *x, int64_t n, float *out)
{
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
  {
    const float s = 1.0f / (1.0f + expf(-x[i]));
    out[i] = grad[i] * (s * (1.0f + x[i] * (1.0f - s)));
  }
}

ORC_EXPORT int orc_num_threads(void)
{
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
