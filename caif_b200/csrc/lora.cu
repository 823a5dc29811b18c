// Small dense helpers of the LoRA adapter path
// (src/caif_device_lora_adapter.cpp:205-281): the two reductions over tokens,
//   dB[out, r] = (alpha/r . dY)^T . H        dA[r, in] = dH^T . X
// (CAIF_Ops::MatMulTransposeA with beta = 0: the destination is overwritten),
// and the in-place Scale.  Operands are read in the adapter's storage dtype,
// products accumulate in fp32, the result is rounded once to the storage dtype.
#include "common.cuh"

namespace caifq
{

namespace
{

constexpr int TP = 32;  // tile of C rows (columns of U)
constexpr int TQ = 32;  // tile of C columns (columns of V)
constexpr int TM = 32;  // tokens per step
constexpr int TN_THREADS = 256;
constexpr int kMaxSplits = 64;

// C[p, q] (+)= sum over a slice of m of U[m, p] * V[m, q].  gridDim.z slices the
// token range; partial tiles are combined with fp32 atomics into `acc`, which
// the caller zeroed, and a second kernel rounds acc into C.
__global__ void __launch_bounds__(TN_THREADS)
gemm_tn_kernel(const void *__restrict__ u, const void *__restrict__ v, float *__restrict__ acc, int dtype,
               int compute_dtype, float u_prescale, int64_t m, int p, int q)
{
  __shared__ float su[TM][TP + 1];
  __shared__ float sv[TM][TQ + 1];
  const int tid = threadIdx.x;
  const int p0 = blockIdx.y * TP;
  const int q0 = blockIdx.x * TQ;
  const int64_t per = (m + gridDim.z - 1) / gridDim.z;
  const int64_t m_begin = per * blockIdx.z;
  const int64_t m_end = (m_begin + per < m) ? (m_begin + per) : m;
  const int tq = tid % 16;  // 2 columns each
  const int tp = tid / 16;  // 2 rows each
  float c[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};
  for (int64_t mb = m_begin; mb < m_end; mb += TM)
  {
    for (int e = tid; e < TM * TP; e += TN_THREADS)
    {
      const int pp = e % TP;
      const int mm = e / TP;
      float val = 0.0f;
      if (mb + mm < m_end && p0 + pp < p)
      {
        val = load_as_float(u, (mb + mm) * p + p0 + pp, dtype);
        if (u_prescale != 1.0f)
        {
          val = round_through_rt(__fmul_rn(val, u_prescale), dtype);
        }
        val = round_through_rt(val, compute_dtype);
      }
      su[mm][pp] = val;
    }
    for (int e = tid; e < TM * TQ; e += TN_THREADS)
    {
      const int qq = e % TQ;
      const int mm = e / TQ;
      float val = 0.0f;
      if (mb + mm < m_end && q0 + qq < q)
      {
        val = round_through_rt(load_as_float(v, (mb + mm) * q + q0 + qq, dtype), compute_dtype);
      }
      sv[mm][qq] = val;
    }
    __syncthreads();
#pragma unroll
    for (int mm = 0; mm < TM; ++mm)
    {
      const float u0 = su[mm][tp * 2];
      const float u1 = su[mm][tp * 2 + 1];
      const float v0 = sv[mm][tq * 2];
      const float v1 = sv[mm][tq * 2 + 1];
      c[0][0] = fmaf(u0, v0, c[0][0]);
      c[0][1] = fmaf(u0, v1, c[0][1]);
      c[1][0] = fmaf(u1, v0, c[1][0]);
      c[1][1] = fmaf(u1, v1, c[1][1]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
  {
#pragma unroll
    for (int j = 0; j < 2; ++j)
    {
      const int gp = p0 + tp * 2 + i;
      const int gq = q0 + tq * 2 + j;
      if (gp < p && gq < q)
      {
        atomicAdd(&acc[static_cast<int64_t>(gp) * q + gq], c[i][j]);
      }
    }
  }
}

__global__ void round_out_kernel(const float *__restrict__ acc, void *__restrict__ c, int dtype, int64_t n)
{
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
  {
    store_from_float(c, i, dtype, acc[i]);
  }
}

__global__ void scale_kernel(const void *__restrict__ src, void *__restrict__ dst, int dtype, float scale, int64_t n)
{
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
  {
    store_from_float(dst, i, dtype, __fmul_rn(load_as_float(src, i, dtype), scale));
  }
}

}  // namespace

// fp32 scratch the reduction needs: p*q floats.
size_t gemm_tn_scratch_bytes(int p, int q) { return static_cast<size_t>(p) * q * sizeof(float); }

int launch_gemm_tn(const void *u, const void *v, void *c, float *scratch, int dtype, int compute_dtype,
                   float u_prescale, int64_t m, int p, int q, cudaStream_t s)
{
  const int64_t n = static_cast<int64_t>(p) * q;
  if (n <= 0)
  {
    return CAIFQ_OK;
  }
  CAIFQ_CHECK_CUDA(cudaMemsetAsync(scratch, 0, static_cast<size_t>(n) * sizeof(float), s));
  if (m > 0)
  {
    const int tiles = ((p + TP - 1) / TP) * ((q + TQ - 1) / TQ);
    int64_t splits = (148 * 4 + tiles - 1) / tiles;
    const int64_t max_splits = (m + TM - 1) / TM;
    if (splits > max_splits)
    {
      splits = max_splits;
    }
    if (splits > kMaxSplits)
    {
      splits = kMaxSplits;
    }
    if (splits < 1)
    {
      splits = 1;
    }
    dim3 grid((q + TQ - 1) / TQ, (p + TP - 1) / TP, static_cast<unsigned>(splits));
    gemm_tn_kernel<<<grid, TN_THREADS, 0, s>>>(u, v, scratch, dtype, compute_dtype, u_prescale, m, p, q);
    CAIFQ_CHECK_LAUNCH();
  }
  int64_t g = (n + 255) / 256;
  if (g > 148 * 8)
  {
    g = 148 * 8;
  }
  round_out_kernel<<<static_cast<unsigned>(g), 256, 0, s>>>(scratch, c, dtype, n);
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_scale(const void *src, void *dst, int dtype, float scale, int64_t n, cudaStream_t s)
{
  if (n <= 0)
  {
    return CAIFQ_OK;
  }
  int64_t g = (n + 255) / 256;
  if (g > 148 * 16)
  {
    g = 148 * 16;
  }
  scale_kernel<<<static_cast<unsigned>(g), 256, 0, s>>>(src, dst, dtype, scale, n);
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

}  // namespace caifq
