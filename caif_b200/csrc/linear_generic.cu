// Shape- and dtype-complete frozen-linear GEMM on fp32 FMA units.
//
// Covers every (storage, compute) cell of CAIF_DeviceFrozenLinear
// (src/caif_device_frozen_linear.cpp:837-853), every scale rule including the
// ones that do not factor out of the product (int4 groups that straddle rows,
// the per-channel index `flat % out_dim`), and every shape.  The weight element
// is dequantized while its tile is staged into shared memory, rounded through
// the compute dtype exactly where the reference rounds it, and multiplied in
// fp32 -- so with compute fp32 the result equals the reference's
// Accuracy_e / host sgemm path up to summation order.
//
//   forward : C[m, out] = A[m, in]  . W[out, in]^T
//   backward: C[m, in]  = A[m, out] . W[out, in]
//
// The tensor-core and weight-streaming kernels take the shapes they are built
// for; this one takes the rest.
#include "common.cuh"

namespace caifq
{

namespace
{

constexpr int BM = 64;
constexpr int BN = 64;
constexpr int BK = 16;
constexpr int THREADS = 256;

template <int STORAGE, int COMPUTE, bool BACKWARD>
__global__ void __launch_bounds__(THREADS)
linear_generic_kernel(caifq_weight w, const void *__restrict__ a, int a_dtype, float a_prescale, int64_t m,
                      void *__restrict__ c, int c_dtype, bool accumulate)
{
  // N = columns of C, K = reduction length
  const int n_dim = BACKWARD ? w.in_dim : w.out_dim;
  const int k_dim = BACKWARD ? w.out_dim : w.in_dim;

  __shared__ float sa[BK][BM + 1];
  __shared__ float sb[BK][BN + 1];

  const int tid = threadIdx.x;
  const int tx = tid % 16;  // column group
  const int ty = tid / 16;  // row group
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * BM;
  const int n0 = blockIdx.x * BN;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
  {
#pragma unroll
    for (int j = 0; j < 4; ++j)
    {
      acc[i][j] = 0.0f;
    }
  }

  for (int k0 = 0; k0 < k_dim; k0 += BK)
  {
    // A tile: BM x BK, k fastest in memory
#pragma unroll
    for (int e = tid; e < BM * BK; e += THREADS)
    {
      const int kk = e % BK;
      const int mm = e / BK;
      const int64_t gm = m0 + mm;
      const int gk = k0 + kk;
      float v = 0.0f;
      if (gm < m && gk < k_dim)
      {
        v = load_as_float(a, gm * k_dim + gk, a_dtype);
        if (a_prescale != 1.0f)
        {
          v = round_through_rt(__fmul_rn(v, a_prescale), a_dtype);
        }
        v = round_through<COMPUTE>(v);
      }
      sa[kk][mm] = v;
    }
    // W tile: BN x BK
#pragma unroll
    for (int e = tid; e < BN * BK; e += THREADS)
    {
      int kk;
      int nn;
      if (BACKWARD)
      {
        nn = e % BN;  // n runs along `in`, contiguous in memory
        kk = e / BN;
      }
      else
      {
        kk = e % BK;  // k runs along `in`
        nn = e / BK;
      }
      const int gn = n0 + nn;
      const int gk = k0 + kk;
      float v = 0.0f;
      if (gn < n_dim && gk < k_dim)
      {
        const int64_t flat = BACKWARD ? (static_cast<int64_t>(gk) * w.in_dim + gn)
                                      : (static_cast<int64_t>(gn) * w.in_dim + gk);
        v = weight_value<STORAGE>(w, flat);
        if (COMPUTE != STORAGE)
        {
          v = round_through<COMPUTE>(v);
        }
      }
      sb[kk][nn] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk)
    {
      float av[4];
      float bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
      {
        av[i] = sa[kk][ty * 4 + i];
        bv[i] = sb[kk][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
      {
#pragma unroll
        for (int j = 0; j < 4; ++j)
        {
          acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
      }
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i)
  {
    const int64_t gm = m0 + ty * 4 + i;
    if (gm >= m)
    {
      continue;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
    {
      const int gn = n0 + tx * 4 + j;
      if (gn < n_dim)
      {
        float v = acc[i][j];
        if (accumulate)
        {
          v = round_through_rt(v, c_dtype) + load_as_float(c, gm * n_dim + gn, c_dtype);
        }
        store_from_float(c, gm * n_dim + gn, c_dtype, v);
      }
    }
  }
}

template <int STORAGE, int COMPUTE>
int launch_sc(const LinearArgs &g, cudaStream_t s)
{
  const int n_dim = g.backward ? g.w.in_dim : g.w.out_dim;
  dim3 grid((n_dim + BN - 1) / BN, static_cast<unsigned>((g.m + BM - 1) / BM));
  if (g.backward)
  {
    linear_generic_kernel<STORAGE, COMPUTE, true>
        <<<grid, THREADS, 0, s>>>(g.w, g.a, g.a_dtype, g.a_prescale, g.m, g.c, g.c_dtype, g.accumulate);
  }
  else
  {
    linear_generic_kernel<STORAGE, COMPUTE, false>
        <<<grid, THREADS, 0, s>>>(g.w, g.a, g.a_dtype, g.a_prescale, g.m, g.c, g.c_dtype, g.accumulate);
  }
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

template <int STORAGE>
int launch_s(const LinearArgs &g, cudaStream_t s)
{
  switch (g.compute_dtype)
  {
    case CAIFQ_F32:
      return launch_sc<STORAGE, CAIFQ_F32>(g, s);
    case CAIFQ_F16:
      return launch_sc<STORAGE, CAIFQ_F16>(g, s);
    case CAIFQ_BF16:
      return launch_sc<STORAGE, CAIFQ_BF16>(g, s);
    default:
      set_error("frozen linear: unsupported compute dtype %d", g.compute_dtype);
      return CAIFQ_ERR_INVALID;
  }
}

}  // namespace

int launch_linear_generic(const LinearArgs &g, cudaStream_t s)
{
  if (g.m <= 0)
  {
    return CAIFQ_OK;
  }
  if (g.m > static_cast<int64_t>(65535) * BM)
  {
    set_error("frozen linear (generic): m=%lld too large", static_cast<long long>(g.m));
    return CAIFQ_ERR_INVALID;
  }
  switch (g.w.storage)
  {
    case CAIFQ_F32:
      return launch_s<CAIFQ_F32>(g, s);
    case CAIFQ_F16:
      return launch_s<CAIFQ_F16>(g, s);
    case CAIFQ_BF16:
      return launch_s<CAIFQ_BF16>(g, s);
    case CAIFQ_I8:
      return launch_s<CAIFQ_I8>(g, s);
    case CAIFQ_I4:
      return launch_s<CAIFQ_I4>(g, s);
    default:
      set_error("frozen linear: unsupported storage dtype %d", g.w.storage);
      return CAIFQ_ERR_INVALID;
  }
}

}  // namespace caifq
