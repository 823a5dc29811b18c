// Small dense helpers of the LoRA adapter path
// (src/caif_device_lora_adapter.cpp:205-281): the two reductions over tokens,
//   dB[out, r] = (alpha/r . dY)^T . H        dA[r, in] = dH^T . X
// (CAIF_Ops::MatMulTransposeA with beta = 0: the destination is overwritten),
// and the in-place Scale.  Operands are read in the adapter's storage dtype,
// products accumulate in fp32, the result is rounded once to the storage dtype.
#include <cstdlib>

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


// ------------------------------------------------------------------------------
// Fast path for bf16 adapters (rank a multiple of 8, at most 64).
// ------------------------------------------------------------------------------

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1)
{
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi)
{
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

// bf16x2 register times a scalar, each product rounded back to bf16
__device__ __forceinline__ uint32_t scale2(uint32_t v, float s)
{
  return pack2(__fmul_rn(__uint_as_float(v << 16), s), __fmul_rn(__uint_as_float(v & 0xFFFF0000u), s));
}

// H[m, R] = (prescale . X)[m, K] . A[R, K]^T, bf16 operands, fp32 accumulation, H rounded to bf16.
// A warp owns 16 rows; a lane streams 16 bytes (8 consecutive k) of rows g and g+8 per step
// straight from global memory into MMA fragments (the k order inside a fragment is the same
// for X and A, which is all a dot product needs).  Optionally also writes
//   Hs[m, 64] = bf16( float(H) * hs_mul / *hs_div ), zero beyond column R,
// the padded operand the tensor-core kernel consumes as one extra k-block.
template <int NT>  // NT = R / 8
__global__ void __launch_bounds__(256)
skinny_nt_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ a,
                 __nv_bfloat16 *__restrict__ h, __nv_bfloat16 *__restrict__ hs, float x_prescale, float hs_mul,
                 const float *__restrict__ hs_div, int64_t m, int k)
{
  // a CTA owns 16 rows; its 8 warps split K and add their partial tiles through shared memory
  __shared__ float part[8][16][NT * 8 + 1];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int t = lane & 3;
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * 16;
  const int64_t r_lo = row0 + g;
  const int64_t r_hi = row0 + g + 8;
  const bool lo_ok = r_lo < m;
  const bool hi_ok = r_hi < m;
  const int steps = k / 32;  // 32 k per step: 4 lanes x 8
  const int st_begin = (steps * warp) / 8;
  const int st_end = (steps * (warp + 1)) / 8;
  const uint4 *x_lo = reinterpret_cast<const uint4 *>(x + (lo_ok ? r_lo : 0) * k) + t;
  const uint4 *x_hi = reinterpret_cast<const uint4 *>(x + (hi_ok ? r_hi : 0) * k) + t;
  const uint4 *a_ptr[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
  {
    a_ptr[nt] = reinterpret_cast<const uint4 *>(a + static_cast<int64_t>(nt * 8 + g) * k) + t;
  }
  float c[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
  {
    c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.0f;
  }
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll 4
  for (int st = st_begin; st < st_end; ++st)
  {
    uint4 xa = lo_ok ? __ldg(x_lo + st * 4) : zero4;
    uint4 xb = hi_ok ? __ldg(x_hi + st * 4) : zero4;
    if (x_prescale != 1.0f)
    {
      xa = make_uint4(scale2(xa.x, x_prescale), scale2(xa.y, x_prescale), scale2(xa.z, x_prescale),
                      scale2(xa.w, x_prescale));
      xb = make_uint4(scale2(xb.x, x_prescale), scale2(xb.y, x_prescale), scale2(xb.z, x_prescale),
                      scale2(xb.w, x_prescale));
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
    {
      const uint4 wa = __ldg(a_ptr[nt] + st * 4);
      mma_bf16(c[nt], xa.x, xb.x, xa.y, xb.y, wa.x, wa.y);
      mma_bf16(c[nt], xa.z, xb.z, xa.w, xb.w, wa.z, wa.w);
    }
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
  {
    part[warp][g][nt * 8 + 2 * t] = c[nt][0];
    part[warp][g][nt * 8 + 2 * t + 1] = c[nt][1];
    part[warp][g + 8][nt * 8 + 2 * t] = c[nt][2];
    part[warp][g + 8][nt * 8 + 2 * t + 1] = c[nt][3];
  }
  __syncthreads();
  constexpr int R = NT * 8;
  float mul = hs_mul;
  if (hs != nullptr && hs_div != nullptr)
  {
    mul = __fdividef(hs_mul, hs_div[0]);
  }
  // 16 rows x 64 padded columns, one element pair per thread-iteration
  for (int e = threadIdx.x; e < 16 * 32; e += 256)
  {
    const int rr = e >> 5;
    const int col = (e & 31) * 2;
    const int64_t row = row0 + rr;
    if (row >= m)
    {
      continue;
    }
    if (col < R)
    {
      float v0 = 0.0f;
      float v1 = 0.0f;
#pragma unroll
      for (int w = 0; w < 8; ++w)
      {
        v0 += part[w][rr][col];
        v1 += part[w][rr][col + 1];
      }
      const uint32_t packed = pack2(v0, v1);
      *reinterpret_cast<uint32_t *>(h + row * R + col) = packed;
      if (hs != nullptr)
      {
        *reinterpret_cast<uint32_t *>(hs + row * 64 + col) = scale2(packed, mul);
      }
    }
    else if (hs != nullptr)
    {
      *reinterpret_cast<uint32_t *>(hs + row * 64 + col) = 0u;
    }
  }
}

__device__ __forceinline__ uint32_t smem_addr(const void *p)
{
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3)
{
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t addr, uint32_t &r0, uint32_t &r1)
{
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}

// C[big, R] (+)= sum over a slice of tokens of (prescale . U)[m, big]^T * V[m, R]   (fp32 atomics into acc).
// Both operands have the reduction index (the token) as their slow axis, so tiles of U and V are
// staged in shared memory as they lie and the tensor-core fragments are read transposed
// (ldmatrix.trans).  A CTA owns 64 columns of U, its 4 warps 16 each; gridDim.y slices the tokens.
// With `transpose_out` the accumulator is indexed [R, big] (dA).
constexpr int TN_COLS = 128;   // 256 bytes of every row per CTA; one warp per 16 columns
constexpr int STN_THREADS = (TN_COLS / 16) * 32;
constexpr int TN_ROWS = 64;
constexpr int TN_UPITCH = TN_COLS + 8;  // bf16 elements: 144-byte rows keep ldmatrix conflict-free

template <int NT>  // R = 8 * NT
__global__ void __launch_bounds__(STN_THREADS)
skinny_tn_kernel(const __nv_bfloat16 *__restrict__ u, const __nv_bfloat16 *__restrict__ v, float *__restrict__ acc,
                 float u_prescale, int64_t m, int big, int transpose_out)
{
  constexpr int R = 8 * NT;
  constexpr int VPITCH = R + 8;
  __shared__ __align__(16) __nv_bfloat16 su[TN_ROWS][TN_UPITCH];
  __shared__ __align__(16) __nv_bfloat16 sv[TN_ROWS][VPITCH];
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int g = lane >> 2;
  const int t = lane & 3;
  const int c0 = blockIdx.x * TN_COLS;
  const int64_t per = ((m + gridDim.y - 1) / gridDim.y + TN_ROWS - 1) / TN_ROWS * TN_ROWS;
  const int64_t m_begin = per * blockIdx.y;
  const int64_t m_end = (m_begin + per < m) ? (m_begin + per) : m;
  float c[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
  {
    c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.0f;
  }
  // A tile of 64 tokens x 128 columns of U (16-byte chunks, coalesced) and 64 x R of V goes through registers
  // into shared memory; the next tile's loads are issued before the current tile's MMAs, so they are in
  // flight while the tensor core works.
  constexpr int U_PER_THREAD = TN_ROWS * (TN_COLS / 8) / STN_THREADS;   // 4
  static_assert(TN_ROWS * (TN_COLS / 8) % STN_THREADS == 0, "whole chunks per thread");
  static_assert(TN_ROWS * NT <= 2 * STN_THREADS, "at most two chunks of V per thread");
  uint4 ru[U_PER_THREAD];
  uint4 rv[2];
  auto fetch = [&](int64_t mb)
  {
#pragma unroll
    for (int i = 0; i < U_PER_THREAD; ++i)
    {
      const int e = tid + i * STN_THREADS;
      const int rr = e / (TN_COLS / 8);
      const int ch = e % (TN_COLS / 8);
      ru[i] = make_uint4(0u, 0u, 0u, 0u);
      if (mb + rr < m_end && c0 + ch * 8 < big)
      {
        ru[i] = __ldg(reinterpret_cast<const uint4 *>(u + (mb + rr) * big + c0 + ch * 8));
      }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
    {
      const int e = tid + i * STN_THREADS;
      rv[i] = make_uint4(0u, 0u, 0u, 0u);
      if (e < TN_ROWS * NT && mb + e / NT < m_end)
      {
        rv[i] = __ldg(reinterpret_cast<const uint4 *>(v + (mb + e / NT) * R + (e % NT) * 8));
      }
    }
  };
  if (m_begin < m_end)
  {
    fetch(m_begin);
  }
  for (int64_t mb = m_begin; mb < m_end; mb += TN_ROWS)
  {
#pragma unroll
    for (int i = 0; i < U_PER_THREAD; ++i)
    {
      const int e = tid + i * STN_THREADS;
      uint4 val = ru[i];
      if (u_prescale != 1.0f)
      {
        val = make_uint4(scale2(val.x, u_prescale), scale2(val.y, u_prescale), scale2(val.z, u_prescale),
                         scale2(val.w, u_prescale));
      }
      *reinterpret_cast<uint4 *>(&su[e / (TN_COLS / 8)][(e % (TN_COLS / 8)) * 8]) = val;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
    {
      const int e = tid + i * STN_THREADS;
      if (e < TN_ROWS * NT)
      {
        *reinterpret_cast<uint4 *>(&sv[e / NT][(e % NT) * 8]) = rv[i];
      }
    }
    __syncthreads();
    if (mb + TN_ROWS < m_end)
    {
      fetch(mb + TN_ROWS);
    }
#pragma unroll
    for (int k16 = 0; k16 < TN_ROWS / 16; ++k16)
    {
      // A fragment: rows = this warp's 16 columns of U, k = 16 tokens.  Tile i of the x4 load:
      // columns (i & 1) * 8.., tokens (i >> 1) * 8..; lane l addresses row (l & 7) of tile (l >> 3).
      const int tile = lane >> 3;
      const uint32_t a_addr =
          smem_addr(&su[k16 * 16 + (tile >> 1) * 8 + (lane & 7)][warp * 16 + (tile & 1) * 8]);
      uint32_t a0, a1, a2, a3;
      ldmatrix_x4_trans(a_addr, a0, a1, a2, a3);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
      {
        // B fragment: k = 16 tokens, n = 8 columns of V; lanes 0..15 address the 16 token rows
        const uint32_t b_addr = smem_addr(&sv[k16 * 16 + (lane & 15)][nt * 8]);
        uint32_t b0, b1;
        ldmatrix_x2_trans(b_addr, b0, b1);
        mma_bf16(c[nt], a0, a1, a2, a3, b0, b1);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
  {
#pragma unroll
    for (int i = 0; i < 4; ++i)
    {
      const int col = c0 + warp * 16 + g + ((i >> 1) ? 8 : 0);  // column of U = row of C
      const int jj = nt * 8 + 2 * t + (i & 1);
      if (col < big)
      {
        const int64_t idx = transpose_out ? (static_cast<int64_t>(jj) * big + col) : (static_cast<int64_t>(col) * R + jj);
        atomicAdd(&acc[idx], c[nt][i]);
      }
    }
  }
}

// Bp[n, 64] = B[n, R] padded with zeros (forward), or Bt[R, n] = B[n, R]^T (backward).
__global__ void lora_pad_b_kernel(const __nv_bfloat16 *__restrict__ b, __nv_bfloat16 *__restrict__ bp, int n, int r)
{
  const int64_t total = static_cast<int64_t>(n) * 64;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
  {
    const int col = static_cast<int>(i & 63);
    const int64_t row = i >> 6;
    bp[i] = (col < r) ? b[row * r + col] : __float2bfloat16(0.0f);
  }
}

__global__ void lora_transpose_b_kernel(const __nv_bfloat16 *__restrict__ b, __nv_bfloat16 *__restrict__ bt, int n,
                                        int r)
{
  const int64_t total = static_cast<int64_t>(n) * r;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
  {
    const int64_t j = i / n;   // output row (rank index)
    const int64_t o = i % n;   // output column
    bt[i] = b[o * r + j];
  }
}

// Ap[64, n] = A[R, n] followed by zero rows.
__global__ void lora_pad_a_kernel(const __nv_bfloat16 *__restrict__ a, __nv_bfloat16 *__restrict__ ap, int n, int r)
{
  const int64_t total = static_cast<int64_t>(64) * n;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
  {
    ap[i] = (i < static_cast<int64_t>(r) * n) ? a[i] : __float2bfloat16(0.0f);
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

bool skinny_supported(int dtype, int rank, int k)
{
  return dtype == CAIFQ_BF16 && (rank == 8 || rank == 16 || rank == 32 || rank == 64) && (k % 32) == 0;
}

int launch_skinny_nt(const void *x, const void *a, void *h, void *hs, float x_prescale, float hs_mul,
                     const float *hs_div, int64_t m, int k, int rank, cudaStream_t s)
{
  if (m <= 0)
  {
    return CAIFQ_OK;
  }
  const unsigned grid = static_cast<unsigned>((m + 15) / 16);
  const __nv_bfloat16 *xp = static_cast<const __nv_bfloat16 *>(x);
  const __nv_bfloat16 *ap = static_cast<const __nv_bfloat16 *>(a);
  __nv_bfloat16 *hp = static_cast<__nv_bfloat16 *>(h);
  __nv_bfloat16 *hsp = static_cast<__nv_bfloat16 *>(hs);
  switch (rank)
  {
    case 8:
      skinny_nt_kernel<1><<<grid, 256, 0, s>>>(xp, ap, hp, hsp, x_prescale, hs_mul, hs_div, m, k);
      break;
    case 16:
      skinny_nt_kernel<2><<<grid, 256, 0, s>>>(xp, ap, hp, hsp, x_prescale, hs_mul, hs_div, m, k);
      break;
    case 32:
      skinny_nt_kernel<4><<<grid, 256, 0, s>>>(xp, ap, hp, hsp, x_prescale, hs_mul, hs_div, m, k);
      break;
    case 64:
      skinny_nt_kernel<8><<<grid, 256, 0, s>>>(xp, ap, hp, hsp, x_prescale, hs_mul, hs_div, m, k);
      break;
    default:
      set_error("LoRA fast path: unsupported rank %d", rank);
      return CAIFQ_ERR_UNSUPPORTED;
  }
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

// C = (prescale . U)^T . V with U [m, big], V [m, rank]; C is [big, rank] or, transposed, [rank, big].
int launch_skinny_tn(const void *u, const void *v, void *c, float *scratch, float u_prescale, int64_t m, int big,
                     int rank, bool transpose_out, cudaStream_t s)
{
  const int64_t n = static_cast<int64_t>(big) * rank;
  if (n <= 0)
  {
    return CAIFQ_OK;
  }
  CAIFQ_CHECK_CUDA(cudaMemsetAsync(scratch, 0, static_cast<size_t>(n) * sizeof(float), s));
  if (m > 0)
  {
    const int col_tiles = (big + TN_COLS - 1) / TN_COLS;
    int64_t slices = (148 * 8 + col_tiles - 1) / col_tiles;   // ~8 CTAs of 128 threads per SM
    const int64_t max_slices = (m + TN_ROWS - 1) / TN_ROWS;
    if (slices > max_slices)
    {
      slices = max_slices;
    }
    if (slices < 1)
    {
      slices = 1;
    }
    dim3 grid(col_tiles, static_cast<unsigned>(slices));
    const __nv_bfloat16 *up = static_cast<const __nv_bfloat16 *>(u);
    const __nv_bfloat16 *vp = static_cast<const __nv_bfloat16 *>(v);
    const int tr = transpose_out ? 1 : 0;
    switch (rank)
    {
      case 8:
        skinny_tn_kernel<1><<<grid, STN_THREADS, 0, s>>>(up, vp, scratch, u_prescale, m, big, tr);
        break;
      case 16:
        skinny_tn_kernel<2><<<grid, STN_THREADS, 0, s>>>(up, vp, scratch, u_prescale, m, big, tr);
        break;
      case 32:
        skinny_tn_kernel<4><<<grid, STN_THREADS, 0, s>>>(up, vp, scratch, u_prescale, m, big, tr);
        break;
      case 64:
        skinny_tn_kernel<8><<<grid, STN_THREADS, 0, s>>>(up, vp, scratch, u_prescale, m, big, tr);
        break;
      default:
        set_error("LoRA fast path: unsupported rank %d", rank);
        return CAIFQ_ERR_UNSUPPORTED;
    }
    CAIFQ_CHECK_LAUNCH();
  }
  int64_t g = (n + 255) / 256;
  if (g > 148 * 8)
  {
    g = 148 * 8;
  }
  round_out_kernel<<<static_cast<unsigned>(g), 256, 0, s>>>(scratch, c, CAIFQ_BF16, n);
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

// The weight's expansion to bf16 and the small re-layouts of the LoRA factors that a call needs, in ONE launch
// (they are independent of each other and each of them alone is mostly launch latency):
//   blockIdx.y == 0: the expansion (8 weights per thread and step);
//   blockIdx.y == 1: Bp = pad(B) [n_b, 64]      (forward), or
//                    Bt = B^T [r, n_b] and Ap = pad(A) [64, n_a]   (backward).
struct ExpandPrepare
{
  const void *codes;
  const __half *scales;
  uint4 *wb;
  int64_t units;      // weights / 8
  int group_size;
  const __nv_bfloat16 *a;   // [r, n_a]
  const __nv_bfloat16 *b;   // [n_b, r]
  __nv_bfloat16 *bp;        // forward: [n_b, 64]
  __nv_bfloat16 *bt;        // backward: [r, n_b]
  __nv_bfloat16 *ap;        // backward: [64, n_a]
  int n_a, n_b, r;
};

template <int STORAGE>
__global__ void expand_prepare_kernel(const ExpandPrepare p)
{
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (blockIdx.y == 0)
  {
    // four units per thread and trip, a block width apart: the loads are all in flight before the first
    // conversion and a warp's accesses stay contiguous
    constexpr int kPerTrip = 4;
    for (int64_t base = static_cast<int64_t>(blockIdx.x) * blockDim.x * kPerTrip + threadIdx.x; base < p.units;
         base += stride * kPerTrip)
    {
      if (STORAGE == CAIFQ_I8)
      {
        uint2 c[kPerTrip];
#pragma unroll
        for (int u = 0; u < kPerTrip; ++u)
        {
          const int64_t i = base + static_cast<int64_t>(u) * blockDim.x;
          c[u] = (i < p.units) ? __ldg(static_cast<const uint2 *>(p.codes) + i) : make_uint2(0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < kPerTrip; ++u)
        {
          const int64_t i = base + static_cast<int64_t>(u) * blockDim.x;
          if (i < p.units)
          {
            p.wb[i] = expand_int8x8(c[u]);
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
          if (i < p.units)
          {
            c[u] = __ldg(static_cast<const uint32_t *>(p.codes) + i);
            sc[u] = __ldg(p.scales + (i * 8) / p.group_size);
          }
        }
#pragma unroll
        for (int u = 0; u < kPerTrip; ++u)
        {
          const int64_t i = base + static_cast<int64_t>(u) * blockDim.x;
          if (i < p.units)
          {
            p.wb[i] = expand_int4x8(c[u], __half2float(sc[u]));
          }
        }
      }
    }
    return;
  }
  const __nv_bfloat16 zero = __float2bfloat16(0.0f);
  if (p.bp != nullptr)
  {
    const int64_t total = static_cast<int64_t>(p.n_b) * 64;
    for (int64_t i = first; i < total; i += stride)
    {
      const int col = static_cast<int>(i & 63);
      p.bp[i] = (col < p.r) ? p.b[(i >> 6) * p.r + col] : zero;
    }
  }
  if (p.bt != nullptr)
  {
    const int64_t total = static_cast<int64_t>(p.n_b) * p.r;
    for (int64_t i = first; i < total; i += stride)
    {
      p.bt[i] = p.b[(i % p.n_b) * p.r + i / p.n_b];
    }
  }
  if (p.ap != nullptr)
  {
    const int64_t total = static_cast<int64_t>(64) * p.n_a;
    const int64_t live = static_cast<int64_t>(p.r) * p.n_a;
    for (int64_t i = first; i < total; i += stride)
    {
      p.ap[i] = (i < live) ? p.a[i] : zero;
    }
  }
}

// forward: bp != null; backward: bt and ap != null.  The weight must be one launch_expand_to_bf16 takes.
int launch_expand_prepare(const caifq_weight &w, void *wb, const void *a, const void *b, void *bp, void *bt, void *ap,
                          int rank, cudaStream_t s)
{
  const int64_t total = static_cast<int64_t>(w.in_dim) * w.out_dim;
  const bool i8 = (w.storage == CAIFQ_I8);
  if ((total % 8) != 0 || (!i8 && !(w.storage == CAIFQ_I4 && w.scales != nullptr && w.group_size > 0 &&
                                    (w.group_size % 8) == 0)) ||
      (reinterpret_cast<uintptr_t>(w.codes) & 7u) != 0)
  {
    set_error("expand_prepare: unsupported weight (storage %d)", w.storage);
    return CAIFQ_ERR_UNSUPPORTED;
  }
  ExpandPrepare p{};
  p.codes = w.codes;
  p.scales = static_cast<const __half *>(w.scales);
  p.wb = static_cast<uint4 *>(wb);
  p.units = total / 8;
  p.group_size = w.group_size;
  p.a = static_cast<const __nv_bfloat16 *>(a);
  p.b = static_cast<const __nv_bfloat16 *>(b);
  p.bp = static_cast<__nv_bfloat16 *>(bp);
  p.bt = static_cast<__nv_bfloat16 *>(bt);
  p.ap = static_cast<__nv_bfloat16 *>(ap);
  p.n_a = w.in_dim;
  p.n_b = w.out_dim;
  p.r = rank;
  const dim3 grid(148 * 8, 2);
  if (i8)
  {
    expand_prepare_kernel<CAIFQ_I8><<<grid, 256, 0, s>>>(p);
  }
  else
  {
    expand_prepare_kernel<CAIFQ_I4><<<grid, 256, 0, s>>>(p);
  }
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_lora_pad_b(const void *b, void *bp, int n, int rank, cudaStream_t s)
{
  lora_pad_b_kernel<<<148 * 2, 256, 0, s>>>(static_cast<const __nv_bfloat16 *>(b), static_cast<__nv_bfloat16 *>(bp), n,
                                           rank);
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_lora_transpose_b(const void *b, void *bt, int n, int rank, cudaStream_t s)
{
  lora_transpose_b_kernel<<<148, 256, 0, s>>>(static_cast<const __nv_bfloat16 *>(b), static_cast<__nv_bfloat16 *>(bt),
                                             n, rank);
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int launch_lora_pad_a(const void *a, void *ap, int n, int rank, cudaStream_t s)
{
  lora_pad_a_kernel<<<148 * 2, 256, 0, s>>>(static_cast<const __nv_bfloat16 *>(a), static_cast<__nv_bfloat16 *>(ap), n,
                                           rank);
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

// AdamW step of the two LoRA factors in one launch (the reference steps every parameter tensor with its own
// launch of fused_adam_kernel, src/caif_cuda_kernels_optimizers.cu:49-92).  Same arithmetic in the same
// order, all in fp32 with fp32 moments; only the loads and stores of the factors and their gradients cross
// to the storage dtype.
struct AdamwParams
{
  void *param[2];
  const void *grad[2];
  float *m[2];
  float *v[2];
  int64_t n[2];
  int dtype;
  float lr, beta1, beta2, epsilon, weight_decay, bias_correction1, bias_correction2;
};

__global__ void lora_adamw_kernel(const AdamwParams a)
{
  const int64_t total = a.n[0] + a.n[1];
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
  {
    const int t = (i < a.n[0]) ? 0 : 1;
    const int64_t idx = (t == 0) ? i : i - a.n[0];
    float p = load_as_float(a.param[t], idx, a.dtype);
    const float g = load_as_float(a.grad[t], idx, a.dtype);
    float m_val = a.m[t][idx];
    float v_val = a.v[t][idx];
    if (a.weight_decay != 0.0f)
    {
      p = p * (1.0f - a.lr * a.weight_decay);
    }
    // The reference's expressions beta1*m + (1-beta1)*g and beta2*v + (1-beta2)*g*g compile to one multiply and
    // one fused multiply-add each; which product is fused decides the last bit.  Written out so that this
    // kernel does not depend on the compiler making the same choice (checked bit for bit against the
    // reference kernel): the gradient term is the fused one.
    m_val = fmaf(__fsub_rn(1.0f, a.beta1), g, __fmul_rn(a.beta1, m_val));
    v_val = fmaf(__fmul_rn(__fsub_rn(1.0f, a.beta2), g), g, __fmul_rn(a.beta2, v_val));
    const float m_hat = m_val / a.bias_correction1;
    const float v_hat = v_val / a.bias_correction2;
    p = p - a.lr * m_hat / (sqrtf(v_hat) + a.epsilon);
    store_from_float(a.param[t], idx, a.dtype, p);
    a.m[t][idx] = m_val;
    a.v[t][idx] = v_val;
  }
}

int launch_lora_adamw(void *a, void *b, const void *d_a, const void *d_b, float *m_a, float *v_a, float *m_b,
                      float *v_b, int64_t n_a, int64_t n_b, int dtype, float lr, float beta1, float beta2,
                      float epsilon, float weight_decay, float bias_correction1, float bias_correction2,
                      cudaStream_t s)
{
  AdamwParams p{};
  p.param[0] = a;
  p.param[1] = b;
  p.grad[0] = d_a;
  p.grad[1] = d_b;
  p.m[0] = m_a;
  p.m[1] = m_b;
  p.v[0] = v_a;
  p.v[1] = v_b;
  p.n[0] = n_a;
  p.n[1] = n_b;
  p.dtype = dtype;
  p.lr = lr;
  p.beta1 = beta1;
  p.beta2 = beta2;
  p.epsilon = epsilon;
  p.weight_decay = weight_decay;
  p.bias_correction1 = bias_correction1;
  p.bias_correction2 = bias_correction2;
  int64_t g = (n_a + n_b + 255) / 256;
  if (g > 148 * 8)
  {
    g = 148 * 8;
  }
  if (g < 1)
  {
    return CAIFQ_OK;
  }
  lora_adamw_kernel<<<static_cast<unsigned>(g), 256, 0, s>>>(p);
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
