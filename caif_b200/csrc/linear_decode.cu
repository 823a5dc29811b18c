// Weight-streaming frozen-linear forward for few tokens (decode shapes).
//
//   y[m, out] = x[m, in] . W_deq[out, in]^T      m <= 16, x bf16, y fp32/bf16/fp16
//
// The call is bound by reading the packed codes once from HBM
// (CAIF_DeviceFrozenLinear::ForwardImpl, src/caif_device_frozen_linear.cpp:381-524,
// does the same product after writing and re-reading an fp32 copy of the whole
// weight, :319-334).  Design:
//   * one persistent CTA per SM owns a contiguous range of 8-row units of the
//     [out, in] code matrix, i.e. one contiguous slab of HBM;
//   * an elected lane streams that slab through a shared-memory ring with bulk
//     async copies (cp.async.bulk + mbarrier transaction counts), several
//     stages (tens of KB) in flight per SM regardless of register pressure;
//   * 16 warps split the reduction dimension; each lane pulls 16 bytes of codes
//     from the ring, turns nibbles/bytes into exact bf16 integers with logic ops
//     (no int->float converts), and feeds them to bf16 tensor-core MMAs against
//     token fragments that stay in registers for the whole kernel;
//   * int4 group scales multiply the fp32 partial sum once per 128-element
//     group; the int8 per-tensor scale multiplies the final sum.
// Codes and activations are exact in bf16 and products accumulate in fp32, so
// the result matches an fp32 GEMM on the dequantized weight up to summation
// order.
#include "common.cuh"

namespace caifq
{

__device__ unsigned int g_decode_timeout_flag = 0;

namespace
{

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kUnitRows = 8;
constexpr int kMaxStages = 8;
constexpr uint32_t kSpinLimit = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

// Bounded wait: gives up after kSpinLimit polls and records it, so a copy that
// never lands turns into wrong numbers plus a flag instead of a hung GPU.
__device__ __forceinline__ void mbar_wait(uint64_t *bar, uint32_t parity)
{
  const uint32_t addr = smem_u32(bar);
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
  {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done)
    {
      return;
    }
  }
  atomicExch(&g_decode_timeout_flag, 1u);
}

__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar)
{
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1)
{
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b)
{
  uint32_t d;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c)
{
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));  // (a & b) | c
  return d;
}

struct DecodeParams
{
  const uint8_t *codes;   // [out, in] packed
  const void *scales;     // int4: fp16 per group; int8: fp32[1] or null
  const __nv_bfloat16 *x; // [m, in]
  void *y;                // [m, out]
  int y_dtype;
  int m;
  int in_dim;
  int out_dim;
  int groups_per_row;     // int4: in_dim / group_size
  int chunks_per_group;   // int4: group_size / 128
  int num_units;          // ceil(out / 8)
  int stages;
  uint32_t row_bytes;     // packed bytes per weight row
  uint32_t row_stride;    // padded row pitch in the ring
  uint32_t scale_bytes;   // int4: bytes of scales per unit (8 rows)
  uint32_t stage_bytes;   // ring stage pitch
};

// BITS: 4 or 8.  MT: token tiles of 8 (1 -> m <= 8, 2 -> m <= 16).
// NCH: 16-byte chunks of one row each lane of a warp handles per unit.
template <int BITS, int MT, int NCH>
__global__ void __launch_bounds__(kThreads, 1) linear_decode_kernel(const DecodeParams p)
{
  constexpr int ELEMS = 128 / BITS;      // codes per 16-byte load: 32 or 16
  constexpr int CHUNK_K = 4 * ELEMS;     // k covered by a quad of lanes: 128 or 64
  constexpr int STEPS = ELEMS / 4;       // MMAs per 16-byte load: 8 or 4
  constexpr int XR = ELEMS / 2;          // bf16x2 registers of x per chunk and token: 16 or 8

  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ uint64_t full_bar[kMaxStages];
  __shared__ float partial[2][kWarps][8 * MT][kUnitRows];

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int g = lane >> 2;  // weight row inside the unit (B fragment column), token inside a tile (A fragment row)
  const int t = lane & 3;

  const int unit_begin = static_cast<int>((static_cast<int64_t>(blockIdx.x) * p.num_units) / gridDim.x);
  const int unit_end = static_cast<int>((static_cast<int64_t>(blockIdx.x + 1) * p.num_units) / gridDim.x);
  const int my_units = unit_end - unit_begin;
  const int num_chunks = p.in_dim / CHUNK_K;

  if (tid == 0)
  {
    for (int s = 0; s < p.stages; ++s)
    {
      mbar_init(&full_bar[s], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // Producer: lanes 0..7 of warp 0 copy one weight row each, lane 8 the scales.
  auto issue = [&](int local_unit)
  {
    const int s = local_unit % p.stages;
    const int unit = unit_begin + local_unit;
    const int row0 = unit * kUnitRows;
    const int rows = min(kUnitRows, p.out_dim - row0);
    uint8_t *stage = smem + static_cast<size_t>(s) * p.stage_bytes;
    if (lane == 0)
    {
      uint32_t bytes = static_cast<uint32_t>(rows) * p.row_bytes;
      if (BITS == 4)
      {
        bytes += static_cast<uint32_t>(rows) * static_cast<uint32_t>(p.groups_per_row) * 2u;
      }
      mbar_expect_tx(&full_bar[s], bytes);
    }
    __syncwarp();
    if (lane < rows)
    {
      bulk_g2s(stage + static_cast<size_t>(lane) * p.row_stride,
               p.codes + static_cast<size_t>(row0 + lane) * p.row_bytes, p.row_bytes, &full_bar[s]);
    }
    if (BITS == 4 && lane == 8)
    {
      const uint8_t *src = static_cast<const uint8_t *>(p.scales) + static_cast<size_t>(row0) * p.groups_per_row * 2;
      bulk_g2s(stage + static_cast<size_t>(kUnitRows) * p.row_stride, src,
               static_cast<uint32_t>(rows) * static_cast<uint32_t>(p.groups_per_row) * 2u, &full_bar[s]);
    }
  };

  if (warp == 0)
  {
    const int pre = min(p.stages, my_units);
    for (int i = 0; i < pre; ++i)
    {
      issue(i);
    }
  }

  // Token fragments, resident for the whole kernel.  For the 16 bytes of codes
  // a lane reads at k-offset kb, word wi and shift sh pair the elements
  // kb + 8*wi + sh (BITS=4: and +4; BITS=8: sh in {0,1}, and +2) -- the same
  // pairing the logic-op dequantization produces.
  uint32_t xf[NCH][MT][XR];
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch)
  {
    const int cidx = warp + ch * kWarps;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
    {
      const int token = g + 8 * mt;
      const bool live = (cidx < num_chunks) && (token < p.m);
      uint32_t raw[XR];
      if (live)
      {
        const uint4 *src =
            reinterpret_cast<const uint4 *>(p.x + static_cast<size_t>(token) * p.in_dim + cidx * CHUNK_K + t * ELEMS);
#pragma unroll
        for (int i = 0; i < XR / 4; ++i)
        {
          const uint4 v = __ldg(src + i);
          raw[4 * i + 0] = v.x;
          raw[4 * i + 1] = v.y;
          raw[4 * i + 2] = v.z;
          raw[4 * i + 3] = v.w;
        }
      }
      else
      {
#pragma unroll
        for (int i = 0; i < XR; ++i)
        {
          raw[i] = 0u;
        }
      }
      if (BITS == 4)
      {
        // per code word (8 elements = 4 raw regs): pairs {0,4},{1,5},{2,6},{3,7}
#pragma unroll
        for (int wi = 0; wi < 4; ++wi)
        {
          xf[ch][mt][4 * wi + 0] = __byte_perm(raw[4 * wi + 0], raw[4 * wi + 2], 0x5410);
          xf[ch][mt][4 * wi + 1] = __byte_perm(raw[4 * wi + 0], raw[4 * wi + 2], 0x7632);
          xf[ch][mt][4 * wi + 2] = __byte_perm(raw[4 * wi + 1], raw[4 * wi + 3], 0x5410);
          xf[ch][mt][4 * wi + 3] = __byte_perm(raw[4 * wi + 1], raw[4 * wi + 3], 0x7632);
        }
      }
      else
      {
        // per code word (4 elements = 2 raw regs): pairs {0,2},{1,3}
#pragma unroll
        for (int wi = 0; wi < 4; ++wi)
        {
          xf[ch][mt][2 * wi + 0] = __byte_perm(raw[2 * wi + 0], raw[2 * wi + 1], 0x5410);
          xf[ch][mt][2 * wi + 1] = __byte_perm(raw[2 * wi + 0], raw[2 * wi + 1], 0x7632);
        }
      }
    }
  }

  float tensor_scale = 1.0f;
  if (BITS == 8 && p.scales != nullptr)
  {
    tensor_scale = static_cast<const float *>(p.scales)[0];
  }

  for (int it = 0; it < my_units; ++it)
  {
    const int s = it % p.stages;
    const uint32_t parity = static_cast<uint32_t>((it / p.stages) & 1);
    mbar_wait(&full_bar[s], parity);
    const uint8_t *stage = smem + static_cast<size_t>(s) * p.stage_bytes;
    const __half *stage_scales = reinterpret_cast<const __half *>(stage + static_cast<size_t>(kUnitRows) * p.row_stride);

    float yacc[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
    {
      yacc[mt][0] = 0.0f;
      yacc[mt][1] = 0.0f;
    }

    // accumulator of the running int4 group (or of everything for int8):
    // c[0],c[1] = token g, rows 2t, 2t+1;  c[2],c[3] = token g+8, same rows
    float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};

#pragma unroll
    for (int ch = 0; ch < NCH; ++ch)
    {
      const int cidx = warp + ch * kWarps;
      if (cidx < num_chunks)
      {
        const uint4 wv = *reinterpret_cast<const uint4 *>(stage + static_cast<size_t>(g) * p.row_stride +
                                                          static_cast<size_t>(cidx) * 64 + t * 16);
        const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
        uint32_t bq[XR];
        if (BITS == 4)
        {
#pragma unroll
          for (int wi = 0; wi < 4; ++wi)
          {
            const uint32_t wx = words[wi] ^ 0x88888888u;  // two's complement nibble -> offset binary
#pragma unroll
            for (int sh = 0; sh < 4; ++sh)
            {
              const uint32_t biased = lop3_and_or(wx >> (4 * sh), 0x000F000Fu, 0x43004300u);  // 128 + u
              bq[4 * wi + sh] = sub_bf16x2(biased, 0x43084308u);                              // - 136
            }
          }
        }
        else
        {
#pragma unroll
          for (int wi = 0; wi < 4; ++wi)
          {
#pragma unroll
            for (int sh = 0; sh < 2; ++sh)
            {
              const uint32_t pr = (words[wi] >> (8 * sh)) & 0x00FF00FFu;
              const uint32_t mag = lop3_and_or(pr, 0x007F007Fu, 0x43004300u);  // 128 + low 7 bits
              const uint32_t off = lop3_and_or(pr, 0x00800080u, 0x43004300u);  // 128 or 256 by sign bit
              bq[2 * wi + sh] = sub_bf16x2(mag, off);
            }
          }
        }
#pragma unroll
        for (int j = 0; j < STEPS; ++j)
        {
          const uint32_t a0 = xf[ch][0][2 * j];
          const uint32_t a2 = xf[ch][0][2 * j + 1];
          const uint32_t a1 = (MT == 2) ? xf[ch][MT - 1][2 * j] : 0u;
          const uint32_t a3 = (MT == 2) ? xf[ch][MT - 1][2 * j + 1] : 0u;
          mma_bf16_16816(c, a0, a1, a2, a3, bq[2 * j], bq[2 * j + 1]);
        }
        if (BITS == 4)
        {
          // this chunk lies inside one scale group of rows 2t and 2t+1; scaling
          // per 128-element chunk equals scaling per group up to rounding order
          const int grp = cidx / p.chunks_per_group;
          const float s0 = __half2float(stage_scales[(2 * t) * p.groups_per_row + grp]);
          const float s1 = __half2float(stage_scales[(2 * t + 1) * p.groups_per_row + grp]);
          yacc[0][0] = fmaf(s0, c[0], yacc[0][0]);
          yacc[0][1] = fmaf(s1, c[1], yacc[0][1]);
          if (MT == 2)
          {
            yacc[MT - 1][0] = fmaf(s0, c[2], yacc[MT - 1][0]);
            yacc[MT - 1][1] = fmaf(s1, c[3], yacc[MT - 1][1]);
          }
          c[0] = c[1] = c[2] = c[3] = 0.0f;
        }
      }
    }
    if (BITS == 8)
    {
      yacc[0][0] = c[0];
      yacc[0][1] = c[1];
      if (MT == 2)
      {
        yacc[MT - 1][0] = c[2];
        yacc[MT - 1][1] = c[3];
      }
    }

    float(*part)[8 * MT][kUnitRows] = partial[it & 1];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
    {
      part[warp][g + 8 * mt][2 * t] = yacc[mt][0];
      part[warp][g + 8 * mt][2 * t + 1] = yacc[mt][1];
    }
    __syncthreads();

    // every warp has finished reading stage s: refill it
    if (warp == 0 && it + p.stages < my_units)
    {
      issue(it + p.stages);
    }

    if (tid < 8 * MT * kUnitRows)
    {
      const int token = tid / kUnitRows;
      const int r = tid % kUnitRows;
      float sum = 0.0f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w)
      {
        sum += part[w][token][r];
      }
      if (BITS == 8)
      {
        sum *= tensor_scale;
      }
      const int row = (unit_begin + it) * kUnitRows + r;
      if (token < p.m && row < p.out_dim)
      {
        store_from_float(p.y, static_cast<int64_t>(token) * p.out_dim + row, p.y_dtype, sum);
      }
    }
  }
}

int sm_count()
{
  static int cached = 0;
  if (cached == 0)
  {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev);
    if (cached <= 0)
    {
      cached = 148;
    }
  }
  return cached;
}

template <int BITS, int MT, int NCH>
int launch_decode_inst(const DecodeParams &p, cudaStream_t s)
{
  auto kernel = linear_decode_kernel<BITS, MT, NCH>;
  const size_t smem = static_cast<size_t>(p.stages) * p.stage_bytes;
  static bool configured = false;
  if (!configured)
  {
    CAIFQ_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    configured = true;
  }
  int grid = sm_count();
  if (grid > p.num_units)
  {
    grid = p.num_units;
  }
  kernel<<<grid, kThreads, smem, s>>>(p);
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int chunks_per_warp(const caifq_weight &w)
{
  const int chunk_k = (w.storage == CAIFQ_I4) ? 128 : 64;
  const int chunks = w.in_dim / chunk_k;
  return (chunks + kWarps - 1) / kWarps;
}

}  // namespace

bool decode_supported(const LinearArgs &args)
{
  const caifq_weight &w = args.w;
  const int x_dtype = args.a_dtype;
  const int64_t m = args.m;
  const int y_dtype = args.c_dtype;
  const int compute_dtype = args.compute_dtype;
  if (args.backward || args.accumulate || args.a_prescale != 1.0f)
  {
    return false;
  }
  if (m < 1 || m > 16 || x_dtype != CAIFQ_BF16 || !is_float_dtype(y_dtype))
  {
    return false;
  }
  // Operands are exact in bf16 and accumulate in fp32: valid for fp32 and bf16
  // compute.  fp16 compute rounds x differently and goes elsewhere.
  if (compute_dtype != CAIFQ_F32 && compute_dtype != CAIFQ_BF16)
  {
    return false;
  }
  if (w.storage == CAIFQ_I4)
  {
    if (w.scales == nullptr || w.group_size < 128 || (w.group_size % 128) != 0 || (w.in_dim % w.group_size) != 0)
    {
      return false;
    }
    // partial last units copy rows * groups_per_row fp16 scales: keep that a 16-byte multiple
    if ((w.out_dim % kUnitRows) != 0 && ((w.in_dim / w.group_size) % 8) != 0)
    {
      return false;
    }
    // bf16 compute in the reference rounds scale*code to bf16 before the
    // product; this kernel keeps the exact fp32 scale.  Both are inside the
    // bf16 tolerance, and fp32 compute is matched exactly.
  }
  else if (w.storage == CAIFQ_I8)
  {
    if (w.scales != nullptr && w.scheme != CAIFQ_PER_TENSOR)
    {
      return false;
    }
    if ((w.in_dim % 64) != 0)
    {
      return false;
    }
  }
  else
  {
    return false;
  }
  const int nch = chunks_per_warp(w);
  const int xr = (w.storage == CAIFQ_I4) ? 16 : 8;
  const int mt = (m > 8) ? 2 : 1;
  if (nch * xr * mt > 64 || nch > 8)
  {
    return false;
  }
  if ((reinterpret_cast<uintptr_t>(w.codes) & 15u) != 0 || (reinterpret_cast<uintptr_t>(w.scales) & 15u) != 0)
  {
    return false;
  }
  return true;
}

int launch_linear_decode(const LinearArgs &args, cudaStream_t s)
{
  const caifq_weight &w = args.w;
  const void *x = args.a;
  const int64_t m = args.m;
  void *y = args.c;
  const int y_dtype = args.c_dtype;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0)
  {
    set_error("frozen linear (decode): x must be 16-byte aligned");
    return CAIFQ_ERR_INVALID;
  }
  DecodeParams p{};
  p.codes = static_cast<const uint8_t *>(w.codes);
  p.scales = w.scales;
  p.x = static_cast<const __nv_bfloat16 *>(x);
  p.y = y;
  p.y_dtype = y_dtype;
  p.m = static_cast<int>(m);
  p.in_dim = w.in_dim;
  p.out_dim = w.out_dim;
  p.num_units = (w.out_dim + kUnitRows - 1) / kUnitRows;
  const bool i4 = (w.storage == CAIFQ_I4);
  p.row_bytes = i4 ? static_cast<uint32_t>(w.in_dim / 2) : static_cast<uint32_t>(w.in_dim);
  // pitch = 64 mod 128 keeps the two rows of a quarter-warp on different banks
  p.row_stride = ((p.row_bytes % 128u) == 0u) ? (p.row_bytes + 64u) : p.row_bytes;
  if (i4)
  {
    p.groups_per_row = w.in_dim / w.group_size;
    p.chunks_per_group = w.group_size / 128;
    p.scale_bytes = static_cast<uint32_t>(kUnitRows * p.groups_per_row * 2);
  }
  else
  {
    p.groups_per_row = 0;
    p.chunks_per_group = 1;
    p.scale_bytes = 0;
  }
  p.stage_bytes = ((kUnitRows * p.row_stride + p.scale_bytes) + 127u) & ~127u;
  int stages = static_cast<int>((160u * 1024u) / p.stage_bytes);
  if (stages > kMaxStages)
  {
    stages = kMaxStages;
  }
  if (stages < 2)
  {
    set_error("frozen linear (decode): row too long for the shared-memory ring");
    return CAIFQ_ERR_UNSUPPORTED;
  }
  p.stages = stages;

  const int nch = chunks_per_warp(w);
  const int mt = (m > 8) ? 2 : 1;
#define CAIFQ_DECODE_CASE(B, M, N)        \
  if (nch <= N && mt == M)                \
  {                                       \
    return launch_decode_inst<B, M, N>(p, s); \
  }
  if (i4)
  {
    CAIFQ_DECODE_CASE(4, 1, 1)
    CAIFQ_DECODE_CASE(4, 1, 2)
    CAIFQ_DECODE_CASE(4, 1, 4)
    CAIFQ_DECODE_CASE(4, 2, 1)
    CAIFQ_DECODE_CASE(4, 2, 2)
  }
  else
  {
    CAIFQ_DECODE_CASE(8, 1, 2)
    CAIFQ_DECODE_CASE(8, 1, 4)
    CAIFQ_DECODE_CASE(8, 1, 8)
    CAIFQ_DECODE_CASE(8, 2, 2)
    CAIFQ_DECODE_CASE(8, 2, 4)
  }
#undef CAIFQ_DECODE_CASE
  set_error("frozen linear (decode): no kernel instance for in_dim=%d m=%lld", w.in_dim, static_cast<long long>(m));
  return CAIFQ_ERR_UNSUPPORTED;
}

}  // namespace caifq
