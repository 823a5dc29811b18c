// Weight-streaming frozen-linear forward for few tokens (decode shapes).
//
//   y[m, out] = x[m, in] . W_deq[out, in]^T      m <= 16, x bf16, y fp32/bf16/fp16
//
// The call is bound by reading the packed codes once from HBM
// (CAIF_DeviceFrozenLinear::ForwardImpl, src/caif_device_frozen_linear.cpp:381-524,
// does the same product after writing and re-reading an fp32 copy of the whole
// weight, :319-334).  Design:
//   * one persistent CTA per SM owns a contiguous range of rows of the
//     [out, in] code matrix, i.e. one contiguous slab of HBM, cut into items of
//     16 rows (the M of the tensor-core instruction);
//   * warp 0 streams that slab through a shared-memory ring with bulk async
//     copies (cp.async.bulk + mbarrier transaction counts): 100+ KB in flight
//     per SM regardless of register pressure;
//   * 16 warps split the reduction dimension; each lane pulls 16 bytes of codes
//     of rows g and g+8 from the ring, turns nibbles/bytes into exact bf16
//     integers with logic ops (no int->float converts), and feeds them as the A
//     operand of bf16 tensor-core MMAs against token fragments (B operand) that
//     stay in registers for the whole kernel;
//   * int4 group scales multiply the fp32 partial sum once per 128-element
//     chunk; the int8 per-tensor scale multiplies the final sum;
//   * the warps never synchronise with each other in the main loop: each parks
//     its partial sums of every item in shared memory, and one pass at the end
//     adds the 16 partials of each output.
// Codes and activations are exact in bf16 and products accumulate in fp32, so
// the result matches an fp32 GEMM on the dequantized weight up to summation
// order.
#include <atomic>

#include "common.cuh"

namespace caifq
{

__device__ unsigned int g_decode_timeout_flag = 0;

// Reads and clears the flag (1 = some bounded wait ran out since the last call; -1 = query failed).
int take_decode_timeout_flag()
{
  unsigned int v = 0;
  const unsigned int zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_decode_timeout_flag, sizeof(v)) != cudaSuccess)
  {
    return -1;
  }
  if (v != 0 && cudaMemcpyToSymbol(g_decode_timeout_flag, &zero, sizeof(zero)) != cudaSuccess)
  {
    return -1;
  }
  return v ? 1 : 0;
}

namespace
{

constexpr int kComputeWarps = 16;                // 4 per scheduler: the 128-register budget holds
constexpr int kThreads = kComputeWarps * 32;
constexpr int kItemRows = 16;                    // weight rows per work item (the MMA's M)
constexpr int kRowQuantum = 8;                   // CTA row ranges start on multiples of this
constexpr int kMaxStages = 8;
constexpr uint32_t kSmemBudget = 220u * 1024u;
constexpr uint32_t kSpinLimit = 1u << 22;

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

__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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

// D(16x8, fp32) += A(16x16, bf16, row) * B(16x8, bf16, col).  Not volatile: a
// pure function of its operands, so the compiler may interleave independent
// accumulation chains.
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1)
{
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
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

__device__ __forceinline__ uint32_t lop3_and_xor(uint32_t a, uint32_t b, uint32_t c)
{
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(a), "r"(b), "r"(c));  // (a & b) ^ c
  return d;
}

// Explicit shared-space accesses with 32-bit addresses.  Volatile keeps them in
// program order after the (volatile) barrier wait that guards the data.
__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

__device__ __forceinline__ float lds_half(uint32_t addr)
{
  unsigned short h;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"(addr));
  return __half2float(__ushort_as_half(h));
}

__device__ __forceinline__ float lds_f32(uint32_t addr)
{
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}

__device__ __forceinline__ void sts_f32(uint32_t addr, float a)
{
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(a) : "memory");
}

struct DecodeParams
{
  const uint8_t *codes;   // [out, in] packed
  const void *scales;     // int4: fp16 per group; int8: fp32[1] or null
  const __nv_bfloat16 *x; // [m, in]
  void *y[kMaxPeers];     // [m, y_ld] on every GPU that receives the result (own buffer included)
  int num_y;
  int64_t y_ld;           // row pitch of the result, in elements
  int64_t y_col0;         // first column this launch writes
  int y_dtype;
  int m;
  int in_dim;
  int out_dim;
  int groups_per_row;     // int4: in_dim / group_size
  int chunks_per_group;   // int4: group_size / 128
  int num_quanta;         // ceil(out / 8)
  int stages;
  uint32_t smem_bytes;     // dynamic shared memory of the launch
  uint32_t partial_offset; // byte offset of the partial sums in dynamic shared memory
  uint32_t row_bytes;      // packed bytes per weight row
  uint32_t row_stride;     // padded row pitch in the ring
  uint32_t stage_bytes;    // ring stage pitch
};

// int4 codes are turned into the bf16 integers 136 + q (q in [-8,7]): the
// nibble, flipped to offset binary, is dropped into the mantissa of 128.0.  The
// constant is taken out again by starting each accumulator at -136 * (sum of x
// over the same 128 elements), so no subtract runs per weight.
constexpr float kInt4Offset = 136.0f;

// BITS: 4 or 8.  MT: token tiles of 8 (1 -> m <= 8, 2 -> m <= 16).
// NCH: chunks (64 bytes of one row: a quad of lanes x 16 bytes) per warp.
template <int BITS, int MT, int NCH>
__global__ void __launch_bounds__(kThreads, 1) linear_decode_kernel(const DecodeParams p)
{
  constexpr int ELEMS = 128 / BITS;      // codes per 16-byte load: 32 or 16
  constexpr int CHUNK_K = 4 * ELEMS;     // k covered by a quad of lanes: 128 or 64
  constexpr int XR = ELEMS / 2;          // bf16x2 registers of x per chunk and token tile: 16 or 8
  constexpr int TOK = 8 * MT;
  constexpr uint32_t kPartWarpBytes = kItemRows * TOK * 4;            // one warp's sums of one item
  constexpr uint32_t kPartItemBytes = kComputeWarps * kPartWarpBytes;  // all warps' sums of one item

  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ uint64_t full_bar[kMaxStages];   // a stage's copies have landed
  __shared__ uint64_t empty_bar[kMaxStages];  // all 16 warps are done reading a stage

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int g = lane >> 2;  // A fragment rows g, g+8 (weight rows); B fragment column g (token)
  const int t = lane & 3;

  const int q_begin = static_cast<int>((static_cast<int64_t>(blockIdx.x) * p.num_quanta) / gridDim.x);
  const int q_end = static_cast<int>((static_cast<int64_t>(blockIdx.x + 1) * p.num_quanta) / gridDim.x);
  const int row_begin = q_begin * kRowQuantum;
  const int row_end = min(q_end * kRowQuantum, p.out_dim);
  const int my_items = (row_end - row_begin + kItemRows - 1) / kItemRows;
  const int num_chunks = p.in_dim / CHUNK_K;
  const int stages = p.stages;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t part_base = smem_base + p.partial_offset;

  if (tid == 0)
  {
    for (int s = 0; s < stages; ++s)
    {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kComputeWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // Producer: the item's rows are contiguous in memory, so one bulk copy brings
  // the codes and a second one the scales (two lanes of warp 0).
  auto issue = [&](int item, int s)
  {
    const int row0 = row_begin + item * kItemRows;
    const int rows = min(kItemRows, row_end - row0);
    uint8_t *stage = smem + static_cast<size_t>(s) * p.stage_bytes;
    const uint32_t code_bytes = static_cast<uint32_t>(rows) * p.row_bytes;
    const uint32_t scale_bytes = (BITS == 4) ? static_cast<uint32_t>(rows * p.groups_per_row * 2) : 0u;
    if (lane == 0)
    {
      mbar_expect_tx(&full_bar[s], code_bytes + scale_bytes);
      bulk_g2s(stage, p.codes + static_cast<size_t>(row0) * p.row_bytes, code_bytes, &full_bar[s]);
    }
    if (BITS == 4 && lane == 1)
    {
      const uint8_t *src = static_cast<const uint8_t *>(p.scales) + static_cast<size_t>(row0) * p.groups_per_row * 2;
      bulk_g2s(stage + static_cast<size_t>(kItemRows) * p.row_stride, src, scale_bytes, &full_bar[s]);
    }
  };
  if (warp == 0)
  {
    const int pre = min(stages, my_items);
    for (int i = 0; i < pre; ++i)
    {
      issue(i, i);
    }
  }

  // Programmatic dependent launch: the frozen codes and scales never depend on earlier work in
  // the stream, so their copies above may start while the previous kernel is still draining.
  // Activations and the output are touched only after that kernel has completed.  The next
  // kernel in the stream may begin its own weight copies as soon as this CTA's resources free up.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // Token fragments (B operand), resident for the whole kernel.  For the 16
  // bytes of codes a lane reads at k-offset kb, the register order pairs the
  // elements the way the logic-op dequantization emits them:
  //   int4, word wi: (8wi+0, 8wi+4) (8wi+2, 8wi+6) (8wi+1, 8wi+5) (8wi+3, 8wi+7)
  //   int8, word wi: (4wi+0, 4wi+2) (4wi+1, 4wi+3)
  uint32_t xf[NCH][MT][XR];
  float sx[NCH][MT][2];     // int4: -136 * (sum of x over the chunk's 128 elements), tokens 2t and 2t+1 of tile mt
  uint32_t code_off[NCH];   // byte offset of this lane's 16 bytes of row g inside a stage
  uint32_t scale_off[NCH];  // byte offset of row g's scale for the chunk inside a stage
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch)
  {
    const int cidx = warp + ch * kComputeWarps;
    code_off[ch] = static_cast<uint32_t>(g) * p.row_stride + static_cast<uint32_t>(cidx) * 64u + static_cast<uint32_t>(t) * 16u;
    scale_off[ch] = static_cast<uint32_t>(kItemRows) * p.row_stride +
                    static_cast<uint32_t>(g * p.groups_per_row + cidx / p.chunks_per_group) * 2u;
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
        float lane_sum = 0.0f;
#pragma unroll
        for (int i = 0; i < XR; ++i)
        {
          lane_sum += __uint_as_float(raw[i] << 16) + __uint_as_float(raw[i] & 0xFFFF0000u);
        }
        lane_sum += __shfl_xor_sync(0xFFFFFFFFu, lane_sum, 1);
        lane_sum += __shfl_xor_sync(0xFFFFFFFFu, lane_sum, 2);
        // every lane of quad g now holds the sum for token g (+8 mt); fetch tokens 2t, 2t+1
        sx[ch][mt][0] = -kInt4Offset * __shfl_sync(0xFFFFFFFFu, lane_sum, (2 * t) * 4);
        sx[ch][mt][1] = -kInt4Offset * __shfl_sync(0xFFFFFFFFu, lane_sum, (2 * t + 1) * 4);
#pragma unroll
        for (int wi = 0; wi < 4; ++wi)
        {
          xf[ch][mt][4 * wi + 0] = __byte_perm(raw[4 * wi + 0], raw[4 * wi + 2], 0x5410);
          xf[ch][mt][4 * wi + 1] = __byte_perm(raw[4 * wi + 1], raw[4 * wi + 3], 0x5410);
          xf[ch][mt][4 * wi + 2] = __byte_perm(raw[4 * wi + 0], raw[4 * wi + 2], 0x7632);
          xf[ch][mt][4 * wi + 3] = __byte_perm(raw[4 * wi + 1], raw[4 * wi + 3], 0x7632);
        }
      }
      else
      {
        sx[ch][mt][0] = 0.0f;
        sx[ch][mt][1] = 0.0f;
#pragma unroll
        for (int wi = 0; wi < 4; ++wi)
        {
          xf[ch][mt][2 * wi + 0] = __byte_perm(raw[2 * wi + 0], raw[2 * wi + 1], 0x5410);
          xf[ch][mt][2 * wi + 1] = __byte_perm(raw[2 * wi + 0], raw[2 * wi + 1], 0x7632);
        }
      }
    }
  }
  const uint32_t row8_off = 8u * p.row_stride;
  const uint32_t scale8_off = static_cast<uint32_t>(8 * p.groups_per_row) * 2u;
  // parked partial sums: [item][warp][token][row], rows fastest
  const uint32_t part_write_off =
      static_cast<uint32_t>(warp) * kPartWarpBytes + static_cast<uint32_t>(2 * t * kItemRows + g) * 4u;

  int s = 0;           // ring stage of the current item
  uint32_t s_par = 0;  // its phase parity
  for (int it = 0; it < my_items; ++it)
  {
    mbar_wait(&full_bar[s], s_par);
    const uint32_t stage_addr = smem_base + static_cast<uint32_t>(s) * p.stage_bytes;

    // all shared-memory reads of the item first, so the stage can be released
    // early and the MMAs of different chunks overlap
    uint32_t wlo[NCH][4];
    uint32_t whi[NCH][4];
    float s_lo[NCH];
    float s_hi[NCH];
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch)
    {
      if (warp + ch * kComputeWarps < num_chunks)
      {
        const uint4 lo = lds128(stage_addr + code_off[ch]);
        const uint4 hi = lds128(stage_addr + code_off[ch] + row8_off);
        wlo[ch][0] = lo.x;
        wlo[ch][1] = lo.y;
        wlo[ch][2] = lo.z;
        wlo[ch][3] = lo.w;
        whi[ch][0] = hi.x;
        whi[ch][1] = hi.y;
        whi[ch][2] = hi.z;
        whi[ch][3] = hi.w;
        if (BITS == 4)
        {
          s_lo[ch] = lds_half(stage_addr + scale_off[ch]);
          s_hi[ch] = lds_half(stage_addr + scale_off[ch] + scale8_off);
        }
      }
    }
    __syncwarp();
    if (lane == 0)
    {
      mbar_arrive(&empty_bar[s]);
    }

    // yacc[mt][0..1]: row g, tokens 2t, 2t+1 of tile mt;  [2..3]: row g+8
    float yacc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
    {
      yacc[mt][0] = yacc[mt][1] = yacc[mt][2] = yacc[mt][3] = 0.0f;
    }
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch)
    {
      if (warp + ch * kComputeWarps < num_chunks)
      {
        // two accumulation chains per token tile (even / odd words)
        float c[2][MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
        {
          c[0][mt][0] = c[0][mt][2] = (BITS == 4) ? sx[ch][mt][0] : 0.0f;  // -136 * sum(x): ends as sum(x * q)
          c[0][mt][1] = c[0][mt][3] = (BITS == 4) ? sx[ch][mt][1] : 0.0f;
          c[1][mt][0] = c[1][mt][1] = c[1][mt][2] = c[1][mt][3] = 0.0f;
        }
#pragma unroll
        for (int wi = 0; wi < 4; ++wi)
        {
          if (BITS == 4)
          {
            uint32_t a_lo[4];
            uint32_t a_hi[4];
            {
              const uint32_t ev = lop3_and_xor(wlo[ch][wi], 0x0F0F0F0Fu, 0x08080808u);
              const uint32_t od = lop3_and_xor(wlo[ch][wi] >> 4, 0x0F0F0F0Fu, 0x08080808u);
              a_lo[0] = __byte_perm(ev, 0x43434343u, 0x4240);
              a_lo[1] = __byte_perm(ev, 0x43434343u, 0x4341);
              a_lo[2] = __byte_perm(od, 0x43434343u, 0x4240);
              a_lo[3] = __byte_perm(od, 0x43434343u, 0x4341);
            }
            {
              const uint32_t ev = lop3_and_xor(whi[ch][wi], 0x0F0F0F0Fu, 0x08080808u);
              const uint32_t od = lop3_and_xor(whi[ch][wi] >> 4, 0x0F0F0F0Fu, 0x08080808u);
              a_hi[0] = __byte_perm(ev, 0x43434343u, 0x4240);
              a_hi[1] = __byte_perm(ev, 0x43434343u, 0x4341);
              a_hi[2] = __byte_perm(od, 0x43434343u, 0x4240);
              a_hi[3] = __byte_perm(od, 0x43434343u, 0x4341);
            }
#pragma unroll
            for (int h = 0; h < 2; ++h)
            {
              const int j = 2 * wi + h;  // k-step: pairs 2j, 2j+1
#pragma unroll
              for (int mt = 0; mt < MT; ++mt)
              {
                mma_bf16_16816(c[h][mt], a_lo[2 * h], a_hi[2 * h], a_lo[2 * h + 1], a_hi[2 * h + 1],
                               xf[ch][mt][2 * j], xf[ch][mt][2 * j + 1]);
              }
            }
          }
          else
          {
            uint32_t a_lo[2];
            uint32_t a_hi[2];
#pragma unroll
            for (int sh = 0; sh < 2; ++sh)
            {
              const uint32_t sel = sh ? 0x4341u : 0x4240u;
              const uint32_t pl = __byte_perm(wlo[ch][wi], 0u, sel);
              const uint32_t ph = __byte_perm(whi[ch][wi], 0u, sel);
              a_lo[sh] = sub_bf16x2(lop3_and_or(pl, 0x007F007Fu, 0x43004300u), lop3_and_or(pl, 0x00800080u, 0x43004300u));
              a_hi[sh] = sub_bf16x2(lop3_and_or(ph, 0x007F007Fu, 0x43004300u), lop3_and_or(ph, 0x00800080u, 0x43004300u));
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
            {
              mma_bf16_16816(c[wi & 1][mt], a_lo[0], a_hi[0], a_lo[1], a_hi[1], xf[ch][mt][2 * wi],
                             xf[ch][mt][2 * wi + 1]);
            }
          }
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
        {
          if (BITS == 4)
          {
            // the chunk lies inside one scale group of rows g and g+8; scaling per
            // 128-element chunk equals scaling per group up to rounding order
            yacc[mt][0] = fmaf(s_lo[ch], c[0][mt][0] + c[1][mt][0], yacc[mt][0]);
            yacc[mt][1] = fmaf(s_lo[ch], c[0][mt][1] + c[1][mt][1], yacc[mt][1]);
            yacc[mt][2] = fmaf(s_hi[ch], c[0][mt][2] + c[1][mt][2], yacc[mt][2]);
            yacc[mt][3] = fmaf(s_hi[ch], c[0][mt][3] + c[1][mt][3], yacc[mt][3]);
          }
          else
          {
#pragma unroll
            for (int i = 0; i < 4; ++i)
            {
              yacc[mt][i] += c[0][mt][i] + c[1][mt][i];
            }
          }
        }
      }
    }
    // park this warp's partial sums of the item; nobody reads them before the end
    const uint32_t dst = part_base + static_cast<uint32_t>(it) * kPartItemBytes + part_write_off;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
    {
      const uint32_t d = dst + static_cast<uint32_t>(8 * mt * kItemRows) * 4u;
      sts_f32(d, yacc[mt][0]);                         // token 2t,   row g
      sts_f32(d + kItemRows * 4u, yacc[mt][1]);        // token 2t+1, row g
      sts_f32(d + 8u * 4u, yacc[mt][2]);               // token 2t,   row g+8
      sts_f32(d + (kItemRows + 8u) * 4u, yacc[mt][3]); // token 2t+1, row g+8
    }
    // warp 0 refills this item's stage once all warps have read it (they read
    // it at the top of the iteration, so by now this rarely waits)
    if (warp == 0 && it + stages < my_items)
    {
      mbar_wait(&empty_bar[s], s_par);
      issue(it + stages, s);
    }
    if (++s == stages)
    {
      s = 0;
      s_par ^= 1u;
    }
  }
  __syncthreads();

  // Cross-warp reduction: output (item, token, row) = sum over the 16 warps.
  float tensor_scale = 1.0f;
  if (BITS == 8 && p.scales != nullptr)
  {
    tensor_scale = static_cast<const float *>(p.scales)[0];
  }
  const int outputs = my_items * kItemRows * TOK;
  for (int o = tid; o < outputs; o += kThreads)
  {
    const int r = o % kItemRows;
    const int token = (o / kItemRows) % TOK;
    const int item = o / (kItemRows * TOK);
    const uint32_t src =
        part_base + static_cast<uint32_t>(item) * kPartItemBytes + static_cast<uint32_t>(token * kItemRows + r) * 4u;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int w = 0; w < kComputeWarps; ++w)
    {
      acc[w & 3] += lds_f32(src + static_cast<uint32_t>(w) * kPartWarpBytes);
    }
    float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    if (BITS == 8)
    {
      sum *= tensor_scale;
    }
    const int row = row_begin + item * kItemRows + r;
    if (token < p.m && row < row_end)
    {
      // plain stores; with peers they travel over NVLink and are complete when the kernel is
      const int64_t idx = static_cast<int64_t>(token) * p.y_ld + p.y_col0 + row;
      for (int r = 0; r < p.num_y; ++r)
      {
        store_from_float(p.y[r], idx, p.y_dtype, sum);
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
    // A host that runs a collective beside this kernel (column-parallel decode) can leave it a few
    // SMs: the kernel keeps one CTA per SM, and a CTA that finds its SM taken waits for the whole
    // collective.  CAIFQ_DECODE_CTAS caps the grid.
    if (const char *e = std::getenv("CAIFQ_DECODE_CTAS"))
    {
      const int v = std::atoi(e);
      if (v >= 1 && v < cached)
      {
        cached = v;
      }
    }
  }
  return cached;
}

}  // namespace

namespace
{
std::atomic<bool> g_codes_written{false};
}

void note_codes_written() { g_codes_written.store(true, std::memory_order_relaxed); }

bool take_codes_written() { return g_codes_written.exchange(false, std::memory_order_relaxed); }

namespace
{

template <int BITS, int MT, int NCH>
int launch_decode_inst(const DecodeParams &p, cudaStream_t s)
{
  auto kernel = linear_decode_kernel<BITS, MT, NCH>;
  const size_t smem = p.smem_bytes;
  static bool configured = false;
  if (!configured)
  {
    CAIFQ_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
    configured = true;
  }
  int grid = sm_count();
  if (grid > p.num_quanta)
  {
    grid = p.num_quanta;
  }
  static const bool pdl = []() {
    const char *e = std::getenv("CAIFQ_PDL");
    return e == nullptr || e[0] != '0';
  }();
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl && !take_codes_written()) ? 1 : 0;
  CAIFQ_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

// Shared memory for the parked partial sums: the largest number of items any CTA gets.
uint32_t partial_bytes_for(int out_dim, int mt)
{
  const int quanta = (out_dim + kRowQuantum - 1) / kRowQuantum;
  int grid = sm_count();
  if (grid > quanta)
  {
    grid = quanta;
  }
  const int max_quanta = (quanta + grid - 1) / grid;
  const int max_items = (max_quanta * kRowQuantum + kItemRows - 1) / kItemRows;
  return static_cast<uint32_t>(max_items * kComputeWarps * kItemRows * 8 * mt * sizeof(float));
}

int chunks_per_warp(const caifq_weight &w)
{
  const int chunk_k = (w.storage == CAIFQ_I4) ? 128 : 64;
  const int chunks = w.in_dim / chunk_k;
  return (chunks + kComputeWarps - 1) / kComputeWarps;
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
    // a ragged last item copies rows * groups_per_row fp16 scales: keep that a 16-byte multiple
    if ((w.out_dim % kRowQuantum) != 0 && ((w.in_dim / w.group_size) % 8) != 0)
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
  // at least two ring stages must fit beside the partial-sum buffers
  {
    const uint32_t row_bytes = (w.storage == CAIFQ_I4) ? static_cast<uint32_t>(w.in_dim / 2) : static_cast<uint32_t>(w.in_dim);
    const uint32_t row_stride = row_bytes;
    const uint32_t scale_bytes =
        (w.storage == CAIFQ_I4) ? static_cast<uint32_t>(kItemRows * (w.in_dim / w.group_size) * 2) : 0u;
    const uint32_t stage_bytes = ((kItemRows * row_stride + scale_bytes) + 127u) & ~127u;
    if (2u * stage_bytes + partial_bytes_for(w.out_dim, mt) > kSmemBudget)
    {
      return false;
    }
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
  if (args.num_peers > 0)
  {
    if (args.num_peers > kMaxPeers || args.c_peers == nullptr)
    {
      set_error("frozen linear (decode): at most %d peers", kMaxPeers);
      return CAIFQ_ERR_INVALID;
    }
    for (int r = 0; r < args.num_peers; ++r)
    {
      if (args.c_peers[r] == nullptr)
      {
        set_error("frozen linear (decode): null peer buffer %d", r);
        return CAIFQ_ERR_INVALID;
      }
      p.y[r] = args.c_peers[r];
    }
    p.num_y = args.num_peers;
    p.y_ld = args.c_ld;
    p.y_col0 = args.c_col0;
  }
  else
  {
    p.y[0] = y;
    p.num_y = 1;
    p.y_ld = w.out_dim;
    p.y_col0 = 0;
  }
  p.y_dtype = y_dtype;
  p.m = static_cast<int>(m);
  p.in_dim = w.in_dim;
  p.out_dim = w.out_dim;
  p.num_quanta = (w.out_dim + kRowQuantum - 1) / kRowQuantum;
  const bool i4 = (w.storage == CAIFQ_I4);
  p.row_bytes = i4 ? static_cast<uint32_t>(w.in_dim / 2) : static_cast<uint32_t>(w.in_dim);
  // rows lie unpadded, as in memory, so one bulk copy fills a stage; the 2-way
  // bank conflict on the four 16-byte reads per item is noise
  p.row_stride = p.row_bytes;
  uint32_t scale_bytes = 0;
  if (i4)
  {
    p.groups_per_row = w.in_dim / w.group_size;
    p.chunks_per_group = w.group_size / 128;
    scale_bytes = static_cast<uint32_t>(kItemRows * p.groups_per_row * 2);
  }
  else
  {
    p.groups_per_row = 0;
    p.chunks_per_group = 1;
  }
  p.stage_bytes = ((kItemRows * p.row_stride + scale_bytes) + 127u) & ~127u;
  const uint32_t partial_bytes = partial_bytes_for(w.out_dim, (m > 8) ? 2 : 1);
  int stages = static_cast<int>((kSmemBudget - partial_bytes) / p.stage_bytes);
  if (stages > kMaxStages)
  {
    stages = kMaxStages;
  }
  if (const char *e = std::getenv("CAIFQ_DECODE_STAGES"))
  {
    const int v = std::atoi(e);
    if (v >= 2 && v < stages)
    {
      stages = v;
    }
  }
  if (stages < 2)
  {
    set_error("frozen linear (decode): row too long for the shared-memory ring");
    return CAIFQ_ERR_UNSUPPORTED;
  }
  p.stages = stages;
  p.partial_offset = static_cast<uint32_t>(stages) * p.stage_bytes;
  p.smem_bytes = p.partial_offset + partial_bytes;

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
