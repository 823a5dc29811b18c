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
//   * the slab streams through a shared-memory ring of three items with bulk
//     async copies (cp.async.bulk + mbarrier transaction counts), started before
//     the kernel waits for the previous kernel in the stream (programmatic
//     dependent launch): the frozen codes never depend on earlier work;
//   * 16 warps split the reduction dimension; each lane pulls 16 bytes of codes
//     of rows g and g+8 from the ring, turns nibbles/bytes into exact bf16
//     integers with logic ops (no int->float converts), and feeds them as the A
//     operand of bf16 tensor-core MMAs against token fragments (B operand) that
//     stay in registers for the whole kernel;
//   * int4 group scales multiply the fp32 partial sum once per 128-element
//     chunk; the int8 per-tensor scale multiplies the final sum;
//   * the warps never synchronise with each other in the main loop: each parks
//     its partial sums of every item (live tokens only) in shared memory, and
//     one pass at the end adds the 16 partials of each output in a fixed order
//     and stores four rows (or, for 9 to 16 tokens, one row of four tokens) per
//     thread.
// After the previous kernel has completed the launch is bound by the logic ops
// of the dequantization (two cycles per warp instruction on this GPU, seven of
// them per eight int4 weights), not by HBM: see the design notes of the package.
// Codes and activations are exact in bf16 and products accumulate in fp32, so
// the result matches an fp32 GEMM on the dequantized weight up to summation
// order.  The summation order of an output does not depend on which CTA owns
// its row, so a row slice of a layer gives the same bits as the whole layer.
#include <atomic>
#include <mutex>
#include <vector>

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

constexpr int kItemRows = 16;                    // weight rows per work item (the MMA's M)
constexpr int kRowQuantum = 8;                   // CTA row ranges start on multiples of this
constexpr int kMaxStages = 8;
constexpr int kWarps = 16;                       // 4 per scheduler: the 128-register budget holds
constexpr int kThreads = kWarps * 32;
constexpr int kRingDepth = 3;                    // items in flight per SM
constexpr uint32_t kSmemBudget = 220u * 1024u;   // dynamic shared memory of the one CTA per SM
constexpr uint32_t kSpinLimit = 1u << 22;        // polls of one wait before it gives up (tens of ms)
constexpr uint32_t kSpinLimitTest = 1u << 12;    // the same for the self-test of the give-up path

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

__device__ __forceinline__ bool mbar_try(uint32_t addr, uint32_t parity)
{
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(addr), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait, called by all lanes of a warp.  Gives up after `limit` polls, or as soon as
// another warp of the CTA has given up, and says so: a copy that never lands turns into a
// flag and missing outputs instead of a hung GPU.  The answer is the same in every lane.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t limit, volatile uint32_t *abort_word)
{
  const uint32_t addr = smem_u32(bar);
  bool done = mbar_try(addr, parity);
  if (!done)
  {
    for (uint32_t spin = 0; spin < limit && !done; ++spin)
    {
      done = mbar_try(addr, parity);
      if (!done && (spin & 255u) == 255u && *abort_word != 0u)
      {
        break;
      }
    }
  }
  done = __all_sync(0xFFFFFFFFu, done);
  if (!done)
  {
    *abort_word = 1u;
    atomicExch(&g_decode_timeout_flag, 1u);
  }
  return done;
}

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint64_t *bar)
{
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
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

__device__ __forceinline__ void sts_f32x2(uint32_t addr, float a, float b)
{
  asm volatile("st.shared.v2.f32 [%0], {%1,%2};" ::"r"(addr), "f"(a), "f"(b) : "memory");
}


constexpr int kMaxSegments = 4;   // code matrices one launch may stream (layers that share their input)

struct DecodeParams
{
  // The rows of the launch are the rows of up to kMaxSegments code matrices laid end to end (q/k/v or
  // gate/up of one input): segment i covers rows seg_row0[i] .. seg_row0[i+1]; a single layer is one segment.
  const uint8_t *codes[kMaxSegments];   // [out_i, in] packed
  const void *scales[kMaxSegments];     // int4: fp16 per group; int8: fp32[1] or null
  int seg_row0[kMaxSegments + 1];
  int num_seg;
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
  int vec4;               // fp32 results may be stored four rows at a time (16-byte aligned on every buffer)
  int tokp;               // tokens per parked row: m rounded up to 2, 4, 8 or 16
  int park_items;         // items whose partial sums fit the parking area: the CTA reduces and stores that often
  uint32_t partial_offset; // byte offset of the parked partial sums in dynamic shared memory
  uint32_t row_bytes;      // packed bytes per weight row
  uint32_t row_stride;     // row pitch in the ring
  uint32_t stage_bytes;    // ring stage pitch
  uint32_t spin_limit;     // polls of one wait before it gives up
  uint32_t stall_bytes;    // self-test only: bytes the first item announces but never receives
};

// int4 codes are turned into the bf16 integers 136 + q (q in [-8,7]): the
// nibble, flipped to offset binary, is dropped into the mantissa of 128.0.  The
// constant is taken out again by starting each accumulator at -136 * (sum of x
// over the same 128 elements), so no subtract runs per weight.
constexpr float kInt4Offset = 136.0f;

// BITS: 4 or 8.  MT: token tiles of 8 (1 -> m <= 8, 2 -> m <= 16).
// NCH: chunks (64 bytes of one row: a quad of lanes x 16 bytes) per warp.
template <int BITS, int MT, int NCH>
__global__ void __launch_bounds__(kThreads, 1) linear_decode_kernel(const __grid_constant__ DecodeParams p)
{
  constexpr int ELEMS = 128 / BITS;      // codes per 16-byte load: 32 or 16
  constexpr int CHUNK_K = 4 * ELEMS;     // k covered by a quad of lanes: 128 or 64
  constexpr int XR = ELEMS / 2;          // bf16x2 registers of x per chunk and token tile: 16 or 8
  constexpr int WARPS = kWarps;
  constexpr int CHAINS = (MT == 1) ? 2 : 1;   // accumulation chains per token tile

  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ uint64_t full_bar[kMaxStages];   // a stage's copies have landed
  __shared__ uint64_t empty_bar[kMaxStages];  // all warps are done reading a stage
  __shared__ uint32_t cta_abort;              // a wait of this CTA has run out

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
  volatile uint32_t *abort_word = &cta_abort;

  // One thread starts the copies of an item: its rows are contiguous in memory, so one bulk copy
  // brings the codes and a second one the scales.
  auto issue = [&](int item, int s)
  {
    const int row0 = row_begin + item * kItemRows;
    const int rows = min(kItemRows, row_end - row0);
    const uint32_t stage = smem_base + static_cast<uint32_t>(s) * p.stage_bytes;
    const uint32_t code_bytes = static_cast<uint32_t>(rows) * p.row_bytes;
    const uint32_t scale_bytes = (BITS == 4) ? static_cast<uint32_t>(rows * p.groups_per_row * 2) : 0u;
    mbar_expect_tx(&full_bar[s], code_bytes + scale_bytes + (item == 0 ? p.stall_bytes : 0u));
    if (p.num_seg == 1)
    {
      bulk_g2s(stage, p.codes[0] + static_cast<size_t>(row0) * p.row_bytes, code_bytes, &full_bar[s]);
      if (BITS == 4)
      {
        const uint8_t *src = static_cast<const uint8_t *>(p.scales[0]) + static_cast<size_t>(row0) * p.groups_per_row * 2;
        bulk_g2s(stage + static_cast<uint32_t>(kItemRows) * p.row_stride, src, scale_bytes, &full_bar[s]);
      }
      return;
    }
    // an item that straddles two code matrices takes one pair of copies from each
    int row = row0;
    while (row < row0 + rows)
    {
      int sg = 0;
      while (sg + 1 < p.num_seg && row >= p.seg_row0[sg + 1])
      {
        ++sg;
      }
      const int n = min(row0 + rows, p.seg_row0[sg + 1]) - row;
      const size_t local = static_cast<size_t>(row - p.seg_row0[sg]);
      const uint32_t done_rows = static_cast<uint32_t>(row - row0);
      bulk_g2s(stage + done_rows * p.row_bytes, p.codes[sg] + local * p.row_bytes, static_cast<uint32_t>(n) * p.row_bytes,
               &full_bar[s]);
      if (BITS == 4)
      {
        const uint32_t per_row = static_cast<uint32_t>(p.groups_per_row) * 2u;
        const uint8_t *src = static_cast<const uint8_t *>(p.scales[sg]) + local * per_row;
        bulk_g2s(stage + static_cast<uint32_t>(kItemRows) * p.row_stride + done_rows * per_row, src,
                 static_cast<uint32_t>(n) * per_row, &full_bar[s]);
      }
      row += n;
    }
  };

  if (tid == 0)
  {
    cta_abort = 0u;
    for (int s = 0; s < stages; ++s)
    {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // The frozen codes and scales never depend on earlier work in the stream: the ring starts before
  // the wait on the previous kernel.  The next kernel in the stream may place its CTAs as soon as
  // this grid's CTAs have all come this far (programmatic dependent launch).
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // Warp 0 is the only producer; it knows how many items it has started (needed if it gives up).
  int issued_items = min(stages, my_items);
  if (tid == 0)
  {
    for (int i = 0; i < issued_items; ++i)
    {
      issue(i, i);
    }
  }

  // Activations and the output are touched only after the previous kernel has completed.
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
    const int cidx = warp + ch * WARPS;
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
#pragma unroll
        for (int wi = 0; wi < 4; ++wi)
        {
          xf[ch][mt][4 * wi + 0] = __byte_perm(raw[4 * wi + 0], raw[4 * wi + 2], 0x5410);
          xf[ch][mt][4 * wi + 1] = __byte_perm(raw[4 * wi + 1], raw[4 * wi + 3], 0x5410);
          xf[ch][mt][4 * wi + 2] = __byte_perm(raw[4 * wi + 0], raw[4 * wi + 2], 0x7632);
          xf[ch][mt][4 * wi + 3] = __byte_perm(raw[4 * wi + 1], raw[4 * wi + 3], 0x7632);
        }
        {
          float lane_sum = 0.0f;
#pragma unroll
          for (int i = 0; i < XR; ++i)
          {
            lane_sum += __uint_as_float(raw[i] << 16) + __uint_as_float(raw[i] & 0xFFFF0000u);
          }
          lane_sum += __shfl_xor_sync(0xFFFFFFFFu, lane_sum, 1);
          lane_sum += __shfl_xor_sync(0xFFFFFFFFu, lane_sum, 2);
          sx[ch][mt][0] = -kInt4Offset * __shfl_sync(0xFFFFFFFFu, lane_sum, (2 * t) * 4);
          sx[ch][mt][1] = -kInt4Offset * __shfl_sync(0xFFFFFFFFu, lane_sum, (2 * t + 1) * 4);
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
  // parked partial sums: [item][warp][row][token], tokens fastest and only the live ones (tokp of
  // them): a lane's two tokens of a row are one 8-byte store.  With 16 tokens the groups of four
  // tokens of a row are stored in an order that depends on the row (quad ^ ((row >> 1) & 3)), so that
  // the 16-byte reads of the final reduction, eight rows at a time, fall into different banks.
  const uint32_t part_warp_bytes = static_cast<uint32_t>(kItemRows * p.tokp) * 4u;
  const uint32_t part_item_bytes = WARPS * part_warp_bytes;
  uint32_t part_write_off[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
  {
    if (MT == 2)
    {
      const int quad = ((t >> 1) + 2 * mt) ^ ((g >> 1) & 3);
      part_write_off[mt] = static_cast<uint32_t>(warp) * part_warp_bytes +
                           static_cast<uint32_t>(g * 16 + 4 * quad + 2 * (t & 1)) * 4u;
    }
    else
    {
      part_write_off[mt] =
          static_cast<uint32_t>(warp) * part_warp_bytes + static_cast<uint32_t>(g * p.tokp + 2 * t) * 4u;
    }
  }
  // int8: the per-tensor scale of every segment; an output row takes the one of its segment
  float seg_scale[kMaxSegments];
#pragma unroll
  for (int sg = 0; sg < kMaxSegments; ++sg)
  {
    seg_scale[sg] = 1.0f;
    if (BITS == 8 && sg < p.num_seg && p.scales[sg] != nullptr)
    {
      seg_scale[sg] = static_cast<const float *>(p.scales[sg])[0];
    }
  }
  auto tensor_scale_of = [&](int row)
  {
    float v = seg_scale[0];
#pragma unroll
    for (int sg = 1; sg < kMaxSegments; ++sg)
    {
      if (sg < p.num_seg && row >= p.seg_row0[sg])
      {
        v = seg_scale[sg];
      }
    }
    return v;
  };
  int s = 0;             // ring stage of the current item
  uint32_t s_par = 0;    // its phase parity
  bool ok = true;
  // Rounds: the parking area holds the partial sums of park_items items (all of a CTA's items for the
  // usual layer sizes, so one round); after each round the CTA adds them up and stores the outputs.
  for (int round_begin = 0; round_begin < my_items; round_begin += p.park_items)
  {
  const int round_end = min(round_begin + p.park_items, my_items);
  for (int it = round_begin; it < round_end; ++it)
  {
    ok = mbar_wait(&full_bar[s], s_par, p.spin_limit, abort_word);
    if (!ok)
    {
      break;
    }
    const uint32_t stage_addr = smem_base + static_cast<uint32_t>(s) * p.stage_bytes;
    // yacc[mt][0..1]: row g, tokens 2t, 2t+1 of tile mt;  [2..3]: row g+8
    float yacc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
    {
      yacc[mt][0] = yacc[mt][1] = yacc[mt][2] = yacc[mt][3] = 0.0f;
    }

    // all shared-memory reads of the item first, so the stage can be released early and the
    // MMAs of different chunks overlap
    uint32_t wlo_all[NCH][4];
    uint32_t whi_all[NCH][4];
    float s_lo_all[NCH];
    float s_hi_all[NCH];
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch)
    {
      s_lo_all[ch] = 0.0f;
      s_hi_all[ch] = 0.0f;
      if (warp + ch * WARPS < num_chunks)
      {
        const uint4 lo = lds128(stage_addr + code_off[ch]);
        const uint4 hi = lds128(stage_addr + code_off[ch] + row8_off);
        wlo_all[ch][0] = lo.x;
        wlo_all[ch][1] = lo.y;
        wlo_all[ch][2] = lo.z;
        wlo_all[ch][3] = lo.w;
        whi_all[ch][0] = hi.x;
        whi_all[ch][1] = hi.y;
        whi_all[ch][2] = hi.z;
        whi_all[ch][3] = hi.w;
        if (BITS == 4)
        {
          s_lo_all[ch] = lds_half(stage_addr + scale_off[ch]);
          s_hi_all[ch] = lds_half(stage_addr + scale_off[ch] + scale8_off);
        }
      }
    }
    // every read of the stage has been issued: count this warp out
    __syncwarp();
    if (lane == 0)
    {
      mbar_arrive(&empty_bar[s]);
    }
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch)
    {
      const uint32_t(&wlo)[4] = wlo_all[ch];
      const uint32_t(&whi)[4] = whi_all[ch];
      const float s_lo = s_lo_all[ch];
      const float s_hi = s_hi_all[ch];
      if (warp + ch * WARPS < num_chunks)
      {
        float c[CHAINS][MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
        {
          c[0][mt][0] = c[0][mt][2] = (BITS == 4) ? sx[ch][mt][0] : 0.0f;  // -136 * sum(x): ends as sum(x * q)
          c[0][mt][1] = c[0][mt][3] = (BITS == 4) ? sx[ch][mt][1] : 0.0f;
          if (CHAINS == 2)
          {
            c[CHAINS - 1][mt][0] = c[CHAINS - 1][mt][1] = c[CHAINS - 1][mt][2] = c[CHAINS - 1][mt][3] = 0.0f;
          }
        }
#pragma unroll
        for (int wi = 0; wi < 4; ++wi)
        {
          if (BITS == 4)
          {
            uint32_t a_lo[4];
            uint32_t a_hi[4];
            {
              const uint32_t ev = lop3_and_xor(wlo[wi], 0x0F0F0F0Fu, 0x08080808u);
              const uint32_t od = lop3_and_xor(wlo[wi] >> 4, 0x0F0F0F0Fu, 0x08080808u);
              a_lo[0] = __byte_perm(ev, 0x43434343u, 0x4240);
              a_lo[1] = __byte_perm(ev, 0x43434343u, 0x4341);
              a_lo[2] = __byte_perm(od, 0x43434343u, 0x4240);
              a_lo[3] = __byte_perm(od, 0x43434343u, 0x4341);
            }
            {
              const uint32_t ev = lop3_and_xor(whi[wi], 0x0F0F0F0Fu, 0x08080808u);
              const uint32_t od = lop3_and_xor(whi[wi] >> 4, 0x0F0F0F0Fu, 0x08080808u);
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
                mma_bf16_16816(c[h % CHAINS][mt], a_lo[2 * h], a_hi[2 * h], a_lo[2 * h + 1], a_hi[2 * h + 1],
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
              const uint32_t pl = __byte_perm(wlo[wi], 0u, sel);
              const uint32_t ph = __byte_perm(whi[wi], 0u, sel);
              a_lo[sh] = sub_bf16x2(lop3_and_or(pl, 0x007F007Fu, 0x43004300u), lop3_and_or(pl, 0x00800080u, 0x43004300u));
              a_hi[sh] = sub_bf16x2(lop3_and_or(ph, 0x007F007Fu, 0x43004300u), lop3_and_or(ph, 0x00800080u, 0x43004300u));
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
            {
              mma_bf16_16816(c[wi % CHAINS][mt], a_lo[0], a_hi[0], a_lo[1], a_hi[1], xf[ch][mt][2 * wi],
                             xf[ch][mt][2 * wi + 1]);
            }
          }
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
        {
          float sum[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
          {
            sum[i] = (CHAINS == 2) ? (c[0][mt][i] + c[CHAINS - 1][mt][i]) : c[0][mt][i];
          }
          if (BITS == 4)
          {
            // the chunk lies inside one scale group of rows g and g+8; scaling per
            // 128-element chunk equals scaling per group up to rounding order
            yacc[mt][0] = fmaf(s_lo, sum[0], yacc[mt][0]);
            yacc[mt][1] = fmaf(s_lo, sum[1], yacc[mt][1]);
            yacc[mt][2] = fmaf(s_hi, sum[2], yacc[mt][2]);
            yacc[mt][3] = fmaf(s_hi, sum[3], yacc[mt][3]);
          }
          else
          {
#pragma unroll
            for (int i = 0; i < 4; ++i)
            {
              yacc[mt][i] += sum[i];
            }
          }
        }
      }
    }
    // park this warp's partial sums of the item; nobody reads them before the end of the kernel
    {
      const uint32_t d0 = part_base + static_cast<uint32_t>(it - round_begin) * part_item_bytes;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
      {
        if (MT == 2 || 2 * t < p.tokp)
        {
          const uint32_t d = d0 + part_write_off[mt];
          sts_f32x2(d, yacc[mt][0], yacc[mt][1]);                                        // row g,   tokens 2t, 2t+1
          sts_f32x2(d + static_cast<uint32_t>(8 * p.tokp) * 4u, yacc[mt][2], yacc[mt][3]);  // row g+8
        }
      }
    }
    // warp 0 refills this item's stage once all warps have read it (they read it at the top of the
    // iteration, so by now this rarely waits)
    if (warp == 0 && it + stages < my_items)
    {
      ok = mbar_wait(&empty_bar[s], s_par, p.spin_limit, abort_word);
      if (!ok)
      {
        break;
      }
      if (lane == 0)
      {
        issue(it + stages, s);
      }
      issued_items = it + stages + 1;
    }

    if (++s == stages)
    {
      s = 0;
      s_par ^= 1u;
    }
  }
  __syncthreads();
  if (*abort_word != 0u)
  {
    // A wait ran out somewhere in the CTA; the outputs stay unwritten and the host sees the flag.
    // Before the CTA gives its shared memory back, every copy that was started into the ring must
    // have landed (a copy must not arrive in memory that already belongs to another CTA).  Warp 0
    // started them all and waits for them; these waits are bounded too.
    if (warp == 0)
    {
      for (int st = 0; st < stages && st < issued_items; ++st)
      {
        // the last item started into this stage; once it has landed the earlier ones have too
        const int j = issued_items - 1 - ((issued_items - 1 - st) % stages);
        const uint32_t addr = smem_u32(&full_bar[st]);
        const uint32_t parity = static_cast<uint32_t>(j / stages) & 1u;
        bool done = false;
        for (uint32_t spin = 0; spin < p.spin_limit && !done; ++spin)
        {
          done = mbar_try(addr, parity);
        }
      }
    }
    return;
  }

  // Cross-warp reduction: an output is the sum of its WARPS partial sums in warp order.
  if (MT == 2)
  {
    // a thread takes four tokens of one row; consecutive lanes take consecutive rows, so the stores
    // of a token are contiguous across the warp
    const int n = (round_end - round_begin) * 64;
    for (int o = tid; o < n; o += WARPS * 32)
    {
      const int r16 = o & 15;
      const int tq = (o >> 4) & 3;
      const int item = o >> 6;
      const int quad = tq ^ ((r16 >> 1) & 3);
      const uint32_t src = part_base + static_cast<uint32_t>(item) * part_item_bytes +
                           static_cast<uint32_t>(r16 * 16 + 4 * quad) * 4u;
      float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int w = 0; w < WARPS; ++w)
      {
        const uint4 v = lds128(src + static_cast<uint32_t>(w) * part_warp_bytes);
        acc[0] += __uint_as_float(v.x);
        acc[1] += __uint_as_float(v.y);
        acc[2] += __uint_as_float(v.z);
        acc[3] += __uint_as_float(v.w);
      }
      const int row = row_begin + (round_begin + item) * kItemRows + r16;
      if (row < row_end)
      {
        const float tensor_scale = (BITS == 8) ? tensor_scale_of(row) : 1.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i)
        {
          const int token = 4 * tq + i;
          if (token < p.m)
          {
            const float v = (BITS == 8) ? acc[i] * tensor_scale : acc[i];
            const int64_t idx = static_cast<int64_t>(token) * p.y_ld + p.y_col0 + row;
            for (int r = 0; r < p.num_y; ++r)
            {
              store_from_float(p.y[r], idx, p.y_dtype, v);
            }
          }
        }
      }
    }
  }
  else
  {
    // a thread takes four consecutive rows of one live token
    const int quads = (round_end - round_begin) * 4 * p.m;
    for (int o = tid; o < quads; o += WARPS * 32)
    {
      const int rq = o & 3;
      const int token = (o >> 2) % p.m;
      const int item = (o >> 2) / p.m;
      const uint32_t src = part_base + static_cast<uint32_t>(item) * part_item_bytes +
                           static_cast<uint32_t>((4 * rq) * p.tokp + token) * 4u;
      float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int w = 0; w < WARPS; ++w)
      {
#pragma unroll
        for (int i = 0; i < 4; ++i)
        {
          acc[i] += lds_f32(src + static_cast<uint32_t>(w) * part_warp_bytes + static_cast<uint32_t>(i * p.tokp) * 4u);
        }
      }
      const int row = row_begin + (round_begin + item) * kItemRows + 4 * rq;
      if (BITS == 8)
      {
        // (four rows that start on a multiple of four lie in one segment: segments start on multiples of 8)
        const float tensor_scale = tensor_scale_of(row);
#pragma unroll
        for (int i = 0; i < 4; ++i)
        {
          acc[i] *= tensor_scale;
        }
      }
      // plain stores; with peers they travel over NVLink and are complete when the kernel is
      const int64_t idx = static_cast<int64_t>(token) * p.y_ld + p.y_col0 + row;
      if (p.vec4 && row + 3 < row_end)
      {
        const float4 v = make_float4(acc[0], acc[1], acc[2], acc[3]);
        for (int r = 0; r < p.num_y; ++r)
        {
          *reinterpret_cast<float4 *>(static_cast<float *>(p.y[r]) + idx) = v;
        }
      }
      else
      {
#pragma unroll
        for (int i = 0; i < 4; ++i)
        {
          if (row + i < row_end)
          {
            for (int r = 0; r < p.num_y; ++r)
            {
              store_from_float(p.y[r], idx + i, p.y_dtype, acc[i]);
            }
          }
        }
      }
    }
  }
  if (round_end < my_items)
  {
    __syncthreads();   // the parking area is free for the next round
  }
  }  // rounds
}

// One CTA per SM, fewer when the host runs a collective beside this kernel and wants to leave it SMs.
int sm_count() { return persistent_ctas("CAIFQ_DECODE_CTAS"); }

// Streams (per device) on which one of this library's calls has just written codes or scales.
std::mutex g_written_mutex;
std::vector<std::pair<int, cudaStream_t>> g_written;

thread_local bool t_stall_next = false;

}  // namespace

void note_codes_written(cudaStream_t s)
{
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(g_written_mutex);
  for (const auto &e : g_written)
  {
    if (e.first == dev && e.second == s)
    {
      return;
    }
  }
  g_written.emplace_back(dev, s);
}

bool take_codes_written(cudaStream_t s)
{
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(g_written_mutex);
  for (size_t i = 0; i < g_written.size(); ++i)
  {
    if (g_written[i].first == dev && g_written[i].second == s)
    {
      g_written.erase(g_written.begin() + static_cast<std::ptrdiff_t>(i));
      return true;
    }
  }
  return false;
}

void decode_stall_next_launch() { t_stall_next = true; }


namespace
{

template <int BITS, int MT, int NCH>
int launch_decode_inst(const DecodeParams &p, uint32_t smem, cudaStream_t s)
{
  auto kernel = linear_decode_kernel<BITS, MT, NCH>;
  static std::atomic<bool> configured[kMaxDevices];
  int dev = 0;
  CAIFQ_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices)
  {
    set_error("frozen linear (decode): device ordinal %d out of range", dev);
    return CAIFQ_ERR_UNSUPPORTED;
  }
  if (!configured[dev].load(std::memory_order_acquire))
  {
    CAIFQ_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(kSmemBudget)));
    configured[dev].store(true, std::memory_order_release);
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
  // codes written just ahead in this stream by one of the library's own calls: a plain launch
  // orders the early copies behind that kernel
  cfg.numAttrs = (pdl && !take_codes_written(s)) ? 1 : 0;
  CAIFQ_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int chunks_per_warp(const caifq_weight &w)
{
  const int chunk_k = (w.storage == CAIFQ_I4) ? 128 : 64;
  const int chunks = w.in_dim / chunk_k;
  return (chunks + kWarps - 1) / kWarps;
}

int tokp_for(int64_t m) { return m <= 2 ? 2 : (m <= 4 ? 4 : (m <= 8 ? 8 : 16)); }

struct Layout
{
  uint32_t stage_bytes;
  uint32_t partial_bytes;
  int stages;
  int park_items;
};

Layout layout_for(const caifq_weight &w, int64_t m)
{
  Layout l{};
  const bool i4 = (w.storage == CAIFQ_I4);
  const uint32_t row_bytes = i4 ? static_cast<uint32_t>(w.in_dim / 2) : static_cast<uint32_t>(w.in_dim);
  const uint32_t scale_bytes = i4 ? static_cast<uint32_t>(kItemRows * (w.in_dim / w.group_size) * 2) : 0u;
  l.stage_bytes = ((kItemRows * row_bytes + scale_bytes) + 127u) & ~127u;
  // parked partial sums: [item][warp][16 rows][tokp] for as many of a CTA's items as fit beside
  // the ring (all of them for the usual layer sizes)
  const int quanta = (w.out_dim + kRowQuantum - 1) / kRowQuantum;
  int grid = sm_count();
  if (grid > quanta)
  {
    grid = quanta;
  }
  const int max_quanta = (quanta + grid - 1) / grid;
  const int max_items = (max_quanta * kRowQuantum + kItemRows - 1) / kItemRows;
  const uint32_t per_item = static_cast<uint32_t>(kWarps * kItemRows * tokp_for(m) * sizeof(float));
  int stages = kRingDepth;
  // Three items in flight per SM are enough to cover the latency of HBM.  More of them make the
  // launch slower, not faster (measured on B200: 10.8 us per launch with three, 11.3 with four,
  // 12.8 with six at in=4096, out=14336): every SM then asks for its whole share at once and the
  // first item of each lands later.
  while (stages > 2 && static_cast<uint32_t>(stages) * l.stage_bytes + per_item > kSmemBudget)
  {
    --stages;
  }
  if (static_cast<uint32_t>(stages) * l.stage_bytes + per_item > kSmemBudget)
  {
    stages = 0;   // a row too long for two stages and one parked item
  }
  int park = max_items;
  if (stages > 0)
  {
    const int fit = static_cast<int>((kSmemBudget - static_cast<uint32_t>(stages) * l.stage_bytes) / per_item);
    if (park > fit)
    {
      park = fit;
    }
  }
  l.park_items = park;
  l.partial_bytes = static_cast<uint32_t>(park) * per_item;
  l.stages = stages;
  return l;
}

}  // namespace

// The launch's rows: the layer's own, or those of all the layers that share the input laid end to end.
static caifq_weight all_rows(const LinearArgs &args)
{
  caifq_weight w = args.w;
  for (int i = 0; i < args.num_more; ++i)
  {
    w.out_dim += args.more[i].out_dim;
  }
  return w;
}

bool decode_supported(const LinearArgs &args)
{
  if (args.num_more < 0 || args.num_more >= kMaxSegments || (args.num_more > 0 && args.more == nullptr))
  {
    return false;
  }
  for (int i = 0; i < args.num_more; ++i)
  {
    // layers of one launch have one storage, row length, scale rule; every one but the last ends on a
    // multiple of 8 rows, so that every copy of a straddling item stays a multiple of 16 bytes
    const caifq_weight &o = args.more[i];
    const caifq_weight &prev = (i == 0) ? args.w : args.more[i - 1];
    if (o.storage != args.w.storage || o.in_dim != args.w.in_dim || o.scheme != args.w.scheme ||
        o.group_size != args.w.group_size || (o.scales == nullptr) != (args.w.scales == nullptr) ||
        (prev.out_dim % kRowQuantum) != 0 || o.out_dim < 1 || (reinterpret_cast<uintptr_t>(o.codes) & 15u) != 0 ||
        (reinterpret_cast<uintptr_t>(o.scales) & 15u) != 0)
    {
      return false;
    }
  }
  const caifq_weight w = all_rows(args);
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
  {
    // the token fragments of a warp's chunks must fit 64 registers
    const int nch = chunks_per_warp(w);
    const int xr = (w.storage == CAIFQ_I4) ? 16 : 8;
    const int mt = (m > 8) ? 2 : 1;
    if (nch * xr * mt > 64 || nch > 8)
    {
      return false;
    }
  }
  // at least two ring stages must fit beside the parked partial sums
  if (layout_for(w, m).stages < 2)
  {
    return false;
  }
  // bulk copies and 16-byte loads need aligned operands; a misaligned call goes to another kernel
  if ((reinterpret_cast<uintptr_t>(w.codes) & 15u) != 0 || (reinterpret_cast<uintptr_t>(w.scales) & 15u) != 0 ||
      (reinterpret_cast<uintptr_t>(args.a) & 15u) != 0)
  {
    return false;
  }
  return true;
}

int launch_linear_decode(const LinearArgs &args, cudaStream_t s)
{
  const caifq_weight w = all_rows(args);
  const int64_t m = args.m;
  const int y_dtype = args.c_dtype;
  DecodeParams p{};
  p.num_seg = 1 + args.num_more;
  p.seg_row0[0] = 0;
  for (int i = 0; i < p.num_seg; ++i)
  {
    const caifq_weight &seg = (i == 0) ? args.w : args.more[i - 1];
    p.codes[i] = static_cast<const uint8_t *>(seg.codes);
    p.scales[i] = seg.scales;
    p.seg_row0[i + 1] = p.seg_row0[i] + seg.out_dim;
  }
  for (int i = p.num_seg; i < kMaxSegments; ++i)
  {
    p.codes[i] = nullptr;
    p.scales[i] = nullptr;
    p.seg_row0[i + 1] = p.seg_row0[p.num_seg];
  }
  p.x = static_cast<const __nv_bfloat16 *>(args.a);
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
    p.y[0] = args.c;
    p.num_y = 1;
    p.y_ld = w.out_dim;
    p.y_col0 = 0;
  }
  p.y_dtype = y_dtype;
  // four rows of one token as one 16-byte store: fp32 results whose rows of four start aligned
  p.vec4 = (y_dtype == CAIFQ_F32 && (p.y_ld % 4) == 0 && (p.y_col0 % 4) == 0) ? 1 : 0;
  for (int r = 0; r < p.num_y; ++r)
  {
    if ((reinterpret_cast<uintptr_t>(p.y[r]) & 15u) != 0)
    {
      p.vec4 = 0;
    }
  }
  p.m = static_cast<int>(m);
  p.tokp = tokp_for(m);
  p.in_dim = w.in_dim;
  p.out_dim = w.out_dim;
  p.num_quanta = (w.out_dim + kRowQuantum - 1) / kRowQuantum;
  const bool i4 = (w.storage == CAIFQ_I4);
  p.row_bytes = i4 ? static_cast<uint32_t>(w.in_dim / 2) : static_cast<uint32_t>(w.in_dim);
  // rows lie unpadded, as in memory, so one bulk copy fills a stage; the 2-way
  // bank conflict on the four 16-byte reads per item is noise
  p.row_stride = p.row_bytes;
  if (i4)
  {
    p.groups_per_row = w.in_dim / w.group_size;
    p.chunks_per_group = w.group_size / 128;
  }
  else
  {
    p.groups_per_row = 0;
    p.chunks_per_group = 1;
  }
  const Layout lay = layout_for(w, m);
  int stages = lay.stages;
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
  p.stage_bytes = lay.stage_bytes;
  p.stages = stages;
  p.park_items = lay.park_items;
  p.partial_offset = static_cast<uint32_t>(stages) * p.stage_bytes;
  const uint32_t smem_bytes = p.partial_offset + lay.partial_bytes;
  p.spin_limit = kSpinLimit;
  p.stall_bytes = 0;
  if (t_stall_next)
  {
    // self-test of the give-up path: the first item announces 16 bytes that never arrive
    t_stall_next = false;
    p.spin_limit = kSpinLimitTest;
    p.stall_bytes = 16;
  }

  const int nch = chunks_per_warp(w);
  const int mt = (m > 8) ? 2 : 1;
#define CAIFQ_DECODE_CASE(B, M, N)                          \
  if (nch <= N && mt == M)                                  \
  {                                                         \
    return launch_decode_inst<B, M, N>(p, smem_bytes, s);   \
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
