// Tensor-core frozen-linear GEMM for many tokens (prefill / training shapes):
//
//   forward : C[m, out] = A[m, in]  . W_deq[out, in]^T     (ForwardImpl,  src/caif_device_frozen_linear.cpp:381-524)
//   backward: C[m, in]  = A[m, out] . W_deq[out, in]       (BackwardImpl, src/caif_device_frozen_linear.cpp:526-660)
//
// Blackwell-native: tcgen05.mma (kind::f16, bf16 operands, fp32 accumulators in
// TMEM), operands staged in shared memory in the canonical 128-byte-swizzled
// layouts, activations fed by TMA.  The weight never exists as a float matrix
// in memory (the reference dequantizes [out,in] to fp32 and hands it to cuBLAS,
// :288-378): eight warps read the packed codes straight from global memory,
// expand them to bf16 in registers and write the B operand tile into shared
// memory, one k-block ahead of the MMA warp.
//
// One persistent CTA per SM, 14 warps:
//   warp 0      TMA producer for the activation tiles (and the weight tiles when
//               the weight is already bf16)
//   warp 1      TMEM allocation, MMA issue (one elected lane)
//   warps 2-5   epilogue: TMEM -> registers -> scale -> global
//   warps 6-13  dequantization of the weight tile
// Tile 256 (two 128-row MMAs that share one dequantized weight tile) x 128 x 64,
// four pipeline stages, two accumulator sets in TMEM (4 x 128 columns) so the
// epilogue of one tile overlaps the main loop of the next.
//
// Forward uses the weight tile K-major (k = in is contiguous in memory);
// backward uses the SAME codes MN-major (n = in is contiguous), so dX needs no
// transposed copy of the weight.
//
// Exactness: int8 codes are exact in bf16 and the per-tensor scale multiplies
// the fp32 accumulator in the epilogue, so with bf16 activations the products
// are exact and the result matches an fp32 GEMM up to summation order.  int4
// weights are scale*code rounded to bf16, the operand the reference's bf16
// compute cell builds (dequantize to fp32, then To(bf16)).
//
// Every wait is bounded; a wait that runs out sets a flag that the host can
// read and lets the kernel finish (with wrong numbers) instead of hanging.
#include <cuda.h>

#include <cstdlib>

#include <atomic>

#include "common.cuh"

namespace caifq
{

__device__ unsigned int g_umma_timeout_flag = 0;

namespace
{
thread_local bool t_umma_stall_next = false;
}

// self-test hook: the next single-layer tensor-core launch of this thread waits for bytes that never arrive
void umma_stall_next_launch() { t_umma_stall_next = true; }

// Reads and clears the flag (1 = some bounded wait ran out since the last call; -1 = query failed).
int take_umma_timeout_flag()
{
  unsigned int v = 0;
  const unsigned int zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_umma_timeout_flag, sizeof(v)) != cudaSuccess)
  {
    return -1;
  }
  if (v != 0 && cudaMemcpyToSymbol(g_umma_timeout_flag, &zero, sizeof(zero)) != cudaSuccess)
  {
    return -1;
  }
  return v ? 1 : 0;
}

namespace
{

constexpr int BM_SUB = 128;          // rows of one MMA
constexpr int MT = 2;                // MMAs (row sub-tiles) per weight tile
constexpr int BM = BM_SUB * MT;      // 256
// BN (columns of the output tile, N of one MMA) is a template parameter: 128 or 256
constexpr int BK = 64;               // one 128-byte swizzle span of bf16
constexpr int UMMA_K = 16;
constexpr int A_SUB_BYTES = BM_SUB * BK * 2;       // 16 KB

constexpr int MAX_STAGES = 6;
constexpr int TMEM_COLS = 512;
constexpr int NUM_WARPS = 14;
constexpr int NUM_THREADS = NUM_WARPS * 32;
constexpr int DEQ_WARP0 = 6;
constexpr int DEQ_THREADS = 8 * 32;
// Teams of dequant warps (see the dequantization role): two for a single CTA's tile; four for a CTA pair,
// whose k-blocks take half as long while a conversion's latency chain (wait, loads, ~150 instructions,
// stores, proxy fence, arrive) stays the same (two teams: 750-830 TFLOP/s on 4096 x 4096 int8, four: 980-1150).
__host__ __device__ constexpr int deq_teams(bool pair) { return pair ? 4 : 2; }
constexpr uint32_t kSpinLimit = 1u << 22;       // polls of one wait before it gives up (tens of ms)
constexpr uint32_t kSpinLimitTest = 1u << 12;   // the same for the self-test of the give-up path

// A weight tile (BM = 256 activation rows x BN output columns) is worked on by one CTA, as two 128-row MMAs that
// share the staged weights, or -- PAIR -- by the two CTAs of a cluster with one `cta_group::2` MMA of 256 rows:
// each CTA stages its own 128 activation rows and its own half of the weight rows, so an SM moves half the
// operand bytes through its shared memory per flop and the 256 accumulator columns leave room for a second
// accumulator set (the epilogue overlaps the next tile).
template <int BN, int PLANES = 1, bool PAIR = false>
struct TileCfg
{
  static constexpr int MTK = PAIR ? 1 : MT;                       // 128-row sub-tiles of a CTA
  static constexpr int BNC = PAIR ? BN / 2 : BN;                  // weight-tile rows a CTA stages
  static constexpr int A_BYTES = A_SUB_BYTES * MTK;               // 16 or 32 KB
  static constexpr int B_PLANE_BYTES = BNC * BK * 2;              // 16 or 32 KB
  static constexpr int B_STAGE_BYTES = B_PLANE_BYTES * PLANES;
  static constexpr int STAGE_BYTES = A_BYTES + B_STAGE_BYTES;
  static constexpr int STAGES = (192 * 1024) / STAGE_BYTES;       // 192 KB of operands in every case: 3, 4 or 6
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;  // + slack to align the base to 1024
  static constexpr int ACC_COLS = PAIR ? BN : MT * BN;            // accumulator columns of a CTA per tile
  static constexpr int ACC_BUFS = TMEM_COLS / ACC_COLS;           // 2 (epilogue overlaps the next tile) or 1
  static_assert(!PAIR || BN == 256, "tile pairs are 256 columns wide");
  static_assert(STAGES >= 3 && STAGES <= MAX_STAGES, "operand ring depth");
};

enum WMode
{
  W_I8 = 0,
  W_I4 = 1,
  W_BF16 = 2,
  // int4 for fp32 compute: scale * code (exact in fp32) goes to the tensor core as two bf16 terms,
  // hi = bf16(w) and lo = bf16(w - hi), in two operand planes; hi + lo equals w to 2^-17 relative
  W_I4S = 3
};

__host__ __device__ constexpr int planes_of(int wmode) { return wmode == W_I4S ? 2 : 1; }

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Bounded wait.  A wait that runs out raises the CTA's abort word and the device flag; from then on
// every wait of the CTA returns at once, so the roles run through the rest of their loops without
// spinning (on garbage: the results are wrong and the host sees the flag) and the kernel ends within
// about one limit, TMEM released.
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity)
{
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_word, uint32_t limit)
{
  // A barrier that is already complete costs one poll and nothing else: the abort word is looked at only
  // once a wait actually has to wait (reading it before every poll cost 12 % of the kernel's throughput).
  if (mbar_try(bar, parity))
  {
    return true;
  }
  if (*abort_word != 0u)
  {
    return false;
  }
  for (uint32_t spin = 0; spin < limit; ++spin)
  {
    if (mbar_try(bar, parity))
    {
      return true;
    }
    if ((spin & 1023u) == 1023u && *abort_word != 0u)
    {
      return false;
    }
  }
  *abort_word = 1u;
  atomicExch(&g_umma_timeout_flag, 1u);
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar)
{
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          dst),
      "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}

// ---- two-CTA (cluster) forms
__device__ __forceinline__ uint32_t cluster_ctarank()
{
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// the shared::cluster address of `addr` (a shared::cta address of this CTA) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank)
{
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar)
{
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

__device__ __forceinline__ uint32_t ld_shared_cluster(uint32_t cluster_addr)
{
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(cluster_addr) : "memory");
  return v;
}

__device__ __forceinline__ void cluster_sync_all()
{
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// A tile load of this CTA's own shared memory whose bytes are counted on a barrier of the pair's leader CTA
// (`cluster_bar`, a shared::cluster address).  No multicast: every CTA fetches its own tile.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int c0, int c1,
                                                 uint32_t cluster_bar)
{
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], "
      "[%4];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(cluster_bar)
      : "memory");
}

__device__ __forceinline__ void fence_proxy_async()
{
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_before()
{
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after()
{
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate)
{
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// one MMA of 256 rows over the CTA pair: each CTA's shared memory holds its 128 rows of A and its half of B
// at the same offsets, the accumulator rows land in each CTA's own tensor memory
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate)
{
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ bool elect_one()
{
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// arrive on an mbarrier once every MMA issued so far by this thread has finished
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// the same for the pair's MMAs; the arrival goes to the barrier at this offset in both CTAs
__device__ __forceinline__ void umma_commit_pair(uint32_t bar)
{
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"(static_cast<uint16_t>(3))
      : "memory");
}

// the same, arriving on a barrier of the issuing CTA only
__device__ __forceinline__ void umma_commit_pair_local(uint32_t bar)
{
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor (sm_100): start address, leading / stride
// byte offsets in 16-byte units, descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;  // version
  d |= 2ull << 61;  // SWIZZLE_128B
  return d;
}

// Instruction descriptor, kind::f16: fp32 accumulate, bf16 x bf16, A K-major,
// B K-major (forward) or MN-major (backward), N = 128, M = 128.
__host__ __device__ constexpr uint32_t make_idesc(bool b_mn_major, int BN, int M = BM_SUB)
{
  return (1u << 4)                          // D format f32
         | (1u << 7)                        // A format bf16
         | (1u << 10)                       // B format bf16
         | (0u << 15)                       // A major: K
         | ((b_mn_major ? 1u : 0u) << 16)   // B major
         | (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c)
{
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b)
{
  uint32_t d;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

// four int8 codes (one 32-bit word, memory order) -> two bf16x2 registers, exact
__device__ __forceinline__ void int8x4_to_bf16(uint32_t w, uint32_t &p01, uint32_t &p23)
{
  const uint32_t a = __byte_perm(w, 0u, 0x4140);  // [b0, 0, b1, 0]
  const uint32_t b = __byte_perm(w, 0u, 0x4342);  // [b2, 0, b3, 0]
  // low 7 bits dropped into the mantissa of 128.0; the sign bit selects 128.0 or 256.0 to subtract
  p01 = sub_bf16x2(lop3_and_or(a, 0x007F007Fu, 0x43004300u), lop3_and_or(a, 0x00800080u, 0x43004300u));
  p23 = sub_bf16x2(lop3_and_or(b, 0x007F007Fu, 0x43004300u), lop3_and_or(b, 0x00800080u, 0x43004300u));
}

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b)
{
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Eight int4 codes (one 32-bit word, memory order) times a scale -> four bf16x2 registers, for bf16
// compute.  The codes become exact bf16 integers with logic ops (the offset-binary nibble dropped into
// the mantissa of 128.0, then 136 subtracted: exact) and are multiplied by the group scale rounded to
// bf16, one rounding.  The reference's dequantize-then-cast forms scale * code in fp32 and rounds once;
// the two differ by the bf16 rounding of the fp16 scale (2^-9 relative), far inside the bf16 bound, and
// the conversion takes 17 instructions per eight weights instead of 31: the int4 launches are bound by
// this conversion, not by the tensor core.
__device__ __forceinline__ void int4x8_to_bf16(uint32_t w, uint32_t scale2, uint32_t (&out)[4])
{
  const uint32_t ev = (w & 0x0F0F0F0Fu) ^ 0x08080808u;         // u0 u2 u4 u6   (u = q + 8)
  const uint32_t od = ((w >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;  // u1 u3 u5 u7
  const uint32_t t0 = __byte_perm(ev, od, 0x5140);             // u0 u1 u2 u3
  const uint32_t t1 = __byte_perm(ev, od, 0x7362);             // u4 u5 u6 u7
  constexpr uint32_t kExp = 0x43434343u;                       // high byte of bf16 128.0 .. 143.0
  constexpr uint32_t k136 = 0x43084308u;
  out[0] = mul_bf16x2(sub_bf16x2(__byte_perm(t0, kExp, 0x4140), k136), scale2);
  out[1] = mul_bf16x2(sub_bf16x2(__byte_perm(t0, kExp, 0x4342), k136), scale2);
  out[2] = mul_bf16x2(sub_bf16x2(__byte_perm(t1, kExp, 0x4140), k136), scale2);
  out[3] = mul_bf16x2(sub_bf16x2(__byte_perm(t1, kExp, 0x4342), k136), scale2);
}

// the same eight codes as two bf16 terms of scale * code: hi = bf16(w), lo = bf16(w - hi)
__device__ __forceinline__ void int4x8_to_bf16_split(uint32_t w, float scale, uint32_t (&hi)[4], uint32_t (&lo)[4])
{
  const uint32_t ev = (w & 0x0F0F0F0Fu) ^ 0x08080808u;
  const uint32_t od = ((w >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;
  const float base = 8388616.0f;   // 2^23 + 8
#pragma unroll
  for (int j = 0; j < 4; ++j)
  {
    const float a = __fmul_rn(__uint_as_float(__byte_perm(ev, 0x4B000000u, 0x7440 + j)) - base, scale);
    const float b = __fmul_rn(__uint_as_float(__byte_perm(od, 0x4B000000u, 0x7440 + j)) - base, scale);
    const uint32_t h = pack_bf16x2(a, b);
    hi[j] = h;
    lo[j] = pack_bf16x2(a - __uint_as_float(h << 16), b - __uint_as_float(h & 0xFFFF0000u));
  }
}

struct UmmaParams
{
  const uint8_t *codes;
  const void *scales;
  void *c;
  int c_dtype;
  int accumulate;    // epilogue: c = round_c(round_c(acc) + c_old)
  int64_t m;
  int n_total;       // columns of C
  int k_total;       // reduction length
  int in_dim;        // row length of the code matrix
  int group_size;    // int4
  int groups_per_row;  // int4: in_dim / group_size
  int num_m_tiles;
  int num_n_tiles;
  const uint8_t *lora_rhs;  // null = no LoRA k-block
  const float *c_scale;     // bf16 weights only: factor of the fp32 accumulator in the epilogue (null = 1)
  int expert_rows;          // grouped bf16 weights: rows of one expert's matrix in the stacked [E * rows, in] matrix
  // dX launch whose result is the gradient of the experts' hidden activation (down^T): instead of storing it, the
  // epilogue applies the SwiGLU backward to it and stores the gradients of the gate and up projections' outputs
  // (c: g_gate, sb_g_up: g_up), reading the forward's gate(x) and up(x) (sb_gate, sb_up).  bf16 only.
  const void *sb_gate;
  const void *sb_up;
  void *sb_g_up;
  int dual_k;               // bf16 weights: the reduction runs over two operand pairs, C = A.W + A2.W2 (A2 through
                            // map_h, W2 through map_l), num_kb k-blocks each
  // Fused gate/up/SwiGLU forward of a frozen expert (forward, 128-wide tiles, 16-bit outputs): a tile's
  // columns 0..63 are features [64 j, 64 j + 64) of the gate projection, columns 64..127 the same
  // features of the up projection.  c receives gate(x), c_up up(x), c_hidden silu(gate(x)) * up(x),
  // each rounded to the storage dtype the way the separate kernels round them.
  uint32_t spin_limit;   // polls of one wait before it gives up
  uint32_t stall_bytes;  // self-test only: bytes the first activation tile announces but never receives
  int swiglu;
  const uint8_t *codes_up;
  const void *scales_up;
  void *c_up;
  void *c_hidden;
};

// Grouped mode: one launch covers the same product for a run of experts whose activation rows lie
// back to back in one packed buffer (rows offsets[e] .. offsets[e+1] belong to expert e).  The table
// travels as a kernel parameter, so nothing is read back from or copied to the device to schedule it.
constexpr int MAX_GROUPS = 80;   // the table must fit the 4 KB of kernel parameters

struct GroupTable
{
  int32_t offsets[MAX_GROUPS + 1];      // first packed row of every expert
  int32_t mtile_start[MAX_GROUPS + 1];  // running count of 256-row tiles
  const uint8_t *codes[MAX_GROUPS];
  const void *scales[MAX_GROUPS];
  const uint8_t *codes_up[MAX_GROUPS];   // fused gate/up mode only
  const void *scales_up[MAX_GROUPS];
  int32_t num_groups;
};

struct NoGroupTable
{
  int32_t unused;
};

template <bool GROUPED>
struct GroupSel
{
  typedef NoGroupTable type;
};
template <>
struct GroupSel<true>
{
  typedef GroupTable type;
};

// What a tile of the schedule works on.
struct TileWork
{
  int expert;        // grouped mode: index of the expert inside this launch's table
  int n_tile;
  int64_t row0;      // first activation / output row of the tile
  int64_t row_end;   // rows at or beyond this one belong to somebody else
  const uint8_t *codes;
  const void *scales;
  const uint8_t *codes_up;
  const void *scales_up;
};

template <bool GROUPED>
__device__ __forceinline__ TileWork locate_tile(int tile, const UmmaParams &p, const typename GroupSel<GROUPED>::type &gt);

template <>
__device__ __forceinline__ TileWork locate_tile<false>(int tile, const UmmaParams &p, const NoGroupTable &)
{
  // column tiles fastest: the CTAs running at one time share a few row tiles of the activations
  // (read from memory once) and sweep the weight, which stays in L2
  TileWork t;
  t.expert = 0;
  t.n_tile = tile % p.num_n_tiles;
  t.row0 = static_cast<int64_t>(tile / p.num_n_tiles) * BM;
  t.row_end = p.m;
  t.codes = p.codes;
  t.scales = p.scales;
  t.codes_up = p.codes_up;
  t.scales_up = p.scales_up;
  return t;
}

template <>
__device__ __forceinline__ TileWork locate_tile<true>(int tile, const UmmaParams &p, const GroupTable &gt)
{
  const int mt = tile / p.num_n_tiles;   // row tile among all experts' row tiles; column tiles fastest
  int lo = 0;
  int hi = gt.num_groups;                // mtile_start[lo] <= mt < mtile_start[hi]
  while (hi - lo > 1)
  {
    const int mid = (lo + hi) >> 1;
    if (gt.mtile_start[mid] <= mt)
    {
      lo = mid;
    }
    else
    {
      hi = mid;
    }
  }
  TileWork t;
  t.expert = lo;
  t.n_tile = tile % p.num_n_tiles;
  t.row0 = static_cast<int64_t>(gt.offsets[lo]) + static_cast<int64_t>(mt - gt.mtile_start[lo]) * BM;
  t.row_end = gt.offsets[lo + 1];
  t.codes = gt.codes[lo];
  t.scales = gt.scales[lo];
  t.codes_up = gt.codes_up[lo];
  t.scales_up = gt.scales_up[lo];
  return t;
}

template <int WMODE, bool BWD, int BN, bool GROUPED, bool PAIR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
linear_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ CUtensorMap map_h, const __grid_constant__ CUtensorMap map_l,
                   const UmmaParams p,
                   const __grid_constant__ typename GroupSel<GROUPED>::type gt)
{
  constexpr int PLANES = planes_of(WMODE);
  constexpr bool IS_I4 = (WMODE == W_I4 || WMODE == W_I4S);
  typedef TileCfg<BN, PLANES, PAIR> Cfg;
  constexpr int MTK = Cfg::MTK;
  constexpr int BNC = Cfg::BNC;
  constexpr int A_STAGE = Cfg::A_BYTES;
  constexpr int B_PLANE_BYTES = Cfg::B_PLANE_BYTES;
  constexpr int B_STAGE_BYTES = Cfg::B_STAGE_BYTES;
  constexpr int STAGE_BYTES = Cfg::STAGE_BYTES;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int ACC_COLS = Cfg::ACC_COLS;
  constexpr int ACC_BUFS = Cfg::ACC_BUFS;
  constexpr uint32_t CTAS = PAIR ? 2u : 1u;   // CTAs that work on one tile
  // A bf16 weight needs no dequant warps: four of them join the epilogue, so every quarter of the accumulator's
  // lanes is drained by two warps that take alternate 32-column chunks.
  constexpr int EPI_GROUPS = (WMODE == W_BF16) ? 2 : 1;
    constexpr int DEQ_TEAMS = deq_teams(PAIR);
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bars[MAX_STAGES * 3 + 4];
  __shared__ uint64_t drain_bar;   // give-up path only: the MMAs issued so far have completed
  __shared__ uint32_t tmem_base_slot;
  __shared__ uint32_t cta_abort;   // a wait of this CTA has run out

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  auto a_addr = [&](int s, int mt) { return smem_base + static_cast<uint32_t>(s) * STAGE_BYTES + mt * A_SUB_BYTES; };
  auto b_addr = [&](int s) { return smem_base + static_cast<uint32_t>(s) * STAGE_BYTES + A_STAGE; };
  const uint32_t bar0 = smem_u32(bars);
  auto a_full = [&](int s) { return bar0 + static_cast<uint32_t>(s) * 8u; };
  auto b_full = [&](int s) { return bar0 + static_cast<uint32_t>(STAGES + s) * 8u; };
  auto empty = [&](int s) { return bar0 + static_cast<uint32_t>(2 * STAGES + s) * 8u; };
  auto acc_full = [&](int a) { return bar0 + static_cast<uint32_t>(3 * STAGES + a) * 8u; };
  auto acc_empty = [&](int a) { return bar0 + static_cast<uint32_t>(3 * STAGES + 2 + a) * 8u; };

  // Pair mode: rank 0 of the cluster (the leader) issues the MMAs; the barriers that gate them (operands
  // landed, accumulator drained) are the leader's, and the other CTA's copies and warps arrive on them
  // through the cluster's shared address space.  The barriers that the MMAs' completion signals (stage free,
  // accumulator ready) exist in both CTAs and get a multicast commit.
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const int worker = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int workers = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  auto lead = [&](uint32_t bar) { return PAIR ? map_to_cta(bar, 0u) : bar; };
  auto arrive_lead = [&](uint32_t bar)
  {
    if (PAIR)
    {
      mbar_arrive_cluster(map_to_cta(bar, 0u));
    }
    else
    {
      mbar_arrive(bar);
    }
  };
  volatile uint32_t *abort_word = &cta_abort;
  auto wait = [&](uint32_t bar, uint32_t parity) { return mbar_wait(bar, parity, abort_word, p.spin_limit); };
  if (threadIdx.x == 0)
  {
    cta_abort = 0u;
    mbar_init(smem_u32(&drain_bar), 1);
    for (int s = 0; s < STAGES; ++s)
    {
      mbar_init(a_full(s), 1);
      mbar_init(b_full(s), (WMODE == W_BF16) ? 1 : (8 / DEQ_TEAMS) * CTAS);
      mbar_init(empty(s), 1);
    }
    for (int a = 0; a < ACC_BUFS; ++a)
    {
      mbar_init(acc_full(a), 1);
      mbar_init(acc_empty(a), 4 * EPI_GROUPS * CTAS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1)
  {
    if (PAIR)
    {
      // both CTAs of the pair run this, from the same warp number
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                   "r"(TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    else
    {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                   "r"(TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR)
  {
    cluster_sync_all();   // the other CTA's barriers are initialised before anything arrives on them
  }
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  const int num_tiles = p.num_m_tiles * p.num_n_tiles;
  const int num_kb = p.k_total / BK;
  // with a LoRA product the loop runs one more k-block whose operands are the padded factors
  const int num_kb_all = (p.dual_k ? 2 * num_kb : num_kb) + ((p.lora_rhs != nullptr) ? 1 : 0);

  if (warp == 0)
  {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0)
    {
      int s = 0;
      uint32_t par = 0;
      for (int tile = worker; tile < num_tiles; tile += workers)
      {
        const TileWork tw = locate_tile<GROUPED>(tile, p, gt);
        const int n_tile = tw.n_tile;
        const int row_tile = static_cast<int>(tw.row0) + static_cast<int>(rank) * BM_SUB;   // pair: this CTA's half
        for (int kb = 0; kb < num_kb_all; ++kb)
        {
          if (!wait(empty(s), par ^ 1u))
          {
            tile = num_tiles;   // nothing new is started once a wait has run out
            break;
          }
          // (pair: the leader announces both CTAs' bytes; the other CTA's copies may complete first, the
          // phase cannot end before the leader's arrival)
          auto load = [&](uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar)
          {
            if (PAIR)
            {
              tma_load_2d_pair(dst, map, c0, c1, lead(bar));
            }
            else
            {
              tma_load_2d(dst, map, c0, c1, bar);
            }
          };
          if (rank == 0)
          {
            mbar_expect_tx(a_full(s), A_STAGE * CTAS + ((tile == worker && kb == 0) ? p.stall_bytes : 0u));
          }
#pragma unroll
          for (int mt = 0; mt < MTK; ++mt)
          {
            if (kb < num_kb)
            {
              load(a_addr(s, mt), &map_a, kb * BK, row_tile + mt * BM_SUB, a_full(s));
            }
            else
            {
              // the LoRA k-block's activation-side operand, or the second operand pair's k-block
              load(a_addr(s, mt), &map_h, p.dual_k ? (kb - num_kb) * BK : 0, row_tile + mt * BM_SUB, a_full(s));
            }
          }
          if (WMODE == W_BF16)
          {
            const int nc0 = n_tile * BN + static_cast<int>(rank) * BNC;   // this CTA's weight rows
            if (rank == 0)
            {
              mbar_expect_tx(b_full(s), B_STAGE_BYTES * CTAS);
            }
            // the LoRA k-block (number num_kb) takes its weight-side operand, the padded factor, from map_l
            const CUtensorMap *bmap = (kb < num_kb) ? &map_b : &map_l;
            const int kc = (kb < num_kb) ? kb * BK : (p.dual_k ? (kb - num_kb) * BK : 0);
            // grouped: the experts' matrices lie stacked in one [E * rows, in] matrix
            const int erow = GROUPED ? tw.expert * p.expert_rows : 0;
            if (!BWD && p.swiglu)
            {
              // HALF features of the gate projection (map_b) and the same features of the up projection (map_l)
              constexpr int HALF = BN / 2;
              const int f0 = erow + n_tile * HALF;
              if (PAIR)
              {
                load(b_addr(s), (rank == 0) ? &map_b : &map_l, kc, f0, b_full(s));
              }
              else
              {
                load(b_addr(s), &map_b, kc, f0, b_full(s));
                load(b_addr(s) + static_cast<uint32_t>(HALF) * 128u, &map_l, kc, f0, b_full(s));
              }
            }
            else if (BWD)
            {
              // [k rows][n cols]: boxes of 64 n x 64 k land as the MN-major blocks
#pragma unroll
              for (int nb = 0; nb < BNC / 64; ++nb)
              {
                load(b_addr(s) + static_cast<uint32_t>(nb) * 8192u, bmap, nc0 + nb * 64, erow + kc, b_full(s));
              }
            }
            else
            {
              load(b_addr(s), bmap, kc, erow + nc0, b_full(s));
            }
          }
          if (++s == STAGES)
          {
            s = 0;
            par ^= 1u;
          }
        }
      }
    }
  }
  else if (warp == 1)
  {
    // -------------------------------------------------------------- MMA issuer
    // The whole warp runs the loop, so addresses and descriptors are warp-uniform values;
    // one elected lane issues the MMAs and the commits.  (Pair: the leader CTA's warp only.)
    if (rank == 0)
    {
      constexpr uint32_t idesc = make_idesc(BWD, BN, PAIR ? 2 * BM_SUB : BM_SUB);
      auto mma = [&](uint32_t d, uint64_t a, uint64_t b, uint32_t accumulate)
      {
        if (PAIR)
        {
          umma_bf16_pair(d, a, b, idesc, accumulate);
        }
        else
        {
          umma_bf16(d, a, b, idesc, accumulate);
        }
      };
      auto commit = [&](uint32_t bar)
      {
        if (PAIR)
        {
          umma_commit_pair(bar);
        }
        else
        {
          umma_commit(bar);
        }
      };
      int s = 0;
      uint32_t par = 0;
      int acc = 0;
      uint32_t acc_par = 0;
      for (int tile = worker; tile < num_tiles; tile += workers)
      {
        wait(acc_empty(acc), acc_par ^ 1u);
        tc_fence_after();
        for (int kb = 0; kb < num_kb_all; ++kb)
        {
          wait(a_full(s), par);
          wait(b_full(s), par);
          tc_fence_after();
          const uint64_t adesc0 = make_desc(a_addr(s, 0), 16, 1024);
          const uint64_t bdesc0 = BWD ? make_desc(b_addr(s), 8192, 1024) : make_desc(b_addr(s), 16, 1024);
          const uint32_t d0 = tmem_base + static_cast<uint32_t>(acc * ACC_COLS);
          if (elect_one())
          {
#pragma unroll
            for (int mt = 0; mt < MTK; ++mt)
            {
#pragma unroll
              for (int k16 = 0; k16 < BK / UMMA_K; ++k16)
              {
                // descriptor address fields count 16-byte units
                const uint64_t adesc = adesc0 + static_cast<uint64_t>((mt * A_SUB_BYTES + k16 * (UMMA_K * 2)) >> 4);
                const uint64_t bdesc = bdesc0 + static_cast<uint64_t>((BWD ? k16 * 2048 : k16 * (UMMA_K * 2)) >> 4);
                mma(d0 + static_cast<uint32_t>(mt * BN), adesc, bdesc, (kb > 0 || k16 > 0) ? 1u : 0u);
                if (PLANES == 2 && kb < num_kb)
                {
                  // the low-order term of the weights (the LoRA k-block has one plane only)
                  mma(d0 + static_cast<uint32_t>(mt * BN), adesc, bdesc + static_cast<uint64_t>(B_PLANE_BYTES >> 4), 1u);
                }
              }
            }
            commit(empty(s));
          }
          __syncwarp();
          if (++s == STAGES)
          {
            s = 0;
            par ^= 1u;
          }
        }
        if (elect_one())
        {
          commit(acc_full(acc));
        }
        __syncwarp();
        if (++acc == ACC_BUFS)
        {
          acc = 0;
          acc_par ^= 1u;
        }
      }
    }
  }
  else if (warp < DEQ_WARP0 + 4 * (EPI_GROUPS - 1))
  {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 are the ones this warp may read
    const int epi_group = (warp - 2) >> 2;   // 0, or 1 for the warps that joined from the dequant role
    int acc = 0;
    uint32_t acc_par = 0;
    for (int tile = worker; tile < num_tiles; tile += workers)
    {
      const TileWork tw = locate_tile<GROUPED>(tile, p, gt);
      const int n_tile = tw.n_tile;
      float out_scale = 1.0f;
      if ((WMODE == W_I8 || (WMODE == W_BF16 && GROUPED)) && tw.scales != nullptr)
      {
        // (grouped bf16 weights: expanded int8 codes, whose per-tensor scale the table still carries)
        out_scale = __ldg(static_cast<const float *>(tw.scales));
      }
      if (WMODE == W_BF16 && p.c_scale != nullptr)
      {
        out_scale = __ldg(p.c_scale);
      }
      wait(acc_full(acc), acc_par);
      tc_fence_after();
      if (!BWD && (BN == 128 || PAIR) && p.swiglu)
      {
        constexpr int HALF = BN / 2;   // features of each projection in a tile
        float up_scale = 1.0f;
        if ((WMODE == W_I8 || (WMODE == W_BF16 && GROUPED)) && tw.scales_up != nullptr)
        {
          up_scale = __ldg(static_cast<const float *>(tw.scales_up));
        }
        const int hid = p.n_total / 2;   // features per projection
#pragma unroll
        for (int mt = 0; mt < MTK; ++mt)
        {
          const int64_t row = tw.row0 + static_cast<int64_t>(rank) * BM_SUB + mt * BM_SUB + quarter * 32 + lane;
#pragma unroll
          for (int cb = 0; cb < HALF / 32; ++cb)
          {
            if (EPI_GROUPS > 1 && (cb % EPI_GROUPS) != epi_group)
            {
              continue;
            }
            uint32_t rg[32];
            uint32_t ru[32];
            const uint32_t tbase = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(acc * ACC_COLS + mt * BN);
            tmem_ld32(tbase + cb * 32, rg);
            tmem_ld32(tbase + HALF + cb * 32, ru);
            tmem_ld_wait();
            if (row < tw.row_end)
            {
              const int64_t off = row * hid + static_cast<int64_t>(n_tile) * HALF + cb * 32;
              uint4 *dg = reinterpret_cast<uint4 *>(static_cast<uint16_t *>(p.c) + off);
              uint4 *du = reinterpret_cast<uint4 *>(static_cast<uint16_t *>(p.c_up) + off);
              uint4 *dh = reinterpret_cast<uint4 *>(static_cast<uint16_t *>(p.c_hidden) + off);
#pragma unroll
              for (int q = 0; q < 4; ++q)
              {
                uint32_t pg[4], pu[4], ph[4];
#pragma unroll
                for (int e = 0; e < 4; ++e)
                {
                  float g2[2], u2[2], h2[2];
#pragma unroll
                  for (int z = 0; z < 2; ++z)
                  {
                    // the separate kernels' roundings: projection outputs to the storage dtype,
                    // silu(gate) to the storage dtype, then the product
                    g2[z] = round_through<CAIFQ_BF16>(__uint_as_float(rg[8 * q + 2 * e + z]) * out_scale);
                    u2[z] = round_through<CAIFQ_BF16>(__uint_as_float(ru[8 * q + 2 * e + z]) * up_scale);
                    const float act = round_through<CAIFQ_BF16>(g2[z] / (1.0f + expf(-g2[z])));
                    h2[z] = act * u2[z];
                  }
                  pg[e] = pack_bf16x2(g2[0], g2[1]);
                  pu[e] = pack_bf16x2(u2[0], u2[1]);
                  ph[e] = pack_bf16x2(h2[0], h2[1]);
                }
                dg[q] = make_uint4(pg[0], pg[1], pg[2], pg[3]);
                du[q] = make_uint4(pu[0], pu[1], pu[2], pu[3]);
                dh[q] = make_uint4(ph[0], ph[1], ph[2], ph[3]);
              }
            }
          }
        }
      }
      else
#pragma unroll
      for (int mt = 0; mt < MTK; ++mt)
      {
        const int64_t row = tw.row0 + static_cast<int64_t>(rank) * BM_SUB + mt * BM_SUB + quarter * 32 + lane;
#pragma unroll
        for (int cb = 0; cb < BN / 32; ++cb)
        {
          if (EPI_GROUPS > 1 && (cb % EPI_GROUPS) != epi_group)
          {
            continue;
          }
          uint32_t r[32];
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                 static_cast<uint32_t>(acc * ACC_COLS + mt * BN + cb * 32);
          tmem_ld32(taddr, r);
          tmem_ld_wait();
          // (the last column tile may reach past the output's width when the width is not a multiple of the
          // tile's: those columns, computed on zero or foreign weight rows, are not stored)
          if (row < tw.row_end && n_tile * BN + cb * 32 < p.n_total)
          {
            const int64_t off = row * p.n_total + static_cast<int64_t>(n_tile) * BN + cb * 32;
            if (BWD && p.sb_gate != nullptr)
            {
              // g_hidden = round(acc); g_up = round(g_hidden * round(silu(gate))); g_gate = round(round(g_hidden *
              // up) * silu'(gate)): the separate kernel's rounding points (see swiglu_bwd_kernel)
              const uint4 *gt4 = reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(p.sb_gate) + off);
              const uint4 *up4 = reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(p.sb_up) + off);
              uint4 *dg = reinterpret_cast<uint4 *>(static_cast<uint16_t *>(p.c) + off);
              uint4 *du = reinterpret_cast<uint4 *>(static_cast<uint16_t *>(p.sb_g_up) + off);
#pragma unroll
              for (int q = 0; q < 4; ++q)
              {
                const uint4 gq = __ldg(gt4 + q);
                const uint4 uq = __ldg(up4 + q);
                const uint32_t gw[4] = {gq.x, gq.y, gq.z, gq.w};
                const uint32_t uw[4] = {uq.x, uq.y, uq.z, uq.w};
                uint32_t pg[4], pu[4];
#pragma unroll
                for (int e = 0; e < 4; ++e)
                {
                  float og[2], ou[2];
#pragma unroll
                  for (int z = 0; z < 2; ++z)
                  {
                    const float x = z ? __uint_as_float(gw[e] & 0xFFFF0000u) : __uint_as_float(gw[e] << 16);
                    const float uv = z ? __uint_as_float(uw[e] & 0xFFFF0000u) : __uint_as_float(uw[e] << 16);
                    const float gh = round_through<CAIFQ_BF16>(__uint_as_float(r[8 * q + 2 * e + z]) * out_scale);
                    // one fast exponential and one fast reciprocal per element: 256 x 128 elements per tile must
                    // fit beside the next tile's MMAs (the exact expf and two IEEE divisions did not: 2x slower);
                    // fp32 relative error ~1e-6 before the bf16 roundings
                    const float sg = __fdividef(1.0f, 1.0f + __expf(-x));
                    const float act = round_through<CAIFQ_BF16>(x * sg);
                    ou[z] = gh * act;
                    const float gv = round_through<CAIFQ_BF16>(gh * uv);
                    og[z] = gv * sg * fmaf(x, 1.0f - sg, 1.0f);
                  }
                  pg[e] = pack_bf16x2(og[0], og[1]);
                  pu[e] = pack_bf16x2(ou[0], ou[1]);
                }
                dg[q] = make_uint4(pg[0], pg[1], pg[2], pg[3]);
                du[q] = make_uint4(pu[0], pu[1], pu[2], pu[3]);
              }
            }
            else if (p.c_dtype == CAIFQ_F32)
            {
              float4 *dst = reinterpret_cast<float4 *>(static_cast<float *>(p.c) + off);
#pragma unroll
              for (int q = 0; q < 8; ++q)
              {
                float4 v;
                v.x = __uint_as_float(r[4 * q + 0]) * out_scale;
                v.y = __uint_as_float(r[4 * q + 1]) * out_scale;
                v.z = __uint_as_float(r[4 * q + 2]) * out_scale;
                v.w = __uint_as_float(r[4 * q + 3]) * out_scale;
                if (p.accumulate)
                {
                  const float4 o = dst[q];
                  v.x += o.x;
                  v.y += o.y;
                  v.z += o.z;
                  v.w += o.w;
                }
                dst[q] = v;
              }
            }
            else
            {
              // 16-bit outputs: 32 values = 64 bytes = four 16-byte stores
              uint4 *dst = reinterpret_cast<uint4 *>(static_cast<uint16_t *>(p.c) + off);
#pragma unroll
              for (int q = 0; q < 4; ++q)
              {
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e)
                {
                  v[e] = __uint_as_float(r[8 * q + e]) * out_scale;
                }
                uint32_t packed[4];
                if (p.accumulate)
                {
                  const uint4 o = dst[q];
                  const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e)
                  {
                    float lo;
                    float hi;
                    if (p.c_dtype == CAIFQ_BF16)
                    {
                      lo = __uint_as_float(ow[e] << 16);
                      hi = __uint_as_float(ow[e] & 0xFFFF0000u);
                      v[2 * e] = round_through<CAIFQ_BF16>(v[2 * e]) + lo;
                      v[2 * e + 1] = round_through<CAIFQ_BF16>(v[2 * e + 1]) + hi;
                    }
                    else
                    {
                      const __half2 h = *reinterpret_cast<const __half2 *>(&ow[e]);
                      v[2 * e] = round_through<CAIFQ_F16>(v[2 * e]) + __low2float(h);
                      v[2 * e + 1] = round_through<CAIFQ_F16>(v[2 * e + 1]) + __high2float(h);
                    }
                  }
                }
#pragma unroll
                for (int e = 0; e < 4; ++e)
                {
                  if (p.c_dtype == CAIFQ_BF16)
                  {
                    packed[e] = pack_bf16x2(v[2 * e], v[2 * e + 1]);
                  }
                  else
                  {
                    const __half2 h = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
                    packed[e] = *reinterpret_cast<const uint32_t *>(&h);
                  }
                }
                dst[q] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0)
      {
        arrive_lead(acc_empty(acc));
      }
      if (++acc == ACC_BUFS)
      {
        acc = 0;
        acc_par ^= 1u;
      }
    }
  }
  else if (WMODE != W_BF16)
  {
    // ------------------------------------------------------ weight dequantization
    // The eight warps work as DEQ_TEAMS teams; team t converts the k-blocks whose number is t modulo
    // DEQ_TEAMS, so with two teams a k-block's conversion (loads, ~150 instructions per thread, stores,
    // proxy fence, barrier arrive) has two k-blocks of MMA time to finish in.
    constexpr int TEAM_THREADS = DEQ_THREADS / DEQ_TEAMS;
    const int team = (threadIdx.x - DEQ_WARP0 * 32) / TEAM_THREADS;
    const int d = (threadIdx.x - DEQ_WARP0 * 32) % TEAM_THREADS;
    // 16-byte chunks of codes per k-block and thread, and where they go:
    //   forward  (K-major B): tile rows are n, a chunk is 16 B of one row's k range
    //   backward (MN-major B): tile rows are k, a chunk is 16 B of one k-row's n range
    constexpr int ELEMS = (WMODE == W_I8) ? 16 : 32;                 // codes per chunk
    constexpr int CHUNKS = (BNC * BK) / ELEMS;                       // per k-block (of this CTA's weight rows)
    constexpr int PER_THREAD = CHUNKS / TEAM_THREADS;
    constexpr int CHUNKS_PER_ROW = (BWD ? BNC : BK) / ELEMS;         // chunks along the contiguous direction
    static_assert(PER_THREAD >= 1, "tile too small for the dequant warps");

    uint32_t gkb0 = 0;   // k-blocks (of all tiles so far) before this tile: the ring position of its first one
    for (int tile = worker; tile < num_tiles; tile += workers, gkb0 += static_cast<uint32_t>(num_kb_all))
    {
      const TileWork tw = locate_tile<GROUPED>(tile, p, gt);
      const int n_tile = tw.n_tile;
      const int n0 = n_tile * BN + static_cast<int>(rank) * BNC;   // first of this CTA's weight rows / columns
      // chunk -> (row inside the tile, part along the contiguous direction)
      int c_row[PER_THREAD];
      int c_part[PER_THREAD];
#pragma unroll
      for (int i = 0; i < PER_THREAD; ++i)
      {
        const int c = d + i * TEAM_THREADS;
        if (BWD)
        {
          // A chunk expands to 64 (int4) or 32 (int8) bytes of one 128-byte operand row, whose 16-byte
          // pieces sit at (piece ^ row % 8).  Eight consecutive threads (one shared-memory store phase)
          // take RPQ neighbouring rows x PPQ neighbouring chunks: eight distinct bank groups, and the
          // PPQ chunks of a row are contiguous in global memory.
          constexpr int PPQ = 128 / (ELEMS * 2);
          constexpr int RPQ = 8 / PPQ;
          const int lo = c & 7;
          const int hi = c >> 3;
          c_row[i] = (hi % (BK / RPQ)) * RPQ + lo / PPQ;
          c_part[i] = (hi / (BK / RPQ)) * PPQ + lo % PPQ;
        }
        else
        {
          c_row[i] = c / CHUNKS_PER_ROW;
          c_part[i] = c % CHUNKS_PER_ROW;
        }
      }
      auto load = [&](int kb, uint4 (&raw)[PER_THREAD], float (&sc)[PER_THREAD])
      {
        const int k0 = kb * BK;
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i)
        {
          // element coordinates of the chunk's first code in the [out, in] matrix
          int64_t o = BWD ? (k0 + c_row[i]) : (n0 + c_row[i]);
          const uint8_t *codes = tw.codes;
          const void *scales = tw.scales;
          if (!BWD && p.swiglu)
          {
            // first half of the tile's rows: gate features HALF j + r; second half: the same up features
            constexpr int HALF = BN / 2;
            const int t = static_cast<int>(rank) * BNC + c_row[i];
            o = static_cast<int64_t>(n_tile) * HALF + (t % HALF);
            if (t >= HALF)
            {
              codes = tw.codes_up;
              scales = tw.scales_up;
            }
          }
          const int64_t ii = BWD ? (n0 + c_part[i] * ELEMS) : (k0 + c_part[i] * ELEMS);
          const int64_t flat = o * p.in_dim + ii;
          const uint8_t *src = codes + ((WMODE == W_I8) ? flat : (flat >> 1));
          raw[i] = __ldg(reinterpret_cast<const uint4 *>(src));
          if (IS_I4)
          {
            // in_dim is a multiple of the group size here, so the flat group index splits into a row
            // part and a 32-bit division inside the row (a 64-bit division costs as much as the conversion)
            const int64_t grp = o * p.groups_per_row + static_cast<int>(ii) / p.group_size;
            sc[i] = __half2float(static_cast<const __half *>(scales)[grp]);
          }
          else
          {
            sc[i] = 1.0f;
          }
        }
      };

      // this team's first k-block of the tile
      const int kb_first = static_cast<int>((static_cast<uint32_t>(team) + DEQ_TEAMS - (gkb0 % DEQ_TEAMS)) % DEQ_TEAMS);
      // With eight chunks per thread the next block's codes are not kept in flight beside the current
      // ones (registers); the other team's block covers the load instead.
      constexpr bool PREFETCH = PER_THREAD <= 4;
      uint4 raw[PER_THREAD];
      float sc[PER_THREAD];
      if (PREFETCH && kb_first < num_kb)
      {
        load(kb_first, raw, sc);
      }
      for (int kb = kb_first; kb < num_kb; kb += DEQ_TEAMS)
      {
        uint4 nraw[PER_THREAD];
        float nsc[PER_THREAD];
        if (!PREFETCH)
        {
          load(kb, raw, sc);
        }
        else if (kb + DEQ_TEAMS < num_kb)
        {
          load(kb + DEQ_TEAMS, nraw, nsc);  // in flight while this block is converted
        }
        const uint32_t gkb = gkb0 + static_cast<uint32_t>(kb);
        const int s = static_cast<int>(gkb % STAGES);
        const uint32_t par = (gkb / STAGES) & 1u;
        wait(empty(s), par ^ 1u);
        const uint32_t bbase = b_addr(s);
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i)
        {
          const uint32_t words[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
          // bf16 output: ELEMS values = ELEMS/8 chunks of 16 bytes
          uint32_t outw[ELEMS / 2];
          uint32_t outl[(WMODE == W_I4S) ? ELEMS / 2 : 1];   // low-order plane (split mode)
          if (WMODE == W_I8)
          {
#pragma unroll
            for (int w = 0; w < 4; ++w)
            {
              int8x4_to_bf16(words[w], outw[2 * w], outw[2 * w + 1]);
            }
          }
          else if (WMODE == W_I4S)
          {
#pragma unroll
            for (int w = 0; w < 4; ++w)
            {
              uint32_t h4[4];
              uint32_t l4[4];
              int4x8_to_bf16_split(words[w], sc[i], h4, l4);
#pragma unroll
              for (int q = 0; q < 4; ++q)
              {
                outw[4 * w + q] = h4[q];
                outl[(WMODE == W_I4S) ? (4 * w + q) : 0] = l4[q];
              }
            }
          }
          else
          {
#pragma unroll
            for (int w = 0; w < 4; ++w)
            {
              uint32_t o4[4];
              int4x8_to_bf16(words[w], pack_bf16x2(sc[i], sc[i]), o4);
              outw[4 * w + 0] = o4[0];
              outw[4 * w + 1] = o4[1];
              outw[4 * w + 2] = o4[2];
              outw[4 * w + 3] = o4[3];
            }
          }
          const int r = c_row[i];
          const int first = c_part[i] * (ELEMS / 8);  // first 16-byte bf16 chunk along the contiguous direction
#pragma unroll
          for (int j = 0; j < ELEMS / 8; ++j)
          {
            const int cb = first + j;
            uint32_t dst;
            if (BWD)
            {
              // MN-major: 64-wide n blocks (8 KB apart), 8-row k groups (1 KB), 128-byte rows, 16-byte chunks XOR row%8
              dst = bbase + static_cast<uint32_t>((cb >> 3) * 8192 + (r >> 3) * 1024 + (r & 7) * 128 +
                                                  (((cb & 7) ^ (r & 7)) << 4));
            }
            else
            {
              // K-major: rows n of 128 bytes, 16-byte chunks XOR row%8
              dst = bbase + static_cast<uint32_t>(r * 128 + ((cb ^ (r & 7)) << 4));
            }
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(outw[4 * j + 0]),
                         "r"(outw[4 * j + 1]), "r"(outw[4 * j + 2]), "r"(outw[4 * j + 3])
                         : "memory");
            if (WMODE == W_I4S)
            {
              constexpr int L = (WMODE == W_I4S) ? 1 : 0;
              asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + static_cast<uint32_t>(B_PLANE_BYTES)),
                           "r"(outl[L * (4 * j + 0)]), "r"(outl[L * (4 * j + 1)]), "r"(outl[L * (4 * j + 2)]),
                           "r"(outl[L * (4 * j + 3)])
                           : "memory");
            }
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0)
        {
          arrive_lead(b_full(s));
        }
        if (PREFETCH)
        {
#pragma unroll
          for (int i = 0; i < PER_THREAD; ++i)
          {
            raw[i] = nraw[i];
            sc[i] = nsc[i];
          }
        }
      }
      if (p.lora_rhs != nullptr && ((gkb0 + static_cast<uint32_t>(num_kb)) % DEQ_TEAMS) == static_cast<uint32_t>(team))
      {
        // LoRA k-block (number num_kb, so one team's): the padded factor is bf16 already; copy its
        // tile into the operand layout
        const uint32_t gkb = gkb0 + static_cast<uint32_t>(num_kb);
        const int s = static_cast<int>(gkb % STAGES);
        const uint32_t par = (gkb / STAGES) & 1u;
        wait(empty(s), par ^ 1u);
        const uint32_t bbase = b_addr(s);
#pragma unroll
        for (int i = 0; i < (BNC * BK * 2 / 16) / TEAM_THREADS; ++i)
        {
          const int c = d + i * TEAM_THREADS;  // 16-byte chunk of the BNC x 64 bf16 tile
          uint32_t dst;
          const uint8_t *src;
          if (BWD)
          {
            const int r = c / (BNC / 8);   // k row (0..63) of the [64, N] factor
            const int cb = c % (BNC / 8);  // 16-byte chunk along n
            src = p.lora_rhs + (static_cast<int64_t>(r) * p.n_total + n0 + cb * 8) * 2;
            dst = bbase + static_cast<uint32_t>((cb >> 3) * 8192 + (r >> 3) * 1024 + (r & 7) * 128 +
                                                (((cb & 7) ^ (r & 7)) << 4));
          }
          else
          {
            const int r = c >> 3;  // n row (0..127) of the [N, 64] factor
            const int cb = c & 7;
            src = p.lora_rhs + (static_cast<int64_t>(n0 + r) * 64 + cb * 8) * 2;
            dst = bbase + static_cast<uint32_t>(r * 128 + ((cb ^ (r & 7)) << 4));
          }
          const uint4 v = __ldg(reinterpret_cast<const uint4 *>(src));
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                       : "memory");
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0)
        {
          arrive_lead(b_full(s));
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  uint32_t gave_up = *abort_word;
  if (PAIR)
  {
    // every role of both CTAs has left its loops; a give-up in either CTA is handled by both
    cluster_sync_all();
    gave_up |= ld_shared_cluster(map_to_cta(smem_u32(&cta_abort), rank ^ 1u));
  }
  if (gave_up != 0u && warp == 0 && lane == 0)
  {
    // activation tiles that were started may still be on their way: give them time to land before the
    // CTA's shared memory goes back (a copy must not arrive in memory that belongs to another CTA)
    for (int i = 0; i < 64; ++i)
    {
      __nanosleep(2000);
    }
  }
  if (gave_up != 0u && warp == 1 && rank == 0)
  {
    // MMAs issued after the give-up may still run: tensor memory is released only after they have
    // completed (a commit tracks every MMA issued before it); bounded like every other wait
    if (elect_one())
    {
      if (PAIR)
      {
        umma_commit_pair_local(smem_u32(&drain_bar));
      }
      else
      {
        umma_commit(smem_u32(&drain_bar));
      }
    }
    __syncwarp();
    const uint32_t addr = smem_u32(&drain_bar);
    bool done = false;
    for (uint32_t spin = 0; spin < p.spin_limit && !done; ++spin)
    {
      uint32_t ok;
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(ok)
          : "r"(addr), "r"(0u)
          : "memory");
      done = ok != 0;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR)
  {
    // neither CTA's shared or tensor memory is touched by the other one after this
    cluster_sync_all();
  }
  if (warp == 1)
  {
    tc_fence_after();
    if (PAIR)
    {
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    else
    {
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn()
{
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr)
  {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
    {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  }
  return fn;
}

// 2-D bf16 tensor map: `inner` contiguous elements per row, `outer` rows, box of 64 x box_rows, 128-byte swizzle.
int make_map_bf16(CUtensorMap *map, const void *base, uint64_t inner, uint64_t outer, uint32_t box_rows)
{
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr)
  {
    set_error("frozen linear (umma): cuTensorMapEncodeTiled is not available from the driver");
    return CAIFQ_ERR_CUDA;
  }
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {inner * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
  {
    set_error("frozen linear (umma): cuTensorMapEncodeTiled failed with %d", static_cast<int>(r));
    return CAIFQ_ERR_CUDA;
  }
  return CAIFQ_OK;
}

// A host that runs a collective beside these persistent kernels leaves it some SMs: a CTA here takes
// a whole SM, and one that finds its SM taken waits for the collective to end.
int sm_count_umma() { return persistent_ctas("CAIFQ_UMMA_CTAS"); }

// CTA pairs that a launch may use (a pair takes the two SMs of one TPC)
int pair_count_umma() { return sm_count_umma() / 2; }

// smallest number of resident pairs any pair-mode kernel reported for a device so far (0 = none launched yet)
std::atomic<int> g_pair_capacity[kMaxDevices];

// Whether 256-wide tiles go to CTA pairs or to single CTAs.  Measured on 4096 x 4096, 8192 tokens: a bf16
// weight (operand fed by copies alone) runs 9 % faster on pairs (1211-1327 against 1109-1219 TFLOP/s); a
// quantized weight does not (int8 980-1150 on pairs, 1026-1140 on single CTAs; int4 950-1015 against
// 1007-1190): there the dequant warps' work per flop is the same in both forms and it, not the operand traffic,
// is the limit.  So pairs are the default for bf16 weights only; CAIFQ_UMMA_PAIR=1 / 0 forces them on / off.
bool pairs_enabled(int mode)
{
  const char *e = std::getenv("CAIFQ_UMMA_PAIR");
  if (e == nullptr)
  {
    return mode == W_BF16;
  }
  return std::atoi(e) != 0;
}

template <int WMODE, bool BWD, int BN, bool GROUPED, bool PAIR = false>
int launch_inst(const CUtensorMap &map_a, const CUtensorMap &map_b, const CUtensorMap &map_h, const CUtensorMap &map_l,
                const UmmaParams &p,
                const typename GroupSel<GROUPED>::type &gt, cudaStream_t s)
{
  auto kernel = linear_umma_kernel<WMODE, BWD, BN, GROUPED, PAIR>;
  constexpr int SMEM_BYTES = TileCfg<BN, planes_of(WMODE), PAIR>::SMEM_BYTES;
  static std::atomic<bool> configured[kMaxDevices];
  int dev = 0;
  CAIFQ_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices)
  {
    set_error("frozen linear (umma): device ordinal %d out of range", dev);
    return CAIFQ_ERR_UNSUPPORTED;
  }
  if (!configured[dev].load(std::memory_order_acquire))
  {
    CAIFQ_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured[dev].store(true, std::memory_order_release);
  }
  const int64_t tiles = static_cast<int64_t>(p.num_m_tiles) * p.num_n_tiles;
  if (PAIR)
  {
    cudaLaunchConfig_t cfg{};
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // The grid is persistent, so it must not hold more pairs than the device keeps resident at a time (a
    // pair that waited for another one to finish would double the launch's time): ask once per device.
    static std::atomic<int> resident[kMaxDevices];
    int cap = resident[dev].load(std::memory_order_acquire);
    if (cap == 0)
    {
      cfg.gridDim = dim3(static_cast<unsigned>(2 * (device_sm_count() / 2)), 1, 1);
      int clusters = 0;
      CAIFQ_CHECK_CUDA(cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg));
      cap = clusters > 0 ? clusters : 1;
      resident[dev].store(cap, std::memory_order_release);
      int seen = g_pair_capacity[dev].load(std::memory_order_relaxed);
      while ((seen == 0 || cap < seen) && !g_pair_capacity[dev].compare_exchange_weak(seen, cap))
      {
      }
    }
    int pairs = pair_count_umma() < cap ? pair_count_umma() : cap;
    if (tiles < pairs)
    {
      pairs = static_cast<int>(tiles);
    }
    cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs), 1, 1);
    CAIFQ_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, map_h, map_l, p, gt));
    return CAIFQ_OK;
  }
  const int grid = tiles < sm_count_umma() ? static_cast<int>(tiles) : sm_count_umma();
  kernel<<<grid, NUM_THREADS, SMEM_BYTES, s>>>(map_a, map_b, map_h, map_l, p, gt);
  CAIFQ_CHECK_LAUNCH();
  return CAIFQ_OK;
}

int wmode_of(const caifq_weight &w, int compute_dtype)
{
  if (w.storage == CAIFQ_I8)
  {
    return W_I8;
  }
  if (w.storage == CAIFQ_I4)
  {
    return (compute_dtype == CAIFQ_F32) ? W_I4S : W_I4;
  }
  return W_BF16;
}

}  // namespace

int umma_pair_capacity()
{
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
  {
    cudaGetLastError();
    return 0;
  }
  return g_pair_capacity[dev].load(std::memory_order_relaxed);
}

bool umma_supported(const LinearArgs &g)
{
  const caifq_weight &w = g.w;
  // (calls of up to 16 tokens are the few-token kernel's; from 17 on one 256-row tile, mostly
  // zero rows, still beats the fp32-FMA kernel by far)
  if (g.a_dtype != CAIFQ_BF16 || g.a_prescale != 1.0f || g.m < 17)
  {
    return false;
  }
  const int n_total = g.backward ? w.in_dim : w.out_dim;
  const int k_total = g.backward ? w.out_dim : w.in_dim;
  if ((n_total % 128) != 0 || (k_total % BK) != 0)
  {
    return false;
  }
  if ((reinterpret_cast<uintptr_t>(g.a) & 15u) != 0 || (reinterpret_cast<uintptr_t>(g.c) & 15u) != 0 ||
      (reinterpret_cast<uintptr_t>(w.codes) & 15u) != 0)
  {
    return false;
  }
  switch (w.storage)
  {
    case CAIFQ_I8:
      // per-tensor scale (or none) factors out of the product: exact for fp32 and bf16 compute
      if (w.scales != nullptr && w.scheme != CAIFQ_PER_TENSOR)
      {
        return false;
      }
      return g.compute_dtype == CAIFQ_BF16 || g.compute_dtype == CAIFQ_F32;
    case CAIFQ_I4:
      // bf16 compute: scale*code rounded once to bf16, the reference's value; fp32 compute: scale*code
      // as two bf16 terms (2^-17 relative), within the fp32 tolerance
      if ((g.compute_dtype != CAIFQ_BF16 && g.compute_dtype != CAIFQ_F32) || w.scales == nullptr)
      {
        return false;
      }
      return (w.group_size % 32) == 0 && (w.in_dim % w.group_size) == 0;
    case CAIFQ_BF16:
      // bf16 x bf16 products are exact in fp32
      return g.compute_dtype == CAIFQ_BF16 || g.compute_dtype == CAIFQ_F32;
    default:
      return false;
  }
}

int launch_linear_umma(const LinearArgs &g, cudaStream_t s)
{
  const caifq_weight &w = g.w;
  UmmaParams p{};
  p.spin_limit = kSpinLimit;
  p.stall_bytes = 0;
  if (t_umma_stall_next)
  {
    // self-test of the give-up path: the first activation tile announces 16 bytes that never arrive
    t_umma_stall_next = false;
    p.spin_limit = kSpinLimitTest;
    p.stall_bytes = 16;
  }
  p.codes = static_cast<const uint8_t *>(w.codes);
  p.scales = w.scales;
  p.c = g.c;
  p.c_dtype = g.c_dtype;
  p.accumulate = g.accumulate ? 1 : 0;
  p.m = g.m;
  p.n_total = g.backward ? w.in_dim : w.out_dim;
  p.k_total = g.backward ? w.out_dim : w.in_dim;
  p.in_dim = w.in_dim;
  p.group_size = w.group_size;
  p.groups_per_row = (w.group_size > 0) ? w.in_dim / w.group_size : 0;
  p.num_m_tiles = static_cast<int>((g.m + BM - 1) / BM);
  // 256-wide tiles feed the tensor core better per shared-memory byte; 128-wide ones keep a
  // second accumulator set so the epilogue overlaps the next tile.  CAIFQ_UMMA_BN overrides.
  // A 256-wide tile goes to a CTA pair (half the operand bytes per SM and flop, two accumulator sets) when
  // there are enough tiles for the pairs, else to a single CTA when there are enough for the SMs.
  const int mode = wmode_of(w, g.compute_dtype);
  const bool pair = pairs_enabled(mode) && (p.n_total % 256) == 0 &&
                    static_cast<int64_t>(p.num_m_tiles) * (p.n_total / 256) >= pair_count_umma();
  int bn = (pair || ((p.n_total % 256) == 0 &&
                     static_cast<int64_t>(p.num_m_tiles) * (p.n_total / 256) >= sm_count_umma()))
               ? 256
               : 128;
  if (const char *e = std::getenv("CAIFQ_UMMA_BN"))
  {
    const int v = std::atoi(e);
    if (v == 128 || (v == 256 && (p.n_total % 256) == 0))
    {
      bn = v;
    }
  }
  if (w.storage == CAIFQ_I4 && g.compute_dtype == CAIFQ_F32 && !(pair && bn == 256))
  {
    bn = 128;   // a single CTA has 128-wide tiles only in the two-plane mode
  }
  p.num_n_tiles = p.n_total / bn;

  CUtensorMap map_a;
  CUtensorMap map_b;
  int rc = make_map_bf16(&map_a, g.a, static_cast<uint64_t>(p.k_total), static_cast<uint64_t>(g.m), BM_SUB);
  if (rc != CAIFQ_OK)
  {
    return rc;
  }
  if (mode == W_BF16)
  {
    // the [out, in] weight itself: forward boxes are 64 k x 128 n rows, backward 64 n x 64 k rows
    rc = make_map_bf16(&map_b, w.codes, static_cast<uint64_t>(w.in_dim), static_cast<uint64_t>(w.out_dim),
                       g.backward ? BK : ((pair && bn == 256) ? 128 : bn));
    if (rc != CAIFQ_OK)
    {
      return rc;
    }
  }
  else
  {
    map_b = map_a;
  }
  CUtensorMap map_h = map_a;
  CUtensorMap map_l = map_b;
  p.c_scale = (mode == W_BF16) ? g.c_scale : nullptr;
  if (g.lora_lhs != nullptr && g.lora_rhs != nullptr)
  {
    rc = make_map_bf16(&map_h, g.lora_lhs, 64, static_cast<uint64_t>(g.m), BM_SUB);
    if (rc != CAIFQ_OK)
    {
      return rc;
    }
    p.lora_rhs = static_cast<const uint8_t *>(g.lora_rhs);
    if (mode == W_BF16)
    {
      // the padded factor as a copy source: [N, 64] (forward, boxes of 64 k x the CTA's rows) or
      // [64, N] (backward, boxes of 64 n x 64 k), like the weight itself
      rc = g.backward ? make_map_bf16(&map_l, g.lora_rhs, static_cast<uint64_t>(p.n_total), 64, BK)
                      : make_map_bf16(&map_l, g.lora_rhs, 64, static_cast<uint64_t>(p.n_total),
                                      (pair && bn == 256) ? 128 : bn);
      if (rc != CAIFQ_OK)
      {
        return rc;
      }
    }
  }
#define CAIFQ_UMMA_PAIR_CASE(MODE)                                                                      \
  if (mode == MODE && bn == 256 && pair)                                                                \
  {                                                                                                     \
    return g.backward ? launch_inst<MODE, true, 256, false, true>(map_a, map_b, map_h, map_l, p, NoGroupTable{}, s)   \
                      : launch_inst<MODE, false, 256, false, true>(map_a, map_b, map_h, map_l, p, NoGroupTable{}, s); \
  }
  CAIFQ_UMMA_PAIR_CASE(W_I8)
  CAIFQ_UMMA_PAIR_CASE(W_I4)
  CAIFQ_UMMA_PAIR_CASE(W_BF16)
  CAIFQ_UMMA_PAIR_CASE(W_I4S)
#undef CAIFQ_UMMA_PAIR_CASE
#define CAIFQ_UMMA_CASE(MODE)                                                        \
  if (mode == MODE && bn == 128)                                                     \
  {                                                                                  \
    return g.backward ? launch_inst<MODE, true, 128, false>(map_a, map_b, map_h, map_l, p, NoGroupTable{}, s)   \
                      : launch_inst<MODE, false, 128, false>(map_a, map_b, map_h, map_l, p, NoGroupTable{}, s); \
  }                                                                                  \
  if (mode == MODE && bn == 256)                                                     \
  {                                                                                  \
    return g.backward ? launch_inst<MODE, true, 256, false>(map_a, map_b, map_h, map_l, p, NoGroupTable{}, s)   \
                      : launch_inst<MODE, false, 256, false>(map_a, map_b, map_h, map_l, p, NoGroupTable{}, s); \
  }
  CAIFQ_UMMA_CASE(W_I8)
  CAIFQ_UMMA_CASE(W_I4)
  CAIFQ_UMMA_CASE(W_BF16)
#undef CAIFQ_UMMA_CASE
  if (mode == W_I4S)   // two operand planes: 128-wide tiles only
  {
    return g.backward ? launch_inst<W_I4S, true, 128, false>(map_a, map_b, map_h, map_l, p, NoGroupTable{}, s)
                      : launch_inst<W_I4S, false, 128, false>(map_a, map_b, map_h, map_l, p, NoGroupTable{}, s);
  }
  set_error("frozen linear (umma): unsupported weight storage %d", w.storage);
  return CAIFQ_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------ grouped (frozen experts)
bool umma_grouped_supported(const GroupedLinearArgs &g)
{
  if (g.num_experts < 1 || g.weights == nullptr || g.offsets == nullptr)
  {
    return false;
  }
  const caifq_weight &w0 = g.weights[0];
  if (w0.storage != CAIFQ_I8 && w0.storage != CAIFQ_I4 && w0.storage != CAIFQ_BF16)
  {
    return false;
  }
  if (w0.storage == CAIFQ_BF16)
  {
    // bf16 experts (expanded copies) are fed by tile copies from ONE tensor map: their matrices must lie
    // stacked, expert e at e * out * in elements behind expert 0
    const size_t stride = static_cast<size_t>(w0.in_dim) * static_cast<size_t>(w0.out_dim) * 2;
    for (int e = 0; e < g.num_experts; ++e)
    {
      if (static_cast<const char *>(g.weights[e].codes) != static_cast<const char *>(w0.codes) + e * stride)
      {
        return false;
      }
    }
  }
  LinearArgs probe{};
  probe.w = w0;
  probe.backward = g.backward;
  probe.a = g.a;
  probe.a_dtype = g.a_dtype;
  probe.a_prescale = 1.0f;
  probe.m = 32;   // the row count of a single expert does not matter here
  probe.c = g.c;
  probe.c_dtype = g.c_dtype;
  probe.accumulate = g.accumulate;
  probe.compute_dtype = g.compute_dtype;
  if (!umma_supported(probe))
  {
    return false;
  }
  for (int e = 0; e < g.num_experts; ++e)
  {
    const caifq_weight &w = g.weights[e];
    if (w.storage != w0.storage || w.scheme != w0.scheme || w.group_size != w0.group_size || w.in_dim != w0.in_dim ||
        w.out_dim != w0.out_dim || (w.scales == nullptr) != (w0.scales == nullptr) ||
        (reinterpret_cast<uintptr_t>(w.codes) & 15u) != 0)
    {
      return false;
    }
  }
  return g.offsets[g.num_experts] > 0;
}

int launch_linear_umma_grouped(const GroupedLinearArgs &g, cudaStream_t s)
{
  const caifq_weight &w0 = g.weights[0];
  const int64_t total_rows = g.offsets[g.num_experts];
  UmmaParams p{};
  p.spin_limit = kSpinLimit;
  p.stall_bytes = 0;
  p.codes = nullptr;
  p.scales = nullptr;
  p.c = g.c;
  p.c_dtype = g.c_dtype;
  p.accumulate = g.accumulate ? 1 : 0;
  p.m = total_rows;
  p.n_total = g.backward ? w0.in_dim : w0.out_dim;
  p.k_total = g.backward ? w0.out_dim : w0.in_dim;
  p.in_dim = w0.in_dim;
  p.group_size = w0.group_size;
  p.groups_per_row = (w0.group_size > 0) ? w0.in_dim / w0.group_size : 0;
  if (g.backward && g.sb_gate != nullptr && g.sb_up != nullptr && g.sb_g_up != nullptr && g.c_dtype == CAIFQ_BF16 &&
      !g.accumulate)
  {
    p.sb_gate = g.sb_gate;
    p.sb_up = g.sb_up;
    p.sb_g_up = g.sb_g_up;
  }
  CUtensorMap map_a;
  int rc = make_map_bf16(&map_a, g.a, static_cast<uint64_t>(p.k_total), static_cast<uint64_t>(total_rows), BM_SUB);
  if (rc != CAIFQ_OK)
  {
    return rc;
  }
  const int mode = wmode_of(w0, g.compute_dtype);
  for (int first = 0; first < g.num_experts; first += MAX_GROUPS)
  {
    const int count = (g.num_experts - first < MAX_GROUPS) ? (g.num_experts - first) : MAX_GROUPS;
    GroupTable gt{};
    int tiles = 0;
    for (int e = 0; e < count; ++e)
    {
      gt.offsets[e] = g.offsets[first + e];
      gt.mtile_start[e] = tiles;
      tiles += (g.offsets[first + e + 1] - g.offsets[first + e] + BM - 1) / BM;
      gt.codes[e] = static_cast<const uint8_t *>(g.weights[first + e].codes);
      gt.scales[e] = g.weights[first + e].scales;
    }
    gt.offsets[count] = g.offsets[first + count];
    gt.mtile_start[count] = tiles;
    gt.num_groups = count;
    if (tiles == 0)
    {
      continue;
    }
    p.num_m_tiles = tiles;
    // (for the experts' shapes the wide tile measured 3 % faster with int4 too, unlike the square case)
    // (an accumulating epilogue reads the output first: with 128-wide tiles it overlaps the next tile)
    // (pairs keep two accumulator sets at 256 columns, so the accumulating epilogue and the two-plane mode
    // can have the wide tile there)
    if (mode == W_BF16)
    {
      // stacked bf16 experts: one map over [count * out, in]; pairs when the width allows, else 128-wide tiles
      // (a width that is a multiple of 128 only, like 1408, still takes 256-wide pair tiles: the last tile's upper
      // half is masked in the epilogue, 9 % of wasted MMAs against 62 -> 85 % tensor activity)
      const int wide_tiles = (p.n_total + 255) / 256;
      const bool wide = static_cast<int64_t>(tiles) * wide_tiles >= pair_count_umma() && pairs_enabled(mode);
      p.num_n_tiles = wide ? wide_tiles : p.n_total / 128;
      p.expert_rows = w0.out_dim;
      CUtensorMap map_b;
      rc = make_map_bf16(&map_b, g.weights[first].codes, static_cast<uint64_t>(w0.in_dim),
                         static_cast<uint64_t>(count) * static_cast<uint64_t>(w0.out_dim), g.backward ? BK : 128);
      if (rc != CAIFQ_OK)
      {
        return rc;
      }
      // second operand pair (dX of two projections that share their input: C = A.W + A2.W2 in one accumulation)
      CUtensorMap map_a2 = map_a;
      CUtensorMap map_b2 = map_b;
      p.dual_k = 0;
      if (g.weights2 != nullptr && g.a2 != nullptr)
      {
        rc = make_map_bf16(&map_a2, g.a2, static_cast<uint64_t>(p.k_total), static_cast<uint64_t>(total_rows), BM_SUB);
        if (rc == CAIFQ_OK)
        {
          rc = make_map_bf16(&map_b2, g.weights2[first].codes, static_cast<uint64_t>(w0.in_dim),
                             static_cast<uint64_t>(count) * static_cast<uint64_t>(w0.out_dim), g.backward ? BK : 128);
        }
        if (rc != CAIFQ_OK)
        {
          return rc;
        }
        p.dual_k = 1;
      }
      if (wide)
      {
        rc = g.backward ? launch_inst<W_BF16, true, 256, true, true>(map_a, map_b, map_a2, map_b2, p, gt, s)
                        : launch_inst<W_BF16, false, 256, true, true>(map_a, map_b, map_a2, map_b2, p, gt, s);
      }
      else
      {
        rc = g.backward ? launch_inst<W_BF16, true, 128, true>(map_a, map_b, map_a2, map_b2, p, gt, s)
                        : launch_inst<W_BF16, false, 128, true>(map_a, map_b, map_a2, map_b2, p, gt, s);
      }
      if (rc != CAIFQ_OK)
      {
        return rc;
      }
      continue;
    }
    const bool pair = pairs_enabled(mode) && (p.n_total % 256) == 0 &&
                      static_cast<int64_t>(tiles) * (p.n_total / 256) >= pair_count_umma();
    const int bn = (pair || (mode != W_I4S && !g.accumulate && (p.n_total % 256) == 0 &&
                             static_cast<int64_t>(tiles) * (p.n_total / 256) >= sm_count_umma()))
                       ? 256
                       : 128;
    p.num_n_tiles = p.n_total / bn;
#define CAIFQ_UMMA_GROUP_PAIR_CASE(MODE)                                                           \
  if (mode == MODE && pair)                                                                        \
  {                                                                                                \
    rc = g.backward ? launch_inst<MODE, true, 256, true, true>(map_a, map_a, map_a, map_a, p, gt, s)      \
                    : launch_inst<MODE, false, 256, true, true>(map_a, map_a, map_a, map_a, p, gt, s);    \
  }
    CAIFQ_UMMA_GROUP_PAIR_CASE(W_I8)
    CAIFQ_UMMA_GROUP_PAIR_CASE(W_I4)
    CAIFQ_UMMA_GROUP_PAIR_CASE(W_I4S)
#undef CAIFQ_UMMA_GROUP_PAIR_CASE
    if (pair)
    {
      if (rc != CAIFQ_OK)
      {
        return rc;
      }
      continue;
    }
#define CAIFQ_UMMA_GROUP_CASE(MODE)                                                              \
  if (mode == MODE && bn == 128)                                                                 \
  {                                                                                              \
    rc = g.backward ? launch_inst<MODE, true, 128, true>(map_a, map_a, map_a, map_a, p, gt, s)          \
                    : launch_inst<MODE, false, 128, true>(map_a, map_a, map_a, map_a, p, gt, s);        \
  }                                                                                              \
  if (mode == MODE && bn == 256)                                                                 \
  {                                                                                              \
    rc = g.backward ? launch_inst<MODE, true, 256, true>(map_a, map_a, map_a, map_a, p, gt, s)          \
                    : launch_inst<MODE, false, 256, true>(map_a, map_a, map_a, map_a, p, gt, s);        \
  }
    CAIFQ_UMMA_GROUP_CASE(W_I8)
    CAIFQ_UMMA_GROUP_CASE(W_I4)
#undef CAIFQ_UMMA_GROUP_CASE
    if (mode == W_I4S)
    {
      rc = g.backward ? launch_inst<W_I4S, true, 128, true>(map_a, map_a, map_a, map_a, p, gt, s)
                      : launch_inst<W_I4S, false, 128, true>(map_a, map_a, map_a, map_a, p, gt, s);
    }
    if (rc != CAIFQ_OK)
    {
      return rc;
    }
  }
  return CAIFQ_OK;
}

// ------------------------------------------------------------------ fused gate / up / SwiGLU
bool umma_swiglu_supported(const GroupedSwigluArgs &g)
{
  if (g.num_experts < 1 || g.gate == nullptr || g.up == nullptr || g.offsets == nullptr || g.dtype != CAIFQ_BF16)
  {
    return false;
  }
  GroupedLinearArgs probe{};
  probe.weights = g.gate;
  probe.num_experts = g.num_experts;
  probe.offsets = g.offsets;
  probe.backward = false;
  probe.a = g.x;
  probe.a_dtype = g.dtype;
  probe.c = g.gate_out;
  probe.c_dtype = g.dtype;
  probe.accumulate = false;
  probe.compute_dtype = g.compute_dtype;
  if (!umma_grouped_supported(probe))
  {
    return false;
  }
  probe.weights = g.up;
  probe.c = g.up_out;
  if (!umma_grouped_supported(probe))
  {
    return false;
  }
  const caifq_weight &w0 = g.gate[0];
  const caifq_weight &u0 = g.up[0];
  if (u0.storage != w0.storage || u0.scheme != w0.scheme || u0.group_size != w0.group_size ||
      u0.in_dim != w0.in_dim || u0.out_dim != w0.out_dim || (w0.out_dim % 64) != 0)
  {
    return false;
  }
  return (reinterpret_cast<uintptr_t>(g.hidden) & 15u) == 0 && (reinterpret_cast<uintptr_t>(g.up_out) & 15u) == 0;
}

int launch_linear_umma_swiglu(const GroupedSwigluArgs &g, cudaStream_t s)
{
  const caifq_weight &w0 = g.gate[0];
  const int64_t total_rows = g.offsets[g.num_experts];
  UmmaParams p{};
  p.spin_limit = kSpinLimit;
  p.stall_bytes = 0;
  p.c = g.gate_out;
  p.c_up = g.up_out;
  p.c_hidden = g.hidden;
  p.c_dtype = g.dtype;
  p.accumulate = 0;
  p.m = total_rows;
  p.n_total = 2 * w0.out_dim;   // gate and up features side by side in every tile
  p.k_total = w0.in_dim;
  p.in_dim = w0.in_dim;
  p.group_size = w0.group_size;
  p.groups_per_row = (w0.group_size > 0) ? w0.in_dim / w0.group_size : 0;
  p.swiglu = 1;
  CUtensorMap map_a;
  int rc = make_map_bf16(&map_a, g.x, static_cast<uint64_t>(p.k_total), static_cast<uint64_t>(total_rows), BM_SUB);
  if (rc != CAIFQ_OK)
  {
    return rc;
  }
  const int mode = wmode_of(w0, g.compute_dtype);
  for (int first = 0; first < g.num_experts; first += MAX_GROUPS)
  {
    const int count = (g.num_experts - first < MAX_GROUPS) ? (g.num_experts - first) : MAX_GROUPS;
    GroupTable gt{};
    int tiles = 0;
    for (int e = 0; e < count; ++e)
    {
      gt.offsets[e] = g.offsets[first + e];
      gt.mtile_start[e] = tiles;
      tiles += (g.offsets[first + e + 1] - g.offsets[first + e] + BM - 1) / BM;
      gt.codes[e] = static_cast<const uint8_t *>(g.gate[first + e].codes);
      gt.scales[e] = g.gate[first + e].scales;
      gt.codes_up[e] = static_cast<const uint8_t *>(g.up[first + e].codes);
      gt.scales_up[e] = g.up[first + e].scales;
    }
    gt.offsets[count] = g.offsets[first + count];
    gt.mtile_start[count] = tiles;
    gt.num_groups = count;
    if (tiles == 0)
    {
      continue;
    }
    p.num_m_tiles = tiles;
    // 128 features of each projection per tile on a CTA pair, 64 on a single CTA
    const bool pair = pairs_enabled(mode) && (w0.out_dim % 128) == 0 &&
                      static_cast<int64_t>(tiles) * (w0.out_dim / 128) >= pair_count_umma();
    p.num_n_tiles = w0.out_dim / (pair ? 128 : 64);
    if (mode == W_BF16)
    {
      p.expert_rows = w0.out_dim;
      CUtensorMap map_g;
      CUtensorMap map_u;
      const uint64_t rows = static_cast<uint64_t>(count) * static_cast<uint64_t>(w0.out_dim);
      rc = make_map_bf16(&map_g, g.gate[first].codes, static_cast<uint64_t>(w0.in_dim), rows, pair ? 128 : 64);
      if (rc == CAIFQ_OK)
      {
        rc = make_map_bf16(&map_u, g.up[first].codes, static_cast<uint64_t>(w0.in_dim), rows, pair ? 128 : 64);
      }
      if (rc != CAIFQ_OK)
      {
        return rc;
      }
      rc = pair ? launch_inst<W_BF16, false, 256, true, true>(map_a, map_g, map_a, map_u, p, gt, s)
                : launch_inst<W_BF16, false, 128, true>(map_a, map_g, map_a, map_u, p, gt, s);
    }
    else if (pair)
    {
      if (mode == W_I8)
      {
        rc = launch_inst<W_I8, false, 256, true, true>(map_a, map_a, map_a, map_a, p, gt, s);
      }
      else if (mode == W_I4S)
      {
        rc = launch_inst<W_I4S, false, 256, true, true>(map_a, map_a, map_a, map_a, p, gt, s);
      }
      else
      {
        rc = launch_inst<W_I4, false, 256, true, true>(map_a, map_a, map_a, map_a, p, gt, s);
      }
    }
    else if (mode == W_I8)
    {
      rc = launch_inst<W_I8, false, 128, true>(map_a, map_a, map_a, map_a, p, gt, s);
    }
    else if (mode == W_I4S)
    {
      rc = launch_inst<W_I4S, false, 128, true>(map_a, map_a, map_a, map_a, p, gt, s);
    }
    else
    {
      rc = launch_inst<W_I4, false, 128, true>(map_a, map_a, map_a, map_a, p, gt, s);
    }
    if (rc != CAIFQ_OK)
    {
      return rc;
    }
  }
  return CAIFQ_OK;
}

}  // namespace caifq
