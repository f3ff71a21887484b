// M<=16 int4 (group 64, bf16) matmul on the 5th-generation tensor cores: tcgen05.mma with the dequantised
// weights as the A operand in TENSOR MEMORY, the activations as the B operand in shared memory and the fp32
// accumulator in tensor memory.  Same contract as qmm_stream_kernel (qmm.cu); replaces the same reference code
// (dflash_mlx/verify_qmm.py:28-331).
//
// Numerics are the reference's own: every weight is dequantised to bf16, w_hat = bf16(nib * scale + bias)
// (verify_qmm.py:75), and the tensor core accumulates x . w_hat over K in fp32.
//
// Dequantisation costs 9 instructions per 8 weights and is exact.  A 16-bit pattern 0x00vv (v < 256) read as bf16 is
// the number v * 2^-133 (the subnormals and the first binade share one spacing), so for a packed word w
//     w & 0x000F000F        = the bf16 pair (nib0, nib4) * 2^-133
//     w & 0x00F000F0        = the pair (nib1, nib5) * 16 * 2^-133
//     (w >> 8) & ...        = the pairs (nib2, nib6) and (nib3, nib7) likewise
// and ONE fma.rn.bf16x2 per pair with the group's pre-scaled constants (scale * 2^101 or scale * 2^97, bias * 2^-32)
// gives bf16(nib * scale + bias) * 2^-32 with a single rounding; the power of two comes off in the epilogue.
// (Scales must be below 2^26 in magnitude; weights below 2^-94 lose precision - neither occurs in a quantised model.)
// The pairs come out in the k order (0,4,1,5,2,6,3,7) inside every 8-block; the activations are put into shared
// memory in the same order, so nothing is shuffled.
//
// Work: unit = 128 weight rows x 8 groups (512 k).  The units of the whole matrix, row tile major, are dealt to the
// CTAs (1 per SM) as equal contiguous spans (stream-K): a CTA streams the same number of bytes whatever the shape, a
// row tile is cut only where a span ends, and only such a tile goes through fp32 partial tiles in the workspace.
// A pipeline stage (4 of them, 52 KB) holds one unit: its packed weights (two 128B-swizzled TMA boxes), scales and
// biases (TMA) and the 16 x 512 slice of the activations it multiplies, as the K-major core-matrix tiles the MMA reads.
// Roles meet only through mbarriers; between dequantisation and MMA the hand-over unit is a PAIR of quantisation
// groups (128 k) of the 128 rows, held in one of 6 operand buffers of 64 TMEM columns:
//   producer warp  : TMEM allocation; TMA loads of a unit's weights, scales and biases.
//   loader warps   : the unit's activations, global (L2) -> registers -> permuted -> shared memory.
//   dequant warps  : a thread owns ONE weight row (its TMEM lane); the four warps of a slot cover the 128 rows and take
//                    every kSlots-th pair.  Per pair: wait(stage landed) -> 4 x LDS.128 -> wait(operand buffer free) ->
//                    AND/FMA -> 2 x tcgen05.st (32 columns each) -> arrive(operand ready).
//   issuing threads: 6 warps with one issuing thread each (measured: a warp issues one tcgen05.mma per ~131 cycles
//                    whatever its shape, while several warps together reach one per ~17 cycles); thread i issues the
//                    four MMAs of group h = i & 1 of the pairs p with p mod 3 == i >> 1 into its OWN 16 accumulator
//                    columns (MMAs of different threads are not ordered against each other), over all its pairs of a
//                    segment (= this CTA's units of one row tile): wait(operand ready) -> 4 x tcgen05.mma M128 x N16 x
//                    K16 -> tcgen05.commit(operand free); after its last pair of a unit tcgen05.commit(stage free),
//                    after its last pair of the segment tcgen05.commit(accumulators ready).
//   epilogue warps : once per segment: wait(accumulators ready) -> tcgen05.ld of the 6 accumulators -> sum ->
//                    arrive(accumulators free) -> store y, or write an fp32 partial tile, take the tile's ticket and,
//                    if it was the last one, sum the tile's partial tiles in a fixed order.
// An mbarrier wait by parity is only right for a waiter at most one phase behind, so every operand buffer is always
// written by the same warps and read by the same issuing threads (slot and class counts divide the ring size).
// Every wait is bounded and reports through the device error word.
#include <stdio.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace dflash {
namespace tc {

constexpr int kRows = 128;               // weight rows per tile
constexpr int kG = 64;                   // quantisation group
constexpr int kBK = 8 * kG;              // k per unit
constexpr int kEpWarps = 4, kXWarps = 4;
constexpr int kEp = kEpWarps * 32;
constexpr int kTileF4 = 512;             // float4 entries of one fp32 partial tile: [token quad][row]
constexpr int kStages = 4;
constexpr int kEarlyUnits = 2;           // units whose weights are requested before the wait on the previous kernel
constexpr int kWBytes = kRows * (kBK / 2);    // 32 KB
constexpr int kSBBytes = kRows * 16;          // 2 KB
constexpr int kXOff = kWBytes + 2 * kSBBytes; // the activation tile of a stage: 8 slabs of [16 tok][64 k] bf16, 128B swizzle
constexpr int kXTileBytes = kBK * 32;         // 16 KB
constexpr int kTmaBytes = kXOff;              // bytes of a stage that arrive by TMA
constexpr int kStageBytes = kXOff + kXTileBytes;
constexpr int kMaxRowTiles = 16384;
constexpr int kNA = 6;                   // operand buffers of 64 TMEM columns (one PAIR of quantisation groups each)
constexpr int kNumBars = 3 * kStages + 2 * kNA + 2;  // full, empty, x_landed, a_ready, a_free, d_ready, d_free
constexpr size_t kSmemBytes = 1024 + (size_t)kStages * kStageBytes + 8 * kNumBars + 128;
constexpr uint32_t kTmemCols = 512;      // operand buffers at columns 0..383, accumulators at 384..479
constexpr uint32_t kDCol0 = 64 * kNA;
#ifndef DFLASH_TC_STAGGER_NS
#define DFLASH_TC_STAGGER_NS 0
#endif
constexpr unsigned kStaggerNs = DFLASH_TC_STAGGER_NS;
constexpr float kPow2Scale = 0x1p101f;   // 2^(133 - 32)
constexpr float kPow2Scale16 = 0x1p97f;  // the same for a nibble that sits 4 bits higher
constexpr float kPow2Bias = 0x1p-32f;
constexpr float kPow2Out = 0x1p32f;

// C = units per row tile, NT = row tiles, ctas = CTAs that have work (each >= 1 unit), maxp = most CTAs a tile is cut over
struct Plan {
  int M, K, N, NT, C, ctas, maxp;
};

__device__ __forceinline__ int cta_of(unsigned u, unsigned units, unsigned ctas) {
  return (int)(((u + 1u) * ctas - 1u) / units);
}
// How many CTAs contribute to row tile nt, and the first of them.
__device__ __forceinline__ int tile_pieces(const Plan& p, int nt, int* first) {
  const unsigned units = (unsigned)p.NT * (unsigned)p.C;
  const int a = cta_of((unsigned)nt * p.C, units, p.ctas);
  const int b = cta_of((unsigned)(nt + 1) * p.C - 1u, units, p.ctas);
  *first = a;
  return b - a + 1;
}

// ---- tcgen05 wrappers ----------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_holder, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_holder), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[128 x 16] (+)= A[128 x 16] (TMEM, bf16) * B[16 x 16] (shared memory descriptor, bf16)
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accum)
      : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// Asynchronous TMEM load of 16 columns; the registers may only be read after tc_ld16_wait on the same array.
__device__ __forceinline__ void tc_ld16_issue(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// The in/out operands tie every later use of the registers to this wait (the compiler cannot hoist them above it).
__device__ __forceinline__ void tc_ld16_wait(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                 "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}
// Shared-memory matrix descriptor, K-major, no swizzle: core matrix = 8 rows x 16 bytes stored as 128 contiguous
// bytes; lbo = byte distance between core matrices along K, sbo = along the row (N) direction.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) |
         ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46);
}
// The same for the 128B-swizzled K-major layout a TMA box of 128-byte rows produces: rows of 128 bytes (64 k), 8-row
// groups 1024 bytes apart (sbo), the leading offset is not used.  The tile must start on a 1024-byte boundary; a k16
// step inside the 128-byte row is taken by advancing the start address by 32 bytes.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor, kind::f16: D = f32, A = B = bf16, both K-major, N = 16, M = 128.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// both halves = bf16(v), round to nearest even
__device__ __forceinline__ uint32_t bf16x2_dup(float v) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %1;" : "=r"(d) : "f"(v));
  return d;
}

// Eight packed words (one quantisation group of one row) -> 32 bf16 pairs, see the head of the file.
__device__ __forceinline__ void dequant_group(const uint4& wa, const uint4& wb, uint32_t S, uint32_t S16, uint32_t B,
                                              uint32_t (&o)[32]) {
  const uint32_t w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t w8 = w[j] >> 8;
    o[4 * j + 0] = fma_bf16x2(w[j] & 0x000F000Fu, S, B);
    o[4 * j + 1] = fma_bf16x2(w[j] & 0x00F000F0u, S16, B);
    o[4 * j + 2] = fma_bf16x2(w8 & 0x000F000Fu, S, B);
    o[4 * j + 3] = fma_bf16x2(w8 & 0x00F000F0u, S16, B);
  }
}

__device__ __forceinline__ void store_row(const float (&v)[16], __nv_bfloat16* __restrict__ y,
                                          const __nv_bfloat16* __restrict__ bias, int n, int M, int N) {
  if (n >= N) return;
  const float bv = bias ? __bfloat162float(bias[n]) : 0.f;
#pragma unroll
  for (int t = 0; t < 16; ++t)
    if (t < M) y[(size_t)t * N + n] = __float2bfloat16_rn(v[t] + bv);
}

// The epilogue warp that took the last ticket of its 32-row slice of row tile nt sums that slice's partial tiles in
// piece order (fixed: deterministic); thread r owns row r.  The loads of up to four partial tiles are in flight together.
__device__ __noinline__ void finalize_slice(const Plan& plan, const float4* pieces, __nv_bfloat16* __restrict__ y,
                                               const __nv_bfloat16* __restrict__ bias, int nt, int np, int r) {
  float4 v[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) v[q] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int p0 = 0; p0 < np; p0 += 4) {
    float4 a[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (p0 + i < np) {
        const float4* src = &pieces[((size_t)(p0 + i) * plan.NT + nt) * kTileF4 + r];
#pragma unroll
        for (int q = 0; q < 4; ++q) a[i][q] = ld_cg_f4(src + q * kRows);
      }
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (p0 + i < np) {
#pragma unroll
        for (int q = 0; q < 4; ++q) { v[q].x += a[i][q].x; v[q].y += a[i][q].y; v[q].z += a[i][q].z; v[q].w += a[i][q].w; }
      }
  }
  const float o[16] = {v[0].x, v[0].y, v[0].z, v[0].w, v[1].x, v[1].y, v[1].z, v[1].w,
                       v[2].x, v[2].y, v[2].z, v[2].w, v[3].x, v[3].y, v[3].z, v[3].w};
  store_row(o, y, bias, nt * kRows + r, plan.M, plan.N);
}

#ifdef DFLASH_TC_TRACE
__device__ int g_trace[148 * 32 * 2];
#define TC_TRACE(code, idx) do { if (blockIdx.x < 148 && (threadIdx.x & 31) == 0) { g_trace[(blockIdx.x * 32 + (threadIdx.x >> 5)) * 2] = (code); g_trace[(blockIdx.x * 32 + (threadIdx.x >> 5)) * 2 + 1] = (int)(idx); } } while (0)
#else
#define TC_TRACE(code, idx) do { } while (0)
#endif

template <int NDQ>
struct Roles {
  static_assert(NDQ == 8 || NDQ == 12, "dequant warps");
  static constexpr int kMma = 6;                               // issuing threads: 3 pair classes x 2 groups of the pair
  static constexpr int kEpWarp0 = NDQ, kXWarp0 = NDQ + kEpWarps, kProducerWarp = kXWarp0 + kXWarps;
  static constexpr int kMmaWarp = kProducerWarp + 1;
  static constexpr int kThreads = (kMmaWarp + kMma) * 32;
  static constexpr int kSlots = NDQ / 4;                       // pairs being dequantised at the same time
  static constexpr int kClasses = 3;                           // pair classes of the issuing threads (p mod 3)
  static_assert(kNA % kSlots == 0 && kNA % kClasses == 0, "a ring buffer must belong to one slot and one pair class");
};

template <int NDQ>
__global__ void __launch_bounds__(Roles<NDQ>::kThreads, 1)
qmm_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmS,
              const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmX,
              const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y, float4* __restrict__ pieces,
              unsigned* __restrict__ counters, const __grid_constant__ Plan plan, int* __restrict__ err,
              unsigned long long* __restrict__ stamps) {
  using R = Roles<NDQ>;
  // Optional time stamps (dflash_verify_qmm_set_stamps): 16 words per CTA, [0] / [1] = %globaltimer at entry / exit,
  // [2..10] = this SM's clock at entry, set-up done, first activation tile landed, first stage complete, first operand
  // ready for the MMA, last MMA issued, last accumulators ready, last output written, exit.
  unsigned long long* const stamp = stamps ? stamps + (size_t)blockIdx.x * 16 : nullptr;
  auto mark = [&](int i) { if (stamp) stamp[i] = (unsigned long long)clock64(); };
  if (stamp && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    stamp[0] = t;
    mark(2);
  }
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* stages = smem;
  uint64_t* bars = (uint64_t*)(stages + kStages * kStageBytes);
  uint32_t* tmem_holder = (uint32_t*)(bars + kNumBars);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_full = bar0, bar_empty = bar_full + 8 * kStages, bar_xraw = bar_empty + 8 * kStages;
  const uint32_t bar_aready = bar_xraw + 8 * kStages, bar_afree = bar_aready + 8 * kNA;
  const uint32_t bar_dready = bar_afree + 8 * kNA, bar_dfree = bar_dready + 8;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int bl = (int)blockIdx.x;
  if (bl >= plan.ctas) return;  // before any allocation or barrier
  const int C = plan.C, NT = plan.NT, M = plan.M, N = plan.N;
  const unsigned units = (unsigned)NT * (unsigned)C;
  const unsigned u_begin = (unsigned)bl * units / plan.ctas, u_end = (unsigned)(bl + 1) * units / plan.ctas;
  const unsigned npairs = (u_end - u_begin) * 4u;
  const int nt0 = (int)(u_begin / (unsigned)C), nt1 = (int)((u_end - 1) / (unsigned)C);

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar_full + 8 * i, 1 + kXWarps);      // the TMA bytes and the loader warps' activation tile
      mbar_init(bar_empty + 8 * i, 16 + R::kMma);    // every (pair, 32-row slice) read, every issuing thread's MMAs done
      mbar_init(bar_xraw + 8 * i, 1);                // the activation tile's TMA bytes
    }
    for (int i = 0; i < kNA; ++i) {
      mbar_init(bar_aready + 8 * i, 4);  // the four warps that cover the 128 rows
      mbar_init(bar_afree + 8 * i, 2);   // tcgen05.commit of the two issuing threads that share a pair
    }
    mbar_init(bar_dready, R::kMma);      // one tcgen05.commit per issuing thread
    mbar_init(bar_dfree, kEpWarps);
    mbar_fence_init();
  }
  if (warp == R::kProducerWarp) {
    if (lane == 0) {  // the first TMA request through a tensor map waits for the map itself: fetch all four now
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmW) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmX) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmS) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
    }
    tmem_alloc(smem_u32(tmem_holder), kTmemCols);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_holder;
  if (tid == 0) mark(3);

  if (warp == R::kProducerWarp) {
    // ======================= TMA producer =======================
    // Weights are written by no kernel, so they are requested at once, before the wait on the previous kernel.
    if (lane == 0) {
      const uint64_t pol_stream = l2_policy_evict_first(), pol_keep = l2_policy_evict_last();
      int stage = 0, nt = nt0, kc = (int)(u_begin % (unsigned)C);
      // x is the previous kernel's output, the weights are nobody's: the weights of the first kEarlyUnits units are
      // requested at once, then the previous kernel is waited for, then every unit's activation tile is requested with
      // (right after) its weights.  Requests are served in order, so an activation tile asked for behind the whole ring
      // of weights would land ~3 us late; behind two units it lands as soon as the MMA could use it.
      uint32_t par = 1;
      unsigned xu = u_begin;  // next unit whose activation tile is still owed
      int xstage = 0, xkc = kc;
      auto request_x = [&](unsigned upto) {
        while (xu < upto) {
          const uint32_t xb = bar_xraw + 8 * xstage;
          mbar_arrive_expect_tx(xb, kXTileBytes);
          tma_load_3d(smem_u32(stages + xstage * kStageBytes + kXOff), &tmX, 0, 0, xkc * (kBK / 64), xb, pol_keep);
          if (++xstage == kStages) xstage = 0;
          if (++xkc == C) xkc = 0;
          ++xu;
        }
      };
      bool waited = false;
      for (unsigned u = u_begin; u < u_end; ++u) {
        if (!waited && u - u_begin == (unsigned)kEarlyUnits) {
          pdl_wait();
          waited = true;
          request_x(u);
        }
        if (!mbar_wait_quiet(bar_empty + 8 * stage, par)) { TC_TRACE(11, u - u_begin); atomicCAS(err, 0, 11 | ((int)(u - u_begin) << 8)); break; }
        const uint32_t full = bar_full + 8 * stage, dst = smem_u32(stages + stage * kStageBytes);
        mbar_arrive_expect_tx(full, kTmaBytes);
        tma_load_2d(dst, &tmW, kc * (kBK / 2), nt * kRows, full, pol_stream);
        tma_load_2d(dst + kRows * 128, &tmW, kc * (kBK / 2) + 128, nt * kRows, full, pol_stream);
        tma_load_2d(dst + kWBytes, &tmS, kc * 8, nt * kRows, full, pol_keep);
        tma_load_2d(dst + kWBytes + kSBBytes, &tmB, kc * 8, nt * kRows, full, pol_keep);
        if (++stage == kStages) { stage = 0; par ^= 1; }
        if (++kc == C) { kc = 0; ++nt; }
        if (waited) request_x(u + 1);
      }
      if (!waited) {
        pdl_wait();
        request_x(u_end);
      }
    }
  } else if (warp >= R::kMmaWarp) {
    // ======================= MMA issue =======================
    if (lane == 0) {
      const int me = warp - R::kMmaWarp;
      const int half = me & 1, cls = me >> 1;
      bool aborted = false;
      unsigned ui = 0;  // unit of the current pair, advanced as the pairs go by (no division in the loop)
      int nt = nt0, kc = (int)(u_begin % (unsigned)C), stage = 0;
      unsigned p_lo = 0, p_hi = (min(u_end, (unsigned)(nt + 1) * C) - u_begin) * 4u;  // this row tile's pairs here
      const uint32_t d = tmem + kDCol0 + (uint32_t)me * 16u;
      int ab = cls;          // p mod kNA, advanced with p
      uint32_t apar = 0;     // (p / kNA) & 1
      for (unsigned p = (unsigned)cls; p < npairs; p += R::kClasses) {
        while ((p >> 2) != ui) {
          ++ui;
          if (++stage == kStages) stage = 0;
          if (++kc == C) {
            kc = 0; ++nt;
            p_lo = ui * 4u;
            p_hi = (min(u_end, (unsigned)(nt + 1) * C) - u_begin) * 4u;
          }
        }
        const bool first = p < p_lo + R::kClasses, last = p + R::kClasses >= p_hi;
        const int seg = nt - nt0;
        // the accumulators are not double buffered: the first MMA of a segment waits for the epilogue's read of the last one
        if (first && !aborted && !mbar_wait_quiet(bar_dfree, (uint32_t)(seg & 1) ^ 1u)) { aborted = true; TC_TRACE(13, p); atomicCAS(err, 0, 13 | ((int)p << 8)); }
        // "operand ready" also covers the stage: the dequant warps waited for it to land before they read it
        if (!aborted && !mbar_wait_quiet(bar_aready + 8 * ab, apar)) { aborted = true; TC_TRACE(12, p); atomicCAS(err, 0, 12 | ((int)p << 8)); }
        tc_fence_after();
        if (p == 0 && me == 0) mark(6);
        const uint32_t a = tmem + 64 * ab + 32 * half;
        // group 2q + h of the unit = one 2 KB slab (16 tokens x 128 bytes) of the stage's activation tile
        const uint64_t dg = smem_desc_sw128(smem_u32(stages + stage * kStageBytes + kXOff)) +
                            (uint64_t)((2 * (int)(p & 3u) + half) * 128);
        tc_mma(d, a, dg, kIdesc, first ? 0u : 1u);
        tc_mma(d, a + 8, dg + 2, kIdesc, 1u);
        tc_mma(d, a + 16, dg + 4, kIdesc, 1u);
        tc_mma(d, a + 24, dg + 6, kIdesc, 1u);
        tc_commit(bar_afree + 8 * ab);
        if (((p + R::kClasses) >> 2) != ui) tc_commit(bar_empty + 8 * stage);  // this thread's last pair of the unit
        if (last) tc_commit(bar_dready);
        ab += R::kClasses;
        if (ab >= kNA) { ab -= kNA; apar ^= 1u; }
      }
      if (me == 0) mark(7);
    }
  } else if (warp >= R::kXWarp0) {
    // ======================= activation permuter =======================
    // A unit's 16 x 512 slice of x lands by TMA as 8 slabs of [16 tokens][64 k] with the 128-byte swizzle (the K-major
    // layout the MMA reads); the k order inside every 8-block (one 16-byte chunk, which the swizzle moves as a whole) is
    // then permuted in place to (0,4,1,5,2,6,3,7), the order in which the dequantised pairs come out.  A thread rewrites
    // its own chunks, so nothing is exchanged.
    const int xt = tid - R::kXWarp0 * 32;  // 0..127
    bool aborted = false;
    int stage = 0;
    uint32_t par = 0;
    for (unsigned u = u_begin; u < u_end; ++u) {
      if (!aborted && !mbar_wait_quiet(bar_xraw + 8 * stage, par)) { aborted = true; TC_TRACE(17, u - u_begin); atomicCAS(err, 0, 17 | ((int)(u - u_begin) << 8)); }
      if (xt == 0 && u == u_begin) mark(4);
      uint4* xs = (uint4*)(stages + stage * kStageBytes + kXOff);
      uint4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = xs[xt + 128 * j];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint4 o;
        o.x = prmt(v[j].x, v[j].z, 0x5410); o.y = prmt(v[j].x, v[j].z, 0x7632);
        o.z = prmt(v[j].y, v[j].w, 0x5410); o.w = prmt(v[j].y, v[j].w, 0x7632);
        xs[xt + 128 * j] = o;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor core reads it through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_full + 8 * stage);
      if (++stage == kStages) { stage = 0; par ^= 1; }
    }
  } else if (warp < NDQ) {
    // ======================= dequantisers =======================
    const int r = ((warp & 3) << 5) | lane;  // TMEM lane = weight row inside the tile
    const uint32_t lane_base = (uint32_t)((warp & 3) << 5) << 16;
    bool aborted = false;
    const int slot = warp >> 2;
    int ab = slot;          // p mod kNA, advanced with p
    uint32_t fpar = 1;      // parity of "buffer free" to wait for: the first use of a buffer passes at once
    for (unsigned p = (unsigned)slot; p < npairs; p += R::kSlots) {
      const unsigned ui = p >> 2;
      const int q = (int)(p & 3u);  // pair of the unit: groups 2q, 2q + 1
      const int stage = (int)(ui % (unsigned)kStages);
      const uint32_t par = (ui / (unsigned)kStages) & 1u;
      if (!aborted && !mbar_wait_quiet(bar_full + 8 * stage, par)) { aborted = true; TC_TRACE(15, p); atomicCAS(err, 0, 15 | ((int)p << 8)); }
      if (tid == 0 && p == 0) mark(5);
      const uint8_t* st = stages + stage * kStageBytes;
      const uint32_t sw = *(const uint32_t*)(st + kWBytes + r * 16 + 4 * q);             // scales of groups 2q, 2q+1
      const uint32_t bw = *(const uint32_t*)(st + kWBytes + kSBBytes + r * 16 + 4 * q);  // and their biases
      const uint8_t* wrow = st + (q >> 1) * (kRows * 128) + r * 128;
      const int c0w = 4 * (q & 1);
      uint4 w4[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) w4[c] = *(const uint4*)(wrow + (((c0w + c) ^ (r & 7)) << 4));
      if (!aborted && !mbar_wait_quiet(bar_afree + 8 * ab, fpar)) { aborted = true; TC_TRACE(16, p); atomicCAS(err, 0, 16 | ((int)p << 8)); }
      tc_fence_after();
      const uint32_t a_addr = tmem + lane_base + 64 * ab;
#pragma unroll
      for (int g2 = 0; g2 < 2; ++g2) {
        const float fs = __uint_as_float(g2 ? (sw & 0xFFFF0000u) : (sw << 16));
        const float fb = __uint_as_float(g2 ? (bw & 0xFFFF0000u) : (bw << 16));
        const uint32_t S = bf16x2_dup(fs * kPow2Scale), S16 = bf16x2_dup(fs * kPow2Scale16);
        const uint32_t B = bf16x2_dup(fb * kPow2Bias);
        uint32_t regs[32];
        dequant_group(w4[2 * g2], w4[2 * g2 + 1], S, S16, B, regs);
        tc_st32(a_addr + 32 * g2, regs);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_empty + 8 * stage);  // this warp's words of the stage are in registers
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_aready + 8 * ab);
      ab += R::kSlots;
      if (ab >= kNA) { ab -= kNA; fpar ^= 1u; }
    }
  } else {
    // ======================= epilogue =======================
    const int r = ((warp & 3) << 5) | lane;  // TMEM lane = weight row inside the tile
    const uint32_t lane_base = (uint32_t)((warp & 3) << 5) << 16;
    const int etid = tid - R::kEpWarp0 * 32;  // 0..127
    bool aborted = false;
    pdl_wait();      // these warps write what a later kernel reads and the previous kernel may still read
    pdl_trigger();
    for (int nt = nt0; nt <= nt1; ++nt) {
      const int seg = nt - nt0;
      if (!aborted && !mbar_wait_quiet(bar_dready, (uint32_t)(seg & 1))) { aborted = true; TC_TRACE(14, seg); atomicCAS(err, 0, 14 | (seg << 8)); }
      tc_fence_after();
      if (etid == 0 && nt == nt1) mark(8);
      float out[16];
#pragma unroll
      for (int t = 0; t < 16; ++t) out[t] = 0.f;
#pragma unroll
      for (int i = 0; i < R::kMma; i += 2) {  // fixed order: deterministic
        uint32_t da[16], db[16];
        tc_ld16_issue(tmem + lane_base + kDCol0 + (uint32_t)i * 16u, da);
        tc_ld16_issue(tmem + lane_base + kDCol0 + (uint32_t)(i + 1) * 16u, db);
        tc_ld16_wait(da);
        tc_ld16_wait(db);
#pragma unroll
        for (int t = 0; t < 16; ++t) out[t] += __uint_as_float(da[t]);
#pragma unroll
        for (int t = 0; t < 16; ++t) out[t] += __uint_as_float(db[t]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_dfree);
#pragma unroll
      for (int t = 0; t < 16; ++t) out[t] *= kPow2Out;
      int first_cta = 0;
      const int total = tile_pieces(plan, nt, &first_cta);  // CTAs that share row tile nt
      if (total > 1) {
        // Every warp looks after its own 32 rows: partial tile -> ticket of (tile, slice) -> the warp that takes the
        // last one sums the slice.  No block-wide barrier; the ticket is one acquire-release atomic.
        float4* base = &pieces[((size_t)(bl - first_cta) * NT + nt) * kTileF4 + r];
#pragma unroll
        for (int qd = 0; qd < 4; ++qd)
          base[qd * kRows] = make_float4(out[4 * qd], out[4 * qd + 1], out[4 * qd + 2], out[4 * qd + 3]);
        __syncwarp();  // orders the 32 lanes' stores before lane 0's release
        unsigned t = 0;
        if (lane == 0)
          asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(t) : "l"(&counters[nt * 4 + (warp & 3)]) : "memory");
        t = __shfl_sync(0xffffffffu, t, 0);  // and lane 0's acquire before the other lanes' loads
        if (t == (unsigned)(total - 1)) {
          finalize_slice(plan, pieces, y, bias, nt, total, r);
          if (lane == 0) counters[nt * 4 + (warp & 3)] = 0;  // ready for the next launch
        }
      } else {
        store_row(out, y, bias, nt * kRows + r, M, N);
      }
      if (etid == 0 && nt == nt1) mark(9);
    }
  }

  // every warp ends here: the tensor memory goes back before the CTA exits
  tc_fence_before();
  __syncthreads();
  if (warp == R::kProducerWarp) tmem_dealloc(tmem, kTmemCols);
  if (stamp && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    stamp[1] = t;
    mark(10);
  }
}

// ------------------------------------------------------------------------------------------------------
namespace {

unsigned long long* g_stamps = nullptr;  // dflash_verify_qmm_set_stamps
int g_ndq = 12;  // dequant warps of the launched instantiation (dflash_verify_qmm_set_tc_roles)

bool make_plan(int M, int K, int N, int device, int max_blocks, Plan* p) {
  p->M = M; p->K = K; p->N = N;
  p->C = K / kBK;
  p->NT = (N + kRows - 1) / kRows;
  if (p->NT > kMaxRowTiles || p->C < 1) return false;
  const long long U = (long long)p->NT * p->C;
  long long ctas = max_blocks > 0 ? max_blocks : sm_count(device);
  if (ctas > U) ctas = U;
  if ((U + 1) * ctas >= (1ll << 31)) return false;  // the kernel's span arithmetic is 32-bit
  p->ctas = (int)ctas;
  const long long L = U / ctas;  // fewest units a CTA gets
  long long mp = p->C > 1 ? (p->C - 1 + L - 1) / L + 1 : 1;
  if (mp > ctas) mp = ctas;
  p->maxp = (int)mp;
  return true;
}

size_t counters_bytes() { return (size_t)kMaxRowTiles * 4 * 4; }  // one ticket counter per (row tile, 32-row slice)
size_t plan_workspace(const Plan& p) { return counters_bytes() + (size_t)p.maxp * p.NT * kTileF4 * sizeof(float4); }

struct MapKey {
  const void* p; int a, b, kind;
  bool operator==(const MapKey& o) const { return p == o.p && a == o.a && b == o.b && kind == o.kind; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.p) ^ ((size_t)k.a * 1000003u) ^ ((size_t)k.b * 7919u) ^ (size_t)k.kind;
  }
};
std::mutex g_mu;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

// kind 0: packed weights uint8 [rows, inner bytes], box 128 B x 128 rows, 128B swizzle
// kind 1: scales / biases uint16 [rows, inner], box 8 x 128
// kind 2: activations bf16 [a = M rows, b = K] viewed as [K/64][M][64], box 64 x 16 x 8, 128B swizzle: lands as 8 slabs of
//         [16 tokens][64 k] (rows M..15 of the box lie outside the tensor and are filled with zeros)
bool get_map(const void* ptr, int a, int b, int kind, CUtensorMap* out) {
  MapKey key{ptr, a, b, kind};
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return true; }
  }
  tensormap_encode_fn enc = get_tensormap_encoder();
  if (!enc) return false;
  CUtensorMap m;
  CUresult r;
  cuuint64_t dims[2] = {(cuuint64_t)b, (cuuint64_t)a};
  cuuint32_t es[2] = {1, 1};
  if (kind == 2) {
    cuuint64_t dims3[3] = {64, (cuuint64_t)a, (cuuint64_t)(b / 64)};
    cuuint64_t strides3[2] = {(cuuint64_t)b * 2, 128};
    cuuint32_t box3[3] = {64, 16, (cuuint32_t)(kBK / 64)};
    cuuint32_t es3[3] = {1, 1, 1};
    r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims3, strides3, box3, es3,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else if (kind == 0) {
    cuuint64_t strides[1] = {(cuuint64_t)b};
    cuuint32_t box[2] = {128, (cuuint32_t)kRows};
    r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    cuuint64_t strides[1] = {(cuuint64_t)b * 2};
    cuuint32_t box[2] = {8, (cuuint32_t)kRows};
    r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(ptr), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) return false;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_maps.size() > 16384) g_maps.clear();
  g_maps.emplace(key, m);
  *out = m;
  return true;
}

template <int NDQ>
cudaError_t launch_variant(int grid, cudaStream_t st, int device, const CUtensorMap& tw, const CUtensorMap& ts,
                           const CUtensorMap& tb, const CUtensorMap& tx, const void* bias, void* y, float4* pieces,
                           unsigned* counters, const Plan& plan) {
  auto kern = qmm_tc_kernel<NDQ>;
  static bool attr_done[64] = {};
  if (!attr_done[device & 63]) {
    cudaError_t e0 = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e0 != cudaSuccess) return e0;
    attr_done[device & 63] = true;
  }
  return launch_kernel(kern, dim3(grid), dim3(Roles<NDQ>::kThreads), kSmemBytes, st, tw, ts, tb, tx,
                       (const __nv_bfloat16*)bias, (__nv_bfloat16*)y, pieces, counters, plan,
                       device_error_word(device), g_stamps);
}

}  // namespace

void set_k_parts(int) {}  // this kernel cuts K only where a CTA's span ends
void set_stamps(void* dev) { g_stamps = (unsigned long long*)dev; }
#ifdef DFLASH_TC_TRACE
}  // namespace tc
}  // namespace dflash
extern "C" __attribute__((visibility("default"))) void dflash_tc_trace_dump(void) {
  static int h[148 * 32 * 2];
  cudaMemcpyFromSymbol(h, dflash::tc::g_trace, sizeof(h));
  for (int b = 0; b < 148; ++b) {
    bool any = false;
    for (int w = 0; w < 32; ++w) any |= h[(b * 32 + w) * 2] != 0;
    if (!any) continue;
    printf("cta %3d:", b);
    for (int w = 0; w < 32; ++w) if (h[(b * 32 + w) * 2]) printf(" w%d=(%d,%d)", w, h[(b * 32 + w) * 2], h[(b * 32 + w) * 2 + 1]);
    printf("\n");
  }
  static int z[148 * 32 * 2];
  cudaMemcpyToSymbol(dflash::tc::g_trace, z, sizeof(z));
}
namespace dflash {
namespace tc {
#endif

void set_roles(int dequant_warps, int issuing_threads) {
  if (dequant_warps == 8 || dequant_warps == 12) g_ndq = dequant_warps;
  (void)issuing_threads;  // fixed at 6 (two per pair class)
}

size_t workspace_bytes(int M, int K, int N, int device, int max_blocks) {
  if (K % kBK != 0) return 0;
  Plan p;
  if (!make_plan(M, K, N, device, max_blocks, &p)) return 0;
  return plan_workspace(p);
}

// Returns DFLASH_OK, a negative status, or +1 when this shape is not handled here (the caller then runs qmm.cu).
int launch(const void* x, const void* wq, const void* sc, const void* bi, const void* bias, void* y, int M, int K, int N,
           void* ws, size_t ws_bytes, cudaStream_t st, int device, int max_blocks) {
  if (K % kBK != 0) return 1;
  Plan plan;
  if (!make_plan(M, K, N, device, max_blocks, &plan)) return 1;
  CUtensorMap tw, ts, tb, tx;
  if (!get_map(wq, N, K / 2, 0, &tw) || !get_map(sc, N, K / kG, 1, &ts) || !get_map(bi, N, K / kG, 1, &tb) ||
      !get_map(x, M, K, 2, &tx))
    return 1;
  const size_t need = plan_workspace(plan);
  if (ws == nullptr || ws_bytes < need)
    return fail(DFLASH_ERR_WORKSPACE, "verify_qmm needs %zu workspace bytes, got %zu", need, ws_bytes);
  unsigned* counters = (unsigned*)ws;
  float4* pieces = (float4*)((uint8_t*)ws + counters_bytes());
  const int grid = plan.ctas;
  cudaError_t e;
  if (g_ndq == 12) e = launch_variant<12>(grid, st, device, tw, ts, tb, tx, bias, y, pieces, counters, plan);
  else e = launch_variant<8>(grid, st, device, tw, ts, tb, tx, bias, y, pieces, counters, plan);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "qmm_tc launch: %s", cudaGetErrorString(e));
  return DFLASH_OK;
}

}  // namespace tc
}  // namespace dflash
