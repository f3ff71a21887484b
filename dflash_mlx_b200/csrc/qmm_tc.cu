// M<=16 int4 (group 64, bf16) matmul on the 5th-generation tensor cores: tcgen05.mma with the dequantised
// weights as the A operand in TENSOR MEMORY, the activations as the B operand in shared memory and the fp32
// accumulator in tensor memory.  Same contract as qmm_stream_kernel (qmm.cu); replaces the same reference code
// (dflash_mlx/verify_qmm.py:28-331).
//
// Numerics are the reference's own: every weight is dequantised to bf16, w_hat = bf16(nib * scale + bias)
// (verify_qmm.py:75), and the tensor core accumulates x . w_hat over the whole K slab in fp32.
//
// Dequantisation costs 9 instructions per 8 weights and is exact.  A 16-bit pattern 0x00vv (v < 256) read as bf16 is
// the number v * 2^-133 (the subnormals and the first binade share one spacing), so for a packed word w
//     w & 0x000F000F        = the bf16 pair (nib0, nib4) * 2^-133
//     w & 0x00F000F0        = the pair (nib1, nib5) * 16 * 2^-133
//     (w >> 8) & ...        = the pairs (nib2, nib6) and (nib3, nib7) likewise
// and ONE fma.rn.bf16x2 per pair with the group's pre-scaled constants (scale * 2^101 or scale * 2^97, bias * 2^-32)
// gives bf16(nib * scale + bias) * 2^-32 with a single rounding; the power of two comes off in the epilogue.
// (Scales must be below 2^26 in magnitude; weights below 2^-94 lose precision - neither occurs in a quantised model.)
// The pairs come out in the k order (0,4,1,5,2,6,3,7) inside every 8-block; the activation slab is stored in shared
// memory in the same order, so nothing is shuffled.
//
// Structure of a CTA (1 per SM, persistent over a span of work units; unit = 128 weight rows x 8 groups = one 36 KB
// TMA stage).  Roles meet only through mbarriers:
//   dequant warps  : a thread owns ONE weight row (its TMEM lane).  Per PAIR of groups (128 k): wait(operand buffer
//                    free) -> 4 x LDS.128 -> AND/FMA -> 2 x tcgen05.st (32 columns each) -> arrive(operand ready).
//   issuing threads: NMMA warps with one issuing thread each; pairs are dealt round robin and every issuing thread
//                    accumulates into its OWN 16 columns (MMAs of different threads are not ordered against each
//                    other), over all pairs of a (row tile, K slab) segment: wait(operand ready) -> 8 x tcgen05.mma
//                    M128 x N16 x K16 -> tcgen05.commit(operand free); after its last pair of the segment
//                    tcgen05.commit(accumulators ready).
//   epilogue warps : once per segment: wait(accumulators ready) -> tcgen05.ld of the NMMA accumulators -> sum ->
//                    arrive(accumulators free; they are double buffered) -> store y, or write an fp32 partial tile,
//                    take the tile's ticket and, if it was the last one, sum the tile's partial tiles in a fixed order.
//   producer warp  : TMEM allocation; TMA loads (weights: 128B-swizzled boxes; scales; biases), 3 stages.
// K is cut into slabs of <= 3072 columns; a CTA works inside one slab, whose 16 x slabK activations it keeps in shared
// memory as the K-major core-matrix tiles the MMA reads.  Units of a slab are dealt to its CTAs as equal contiguous
// spans (stream-K).  Every wait is bounded and reports through the device error word.
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace dflash {
namespace tc {

constexpr int kRows = 128;               // weight rows per tile
constexpr int kG = 64;                   // quantisation group
constexpr int kBK = 8 * kG;              // k per stage
constexpr int kEpWarps = 4;
constexpr int kEp = kEpWarps * 32;
constexpr int kTileF4 = 512;             // float4 entries of one fp32 partial tile: [token quad][row]
constexpr int kStages = 3;
constexpr int kWBytes = kRows * (kBK / 2);    // 32 KB
constexpr int kSBBytes = kRows * 16;          // 2 KB
constexpr int kStageBytes = kWBytes + 2 * kSBBytes;
constexpr int kSlabUnits = 6;
constexpr int kSlabK = kSlabUnits * kBK;      // 3072
constexpr int kXBytes = kSlabK * 32;          // [k/8][16 tok][8] bf16
constexpr int kMaxSlabs = 64;
constexpr int kMaxRowTiles = 16384;
constexpr int kNA = 6;                   // operand buffers of 64 TMEM columns (one pair of groups each)
constexpr int kMaxMma = 4;
constexpr int kNumBars = 2 * kStages + 2 * kNA + 4;  // full, empty, a_ready, a_free, d_ready[2], d_free[2]
constexpr size_t kSmemBytes = 1024 + (size_t)kStages * kStageBytes + kXBytes + 8 * kNumBars + 64;
constexpr uint32_t kTmemCols = 512;      // operand buffers at columns 0..383, accumulators at 384..511
constexpr uint32_t kDCol0 = 64 * kNA;
constexpr float kPow2Scale = 0x1p101f;   // 2^(133 - 32)
constexpr float kPow2Scale16 = 0x1p97f;  // the same for a nibble that sits 4 bits higher
constexpr float kPow2Bias = 0x1p-32f;
constexpr float kPow2Out = 0x1p32f;

struct Plan {
  int M, K, N, NT, S, maxp;
  int slab_chunk0[kMaxSlabs + 1];
  int slab_cta0[kMaxSlabs + 1];
};

__device__ __forceinline__ int cta_of(unsigned u, unsigned units, unsigned ctas) {
  return (int)(((u + 1u) * ctas - 1u) / units);
}
struct SlabGeom {
  int c0, cs, cta0, ctas;
  unsigned units;
};
__device__ __forceinline__ SlabGeom slab_geom(const Plan& p, int s) {
  SlabGeom g;
  g.c0 = p.slab_chunk0[s];
  g.cs = p.slab_chunk0[s + 1] - g.c0;
  g.cta0 = p.slab_cta0[s];
  g.units = (unsigned)p.NT * (unsigned)g.cs;
  const unsigned ctas = (unsigned)(p.slab_cta0[s + 1] - g.cta0);
  g.ctas = (int)(ctas < g.units ? ctas : g.units);
  return g;
}
__device__ __forceinline__ int tile_pieces(const SlabGeom& g, int nt, int* first) {
  const int a = cta_of((unsigned)nt * g.cs, g.units, g.ctas);
  const int b = cta_of((unsigned)(nt + 1) * g.cs - 1u, g.units, g.ctas);
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

// The epilogue threads of the CTA that took the last ticket of row tile nt sum that tile's partial tiles in a fixed
// order (slab-major, then piece index); thread r owns row r of the tile.
__device__ __noinline__ void finalize_tile(const Plan& plan, const float4* pieces, unsigned* counters,
                                           __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ bias, int nt,
                                           int r) {
  float4 v[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) v[q] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s2 = 0; s2 < plan.S; ++s2) {
    const SlabGeom g2 = slab_geom(plan, s2);
    int f;
    const int np = tile_pieces(g2, nt, &f);
    for (int p = 0; p < np; ++p) {
      const float4* base = &pieces[((size_t)(s2 * plan.maxp + p) * plan.NT + nt) * kTileF4 + r];
      float4 a[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) a[q] = ld_cg_f4(base + q * kRows);
#pragma unroll
      for (int q = 0; q < 4; ++q) { v[q].x += a[q].x; v[q].y += a[q].y; v[q].z += a[q].z; v[q].w += a[q].w; }
    }
  }
  if (r == 0) counters[nt] = 0;
  const float o[16] = {v[0].x, v[0].y, v[0].z, v[0].w, v[1].x, v[1].y, v[1].z, v[1].w,
                       v[2].x, v[2].y, v[2].z, v[2].w, v[3].x, v[3].y, v[3].z, v[3].w};
  store_row(o, y, bias, nt * kRows + r, plan.M, plan.N);
}

template <int NDQ, int NMMA>
struct Roles {
  static constexpr int kWorkers = (NDQ + kEpWarps) * 32;      // these threads also load the activation slab
  static constexpr int kProducerWarp = NDQ + kEpWarps;
  static constexpr int kMmaWarp = kProducerWarp + 1;
  static constexpr int kThreads = kWorkers + 32 + 32 * NMMA;
  static constexpr int kPairSlots = NDQ / 4;                  // pairs of groups being dequantised at the same time
};

template <int NDQ, int NMMA>
__global__ void __launch_bounds__(Roles<NDQ, NMMA>::kThreads, 1)
qmm_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmS,
              const __grid_constant__ CUtensorMap tmB, const __nv_bfloat16* __restrict__ x,
              const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y, float4* __restrict__ pieces,
              unsigned* __restrict__ counters, const __grid_constant__ Plan plan, int* __restrict__ err) {
  using R = Roles<NDQ, NMMA>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* stages = smem;
  uint8_t* xbuf = stages + kStages * kStageBytes;
  uint64_t* bars = (uint64_t*)(xbuf + kXBytes);
  uint32_t* tmem_holder = (uint32_t*)(bars + kNumBars);
  volatile int* flags = (volatile int*)(tmem_holder + 1);  // [2]: "this CTA took the last ticket", double buffered
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_full = bar0, bar_empty = bar_full + 8 * kStages;
  const uint32_t bar_aready = bar_empty + 8 * kStages, bar_afree = bar_aready + 8 * kNA;
  const uint32_t bar_dready = bar_afree + 8 * kNA, bar_dfree = bar_dready + 8 * 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;

  int s = 0;
  while (s + 1 < plan.S && (int)blockIdx.x >= plan.slab_cta0[s + 1]) ++s;
  const SlabGeom sg = slab_geom(plan, s);
  const int bl = (int)blockIdx.x - sg.cta0;
  if (bl >= sg.ctas) return;  // before any allocation or barrier
  const unsigned u_begin = (unsigned)bl * sg.units / sg.ctas, u_end = (unsigned)(bl + 1) * sg.units / sg.ctas;
  const unsigned npairs = (u_end - u_begin) * 4u;
  const int NT = plan.NT, M = plan.M, N = plan.N;

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, 16);  // every (pair of groups, 32-row slice) of the unit has been read
    }
    for (int i = 0; i < kNA; ++i) {
      mbar_init(bar_aready + 8 * i, 4);  // the four warps that cover the 128 rows
      mbar_init(bar_afree + 8 * i, 1);   // tcgen05.commit
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_dready + 8 * i, NMMA);     // one tcgen05.commit per issuing thread
      mbar_init(bar_dfree + 8 * i, kEpWarps);
    }
    mbar_fence_init();
  }
  if (warp == R::kProducerWarp) tmem_alloc(smem_u32(tmem_holder), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_holder;

  if (warp == R::kProducerWarp) {
    // ======================= TMA producer =======================
    // Weights are written by no kernel, so they are requested at once, before the wait on the previous kernel.
    if (lane == 0) {
      const uint64_t pol_stream = l2_policy_evict_first(), pol_keep = l2_policy_evict_last();
      int stage = 0, nt = (int)(u_begin / sg.cs), kc = (int)(u_begin % sg.cs);
      uint32_t par = 1;
      for (unsigned u = u_begin; u < u_end; ++u) {
        if (!mbar_wait(bar_empty + 8 * stage, par)) { atomicExch(err, 11); break; }
        const uint32_t full = bar_full + 8 * stage, dst = smem_u32(stages + stage * kStageBytes);
        mbar_arrive_expect_tx(full, kStageBytes);
        tma_load_2d(dst, &tmW, (sg.c0 + kc) * (kBK / 2), nt * kRows, full, pol_stream);
        tma_load_2d(dst + kRows * 128, &tmW, (sg.c0 + kc) * (kBK / 2) + 128, nt * kRows, full, pol_stream);
        tma_load_2d(dst + kWBytes, &tmS, (sg.c0 + kc) * 8, nt * kRows, full, pol_keep);
        tma_load_2d(dst + kWBytes + kSBBytes, &tmB, (sg.c0 + kc) * 8, nt * kRows, full, pol_keep);
        if (++stage == kStages) { stage = 0; par ^= 1; }
        if (++kc == sg.cs) { kc = 0; ++nt; }
      }
    }
  } else if (warp >= R::kMmaWarp) {
    // ======================= MMA issue =======================
    named_bar_sync(2, R::kWorkers + 32 * NMMA);  // the worker warps have written the activation slab
    if (lane == 0) {
      const int me = warp - R::kMmaWarp;
      const uint64_t desc0 = smem_desc(smem_u32(xbuf), 256u, 128u);
      bool aborted = false;
      const int nt0 = (int)(u_begin / sg.cs);
      for (unsigned p = (unsigned)me; p < npairs; p += NMMA) {
        const unsigned ui = p >> 2;
        const int q = (int)(p & 3u);
        const unsigned u = u_begin + ui;
        const int nt = (int)(u / (unsigned)sg.cs), kc = (int)(u - (unsigned)nt * sg.cs);
        // the segment (this CTA's units of row tile nt) as a range of pairs
        const unsigned seg_u0 = max(u_begin, (unsigned)nt * sg.cs), seg_u1 = min(u_end, (unsigned)(nt + 1) * sg.cs);
        const unsigned p_lo = (seg_u0 - u_begin) * 4u, p_hi = (seg_u1 - u_begin) * 4u;
        const bool first = p < p_lo + NMMA, last = p + NMMA >= p_hi;
        const int seg = nt - nt0, tp = seg & 1;
        const int ab = (int)(p % (unsigned)kNA);
        const uint32_t apar = (p / (unsigned)kNA) & 1u;
        if (first && !aborted && !mbar_wait(bar_dfree + 8 * tp, ((seg >> 1) & 1) ^ 1)) { aborted = true; atomicExch(err, 13); }
        if (!aborted && !mbar_wait(bar_aready + 8 * ab, apar)) { aborted = true; atomicExch(err, 12); }
        tc_fence_after();
        const uint32_t d = tmem + kDCol0 + (uint32_t)(tp * NMMA + me) * 16u;
#pragma unroll
        for (int g2 = 0; g2 < 2; ++g2) {
          const int gs = kc * 8 + 2 * q + g2;  // group index inside the slab
          const uint32_t a = tmem + 64 * ab + 32 * g2;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            tc_mma(d, a + 8 * i, desc0 + (uint64_t)((gs * 8 + 2 * i) * 16), kIdesc, (first && g2 == 0 && i == 0) ? 0u : 1u);
        }
        tc_commit(bar_afree + 8 * ab);
        if (last) tc_commit(bar_dready + 8 * tp);
      }
    }
  } else {
    // ======================= worker warps: dequantisers and epilogue =======================
    const int r = ((warp & 3) << 5) | lane;  // TMEM lane = weight row inside the tile
    const uint32_t lane_base = (uint32_t)((warp & 3) << 5) << 16;
    bool aborted = false;
    // These warps read the previous kernel's output (x) and write this kernel's: wait for the previous kernel.
    pdl_wait();
    pdl_trigger();
    // Activation slab: read straight from global memory (it is L2 resident), re-tiled to the K-major core-matrix
    // layout [k/8][16 tokens][8] with the k order inside every 8-block permuted to (0,4,1,5,2,6,3,7).  A warp covers
    // 16 tokens x 2 k-blocks: full 32-byte sectors from global memory, consecutive 16-byte chunks in shared memory.
    {
      const int nchunks = sg.cs * (kBK / 8) * 16;
      const __nv_bfloat16* xs0 = x + (size_t)sg.c0 * kBK;
      for (int c0 = tid; c0 < nchunks; c0 += 4 * R::kWorkers) {
        uint4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int ci = c0 + j * R::kWorkers, tok = ci & 15, kb = ci >> 4;
          v[j] = make_uint4(0, 0, 0, 0);
          if (ci < nchunks && tok < M) v[j] = *(const uint4*)(xs0 + (size_t)tok * plan.K + kb * 8);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int ci = c0 + j * R::kWorkers;
          uint4 o;
          o.x = prmt(v[j].x, v[j].z, 0x5410); o.y = prmt(v[j].x, v[j].z, 0x7632);
          o.z = prmt(v[j].y, v[j].w, 0x5410); o.w = prmt(v[j].y, v[j].w, 0x7632);
          if (ci < nchunks) ((uint4*)xbuf)[ci] = o;
        }
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("bar.arrive 2, %0;" ::"r"(R::kWorkers + 32 * NMMA) : "memory");  // the issuing threads wait on it

    if (warp < NDQ) {
      // ----------------------------- dequantisers -----------------------------
      const int slot = warp >> 2;
      for (unsigned p = (unsigned)slot; p < npairs; p += R::kPairSlots) {
        const unsigned ui = p >> 2;
        const int q = (int)(p & 3u);
        const int stage = (int)(ui % (unsigned)kStages);
        const uint32_t par = (ui / (unsigned)kStages) & 1u;
        const int ab = (int)(p % (unsigned)kNA);
        const uint32_t fpar = ((p / (unsigned)kNA) & 1u) ^ 1u;  // the first use of a buffer passes at once
        if (!aborted && !mbar_wait(bar_full + 8 * stage, par)) { aborted = true; atomicExch(err, 15); }
        const uint8_t* st = stages + stage * kStageBytes;
        const uint32_t sw = *(const uint32_t*)(st + kWBytes + r * 16 + 4 * q);             // scales of groups 2q, 2q+1
        const uint32_t bw = *(const uint32_t*)(st + kWBytes + kSBBytes + r * 16 + 4 * q);  // and their biases
        const uint8_t* wrow = st + (q >> 1) * (kRows * 128) + r * 128;
        const int c0 = 4 * (q & 1);
        uint4 w4[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) w4[c] = *(const uint4*)(wrow + (((c0 + c) ^ (r & 7)) << 4));
        if (!aborted && !mbar_wait(bar_afree + 8 * ab, fpar)) { aborted = true; atomicExch(err, 16); }
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
      }
    } else {
      // ----------------------------- epilogue -----------------------------
      const int etid = tid - NDQ * 32;  // 0..127 = row
      const int nt0 = (int)(u_begin / sg.cs), nt1 = (int)((u_end - 1) / sg.cs);
      for (int nt = nt0; nt <= nt1; ++nt) {
        const int seg = nt - nt0, tp = seg & 1;
        if (!aborted && !mbar_wait(bar_dready + 8 * tp, (seg >> 1) & 1)) { aborted = true; atomicExch(err, 14); }
        tc_fence_after();
        float out[16];
#pragma unroll
        for (int t = 0; t < 16; ++t) out[t] = 0.f;
#pragma unroll
        for (int i = 0; i < NMMA; ++i) {  // fixed order: deterministic
          uint32_t dr[16];
          tc_ld16_issue(tmem + lane_base + kDCol0 + (uint32_t)(tp * NMMA + i) * 16u, dr);
          tc_ld16_wait(dr);
#pragma unroll
          for (int t = 0; t < 16; ++t) out[t] += __uint_as_float(dr[t]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_dfree + 8 * tp);
#pragma unroll
        for (int t = 0; t < 16; ++t) out[t] *= kPow2Out;
        // how many partial tiles make up row tile nt, over all K slabs
        int total = 0, first_here = 0;
        for (int sl = lane; sl < plan.S; sl += 32) {
          const SlabGeom g2 = slab_geom(plan, sl);
          int f;
          total += tile_pieces(g2, nt, &f);
        }
        total = __reduce_add_sync(0xffffffffu, total);
        tile_pieces(sg, nt, &first_here);
        if (total > 1) {
          float4* base = &pieces[((size_t)(s * plan.maxp + (bl - first_here)) * NT + nt) * kTileF4 + r];
#pragma unroll
          for (int qd = 0; qd < 4; ++qd)
            base[qd * kRows] = make_float4(out[4 * qd], out[4 * qd + 1], out[4 * qd + 2], out[4 * qd + 3]);
          named_bar_sync(3, kEp);
          if (etid == 0) {
            __threadfence();
            const unsigned t = atomicAdd(&counters[nt], 1u);
            __threadfence();
            flags[seg & 1] = (t == (unsigned)(total - 1)) ? 1 : 0;
          }
          named_bar_sync(3, kEp);
          if (flags[seg & 1]) finalize_tile(plan, pieces, counters, y, bias, nt, r);
        } else {
          store_row(out, y, bias, nt * kRows + r, M, N);
        }
      }
    }
  }

  // every warp ends here: the tensor memory goes back before the CTA exits
  tc_fence_before();
  __syncthreads();
  if (warp == R::kProducerWarp) tmem_dealloc(tmem, kTmemCols);
}

// ------------------------------------------------------------------------------------------------------
namespace {

int g_ndq = 16, g_nmma = 3;  // role counts of the launched instantiation (dflash_verify_qmm_set_tc_roles)

bool make_plan(int M, int K, int N, int device, int max_blocks, Plan* p) {
  const int C = K / kBK, csmax = kSlabUnits;
  p->M = M; p->K = K; p->N = N;
  p->NT = (N + kRows - 1) / kRows;
  p->S = (C + csmax - 1) / csmax;
  if (p->S > kMaxSlabs || p->NT > kMaxRowTiles) return false;
  for (int i = 0; i <= p->S; ++i) p->slab_chunk0[i] = (int)((long long)i * C / p->S);
  const long long U = (long long)p->NT * C;
  long long grid = max_blocks > 0 ? max_blocks : sm_count(device);
  if (grid > U) grid = U;
  if (grid < p->S) grid = p->S;
  for (int i = 0; i <= p->S; ++i) p->slab_cta0[i] = (int)(grid * p->slab_chunk0[i] / C);
  for (int i = 1; i <= p->S; ++i)
    if (p->slab_cta0[i] < p->slab_cta0[i - 1] + 1) p->slab_cta0[i] = p->slab_cta0[i - 1] + 1;
  p->slab_cta0[p->S] = (int)grid;
  for (int i = p->S - 1; i >= 1; --i)
    if (p->slab_cta0[i] > p->slab_cta0[i + 1] - 1) p->slab_cta0[i] = p->slab_cta0[i + 1] - 1;
  int maxp = 1;
  for (int i = 0; i < p->S; ++i) {
    const int cs = p->slab_chunk0[i + 1] - p->slab_chunk0[i];
    const long long Us = (long long)p->NT * cs;
    long long ctas = p->slab_cta0[i + 1] - p->slab_cta0[i];
    if (ctas > Us) ctas = Us;
    const long long L = Us / ctas;
    const int mp = (int)((cs - 1 + L - 1) / L) + 1;
    if (cs > 1 && mp > maxp) maxp = mp;
    if ((Us + 1) * (p->slab_cta0[i + 1] - p->slab_cta0[i]) >= (1ll << 31)) return false;
  }
  p->maxp = maxp;
  return true;
}

size_t counters_bytes() { return (size_t)kMaxRowTiles * 4; }
size_t plan_workspace(const Plan& p) { return counters_bytes() + (size_t)p.S * p.maxp * p.NT * kTileF4 * sizeof(float4); }

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
  if (kind == 0) {
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

template <int NDQ, int NMMA>
cudaError_t launch_variant(int grid, cudaStream_t st, int device, const CUtensorMap& tw, const CUtensorMap& ts,
                           const CUtensorMap& tb, const void* x, const void* bias, void* y, float4* pieces,
                           unsigned* counters, const Plan& plan) {
  auto kern = qmm_tc_kernel<NDQ, NMMA>;
  static bool attr_done[64] = {};
  if (!attr_done[device & 63]) {
    cudaError_t e0 = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e0 != cudaSuccess) return e0;
    attr_done[device & 63] = true;
  }
  return launch_kernel(kern, dim3(grid), dim3(Roles<NDQ, NMMA>::kThreads), kSmemBytes, st, tw, ts, tb,
                       (const __nv_bfloat16*)x, (const __nv_bfloat16*)bias, (__nv_bfloat16*)y, pieces, counters, plan,
                       device_error_word(device));
}

}  // namespace

void set_roles(int dequant_warps, int issuing_threads) {
  if (dequant_warps == 8 || dequant_warps == 12 || dequant_warps == 16) g_ndq = dequant_warps;
  if (issuing_threads >= 2 && issuing_threads <= 4) g_nmma = issuing_threads;
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
  CUtensorMap tw, ts, tb;
  if (!get_map(wq, N, K / 2, 0, &tw) || !get_map(sc, N, K / kG, 1, &ts) || !get_map(bi, N, K / kG, 1, &tb)) return 1;
  const size_t need = plan_workspace(plan);
  if (ws == nullptr || ws_bytes < need)
    return fail(DFLASH_ERR_WORKSPACE, "verify_qmm needs %zu workspace bytes, got %zu", need, ws_bytes);
  unsigned* counters = (unsigned*)ws;
  float4* pieces = (float4*)((uint8_t*)ws + counters_bytes());
  const int grid = plan.slab_cta0[plan.S];
  cudaError_t e;
#define DFLASH_TC_CASE(D, I) \
  if (g_ndq == D && g_nmma == I) e = launch_variant<D, I>(grid, st, device, tw, ts, tb, x, bias, y, pieces, counters, plan); else
  DFLASH_TC_CASE(16, 3) DFLASH_TC_CASE(16, 2) DFLASH_TC_CASE(16, 4) DFLASH_TC_CASE(12, 3) DFLASH_TC_CASE(12, 2)
  DFLASH_TC_CASE(12, 4) DFLASH_TC_CASE(8, 3) DFLASH_TC_CASE(8, 2) DFLASH_TC_CASE(8, 4)
  e = cudaErrorInvalidValue;
#undef DFLASH_TC_CASE
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "qmm_tc launch: %s", cudaGetErrorString(e));
  return DFLASH_OK;
}

}  // namespace tc
}  // namespace dflash
