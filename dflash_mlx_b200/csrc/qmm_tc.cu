// M<=16 int4 (group 64, bf16) matmul on the 5th-generation tensor cores: tcgen05.mma with the dequantised
// weights as the A operand in TENSOR MEMORY, the activations as the B operand in shared memory and the fp32
// accumulator in tensor memory.  Same contract as qmm_stream_kernel (qmm.cu); replaces the same reference code
// (dflash_mlx/verify_qmm.py:28-331).
//
// A thread owns ONE weight row: it reads 32 bytes of nibbles per quantisation group, turns them into bf16
// (128 + nib) with LOP3 and writes them straight into tensor memory (tcgen05.st); one thread issues the MMAs
// (M = 128 rows, N = 16 tokens, K = 16); the per-group result comes back with tcgen05.ld and is folded into 16 fp32
// registers with the row's scale - a per-thread scalar - as   out += s * acc + (b - 128 s) * sum_{k in group} x[k].
//
// Structure of a CTA (1 per SM, persistent over a span of work units).  The three steps of a PAIR of groups (128 k)
// run in different warps and meet only through mbarriers, with several operand and accumulator buffers in flight, so
// no warp waits for the round trip of its own work.  (Measured on B200: a satisfied mbarrier wait costs ~80 cycles,
// a hand-over ~90, one M128 x N16 x K16 tcgen05.mma ~64 cycles of its issuing thread and ~42 of the tensor pipe -
// hence hand-overs per pair, not per group, and three issuing threads.)
//   warps 0-7   : dequantisers.  Warp w may touch TMEM lanes 32*(w%4)..+31; warps 0-3 take the even pairs of the
//                 sequence, warps 4-7 the odd ones.  wait(operand buffer free) -> LOP3 -> tcgen05.st -> arrive.
//   warps 8-15  : epilogue.  Warps 8-11 own tokens 0-7, warps 12-15 tokens 8-15, of every pair:
//                 wait(accumulators ready) -> tcgen05.ld -> arrive(accumulators free) -> FMAs; a thread ends up with
//                 its row's 8 outputs, so the end of a row tile needs no exchange between warps.
//   warp 16     : TMEM allocation and TMA producer (weights: 128B-swizzled boxes; scales; biases).
//   warps 17-19 : one thread each issues MMAs, pairs dealt round robin: wait(operand ready, accumulators free) ->
//                 8 x tcgen05.mma -> tcgen05.commit to "operand free" and to "accumulators ready".
// Work unit = 128 rows x 8 groups (one 36 KB stage); K slabs, stream-K spans, fp32 partial tiles, batched
// tickets and the deterministic last-arriver reduction are those of qmm.cu.
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace dflash {
namespace tc {

constexpr int kRows = 128;               // weight rows per tile
constexpr int kG = 64;                   // quantisation group
constexpr int kBK = 8 * kG;              // k per stage
constexpr int kDqWarps = 8, kEpWarps = 8;
constexpr int kWorkers = (kDqWarps + kEpWarps) * 32;  // 512: these threads also load the activation slab
constexpr int kEp = kEpWarps * 32;                    // 256
constexpr int kProducerWarp = kDqWarps + kEpWarps, kMmaWarp = kProducerWarp + 1;
constexpr int kMmaWarps = 3;             // one issuing thread each; pairs of groups are dealt to them round robin
constexpr int kThreads = kWorkers + 32 + 32 * kMmaWarps;
constexpr int kTileF4 = 512;             // float4 entries of one fp32 partial tile: [token quad][row]
constexpr int kStages = 4;
constexpr int kWBytes = kRows * (kBK / 2);    // 32 KB
constexpr int kSBBytes = kRows * 16;          // 2 KB
constexpr int kStageBytes = kWBytes + 2 * kSBBytes;
constexpr int kSlabK = 2048;
constexpr int kXBytes = kSlabK * 32;          // [k/8][16 tok][8] bf16
constexpr int kXsBytes = (kSlabK / kG) * 16 * 4;
constexpr int kMaxSlabs = 64;
constexpr int kMaxPend = 32;
constexpr int kMaxRowTiles = 16384;
constexpr int kNP = 4;                   // buffers, one per PAIR of groups of a unit: operand 64 TMEM columns (128 k),
                                         // accumulator 2 x 16 columns
constexpr int kNA = 6, kND = kNP;        // operand buffers: pair p of the span uses p % 6; accumulators: p % 4
constexpr int kNumBars = 2 * kStages + 2 * kNA + 2 * kND;  // full, empty, a_ready, a_free, d_ready, d_free
constexpr size_t kSmemBytes = 1024 + (size_t)kStages * kStageBytes + kXBytes + kXsBytes + 8 * kNumBars +
                              3 * kMaxPend * 4 + 64;
constexpr uint32_t kTmemCols = 512;      // A buffers at columns 0..255, accumulators at 256..383
constexpr uint32_t kDCol0 = 64 * kNA;

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
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
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
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
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
__device__ __forceinline__ void tc_ld8_issue(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tc_ld8_wait(uint32_t (&r)[8]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7])
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

template <typename T>
__device__ __forceinline__ void store_rows(const float4& v, T* __restrict__ y, const T* __restrict__ bias, int n, int set,
                                           int M, int N) {
  if (n >= N) return;
  const float bv = bias ? __bfloat162float(bias[n]) : 0.f;
  const int tok = 4 * set;
  if (tok < M) y[(size_t)tok * N + n] = __float2bfloat16_rn(v.x + bv);
  if (tok + 1 < M) y[(size_t)(tok + 1) * N + n] = __float2bfloat16_rn(v.y + bv);
  if (tok + 2 < M) y[(size_t)(tok + 2) * N + n] = __float2bfloat16_rn(v.z + bv);
  if (tok + 3 < M) y[(size_t)(tok + 3) * N + n] = __float2bfloat16_rn(v.w + bv);
}

// The epilogue threads of the CTA that took the last ticket of row tile nt sum that tile's partial tiles in a fixed
// order; thread (half, r) owns token quads 2*half and 2*half+1 of row r.
__device__ __noinline__ void finalize_tile(const Plan& plan, const float4* pieces, unsigned* counters,
                                           __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ bias, int nt,
                                           int etid, int half, int r) {
  float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
  const int i0 = (2 * half) * kRows + r, i1 = i0 + kRows;
  for (int s2 = 0; s2 < plan.S; ++s2) {
    const SlabGeom g2 = slab_geom(plan, s2);
    int f;
    const int np = tile_pieces(g2, nt, &f);
    for (int p = 0; p < np; ++p) {
      const float4* base = &pieces[((size_t)(s2 * plan.maxp + p) * plan.NT + nt) * kTileF4];
      const float4 a = ld_cg_f4(base + i0), b = ld_cg_f4(base + i1);
      v0.x += a.x; v0.y += a.y; v0.z += a.z; v0.w += a.w;
      v1.x += b.x; v1.y += b.y; v1.z += b.z; v1.w += b.w;
    }
  }
  if (etid == 0) counters[nt] = 0;
  store_rows<__nv_bfloat16>(v0, y, bias, nt * kRows + r, 2 * half, plan.M, plan.N);
  store_rows<__nv_bfloat16>(v1, y, bias, nt * kRows + r, 2 * half + 1, plan.M, plan.N);
}

__global__ void __launch_bounds__(kThreads, 1)
qmm_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmS,
              const __grid_constant__ CUtensorMap tmB, const __nv_bfloat16* __restrict__ x,
              const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y, float4* __restrict__ pieces,
              unsigned* __restrict__ counters, const __grid_constant__ Plan plan, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* stages = smem;
  uint8_t* xbuf = stages + kStages * kStageBytes;
  float* xs = (float*)(xbuf + kXBytes);
  uint64_t* bars = (uint64_t*)((uint8_t*)xs + kXsBytes);
  volatile int* pend = (volatile int*)(bars + kNumBars);
  uint32_t* tmem_holder = (uint32_t*)(pend + 3 * kMaxPend);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_full = bar0, bar_empty = bar_full + 8 * kStages;
  const uint32_t bar_aready = bar_empty + 8 * kStages, bar_afree = bar_aready + 8 * kNA;
  const uint32_t bar_dready = bar_afree + 8 * kNA, bar_dfree = bar_dready + 8 * kND;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;

  int s = 0;
  while (s + 1 < plan.S && (int)blockIdx.x >= plan.slab_cta0[s + 1]) ++s;
  const SlabGeom sg = slab_geom(plan, s);
  const int bl = (int)blockIdx.x - sg.cta0;
  if (bl >= sg.ctas) return;  // before any allocation or barrier
  const unsigned u_begin = (unsigned)bl * sg.units / sg.ctas, u_end = (unsigned)(bl + 1) * sg.units / sg.ctas;
  const int NT = plan.NT, M = plan.M, N = plan.N;

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, kDqWarps + kEpWarps);
    }
    for (int i = 0; i < kNA; ++i) {
      mbar_init(bar_aready + 8 * i, 4);  // the four warps that cover the 128 rows
      mbar_init(bar_afree + 8 * i, 1);   // tcgen05.commit
    }
    for (int i = 0; i < kND; ++i) {
      mbar_init(bar_dready + 8 * i, 1);  // tcgen05.commit
      mbar_init(bar_dfree + 8 * i, kEpWarps);  // both token halves have read the pair's accumulators
    }
    mbar_fence_init();
  }
  if (warp == kProducerWarp) tmem_alloc(smem_u32(tmem_holder), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_holder;

  if (warp == kProducerWarp) {
    // ======================= TMA producer =======================
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
  } else if (warp >= kMmaWarp) {
    // ======================= MMA issue =======================
    named_bar_sync(2, kWorkers + 32 * kMmaWarps);  // the worker warps have written the activation slab
    if (lane == 0) {
      const uint32_t xaddr = smem_u32(xbuf);
      bool aborted = false;
      // Pair p of the span (4 per unit) is handled by issuing thread p % kMmaWarps and uses buffer p % 4; waits
      // and commits are per pair, so a thread pays their latency once per 8 MMAs.
      const unsigned npairs = (u_end - u_begin) * 4u;
      for (unsigned p = (unsigned)(warp - kMmaWarp); p < npairs; p += kMmaWarps) {
        const unsigned ui = p >> 2;
        const int j = (int)(p & 3u);
        const uint32_t upar = ui & 1u;
        const int kc = (int)((u_begin + ui) % (unsigned)sg.cs);
        const int ab = (int)(p % (unsigned)kNA);
        const uint32_t apar = (p / (unsigned)kNA) & 1u;
        if (!aborted && !mbar_wait(bar_aready + 8 * ab, apar)) { aborted = true; atomicExch(err, 12); }
        if (!aborted && !mbar_wait(bar_dfree + 8 * j, upar ^ 1)) { aborted = true; atomicExch(err, 13); }
        tc_fence_after();
#pragma unroll
        for (int g2 = 0; g2 < 2; ++g2) {
          const int gs = kc * 8 + 2 * j + g2;  // group index inside the slab
          const uint32_t d = tmem + kDCol0 + 32 * j + 16 * g2, a = tmem + 64 * ab + 32 * g2;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            tc_mma(d, a + 8 * i, smem_desc(xaddr + (uint32_t)(gs * 8 + 2 * i) * 256u, 256u, 128u), kIdesc, i > 0);
        }
        tc_commit(bar_afree + 8 * ab);
        tc_commit(bar_dready + 8 * j);
      }
    }
  } else {
    // ======================= worker warps: dequantisers (0-7) and epilogue (8-15) =======================
    const int r = ((warp & 3) << 5) | lane;  // TMEM lane = weight row inside the tile
    const uint32_t lane_base = (uint32_t)((warp & 3) << 5) << 16;
    bool aborted = false;
    // The producer warp above requests weights (written by no kernel) at once; the warps here read the previous
    // kernel's output and write this kernel's, so they first wait for the previous kernel of the stream.
    pdl_wait();
    pdl_trigger();
    // Activation slab: read straight from global memory (it is L2 resident), re-tiled to the K-major core-matrix
    // layout [k/8][16 tokens][8] with the k order inside every 8-block permuted to (0,4,1,5,2,6,3,7) - the order in
    // which LOP3 yields nibble pairs.  A warp covers 16 tokens x 2 k-blocks: full 32-byte sectors from global
    // memory, consecutive 16-byte chunks in shared memory.
    {
      const int kb_lim = (plan.K - sg.c0 * kBK) / 8;  // k-blocks that exist from the slab start
      uint4 v[kXBytes / 16 / kWorkers];
#pragma unroll
      for (int j = 0; j < kXBytes / 16 / kWorkers; ++j) {
        const int ci = tid + j * kWorkers, tok = ci & 15, kb = ci >> 4;
        v[j] = make_uint4(0, 0, 0, 0);
        if (tok < M && kb < kb_lim) v[j] = *(const uint4*)(x + (size_t)tok * plan.K + (size_t)sg.c0 * kBK + kb * 8);
      }
#pragma unroll
      for (int j = 0; j < kXBytes / 16 / kWorkers; ++j) {
        uint4 o;
        o.x = prmt(v[j].x, v[j].z, 0x5410); o.y = prmt(v[j].x, v[j].z, 0x7632);
        o.z = prmt(v[j].y, v[j].w, 0x5410); o.w = prmt(v[j].y, v[j].w, 0x7632);
        ((uint4*)xbuf)[tid + j * kWorkers] = o;
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    named_bar_sync(2, kWorkers + 32 * kMmaWarps);  // the slab is complete: the MMA warp may read it
    // group sums of x: thread (g, tok) adds the 64 activations of group g for token tok
    {
      const int g = tid >> 4, tok = tid & 15;
      float acc = 0.f;
#pragma unroll
      for (int kb = 0; kb < 8; ++kb) {
        const uint4 vv = *(const uint4*)(xbuf + ((size_t)(g * 8 + kb) * 16 + tok) * 16);
        const __nv_bfloat162* p = (const __nv_bfloat162*)&vv;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(p[j]);
          acc += f.x + f.y;
        }
      }
      xs[g * 16 + tok] = acc;
    }
    named_bar_sync(1, kWorkers);

    if (warp < kDqWarps) {
      // ----------------------------- dequantisers -----------------------------
      const int ph = warp >> 2;  // 0: even pairs of the sequence, 1: odd pairs
      int stage = 0;
      uint32_t par = 0;
      int ab = ph;         // this warp's pairs use operand buffers ph, ph+2, ph+4, ph, ...
      uint32_t fpar = 1;   // parity to wait for on "operand free" (the first use of a buffer passes at once)
      for (unsigned u = u_begin; u < u_end; ++u) {
        if (!aborted && !mbar_wait(bar_full + 8 * stage, par)) { aborted = true; atomicExch(err, 15); }
        const uint8_t* st = stages + stage * kStageBytes;
        // This warp's two pairs of groups (128 k = 64 bytes of nibbles per row each).
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          const int j = 2 * jj + ph;
          const uint8_t* wrow = st + (j >> 1) * (kRows * 128) + r * 128;
          const int c0 = 4 * (j & 1);
          uint4 w4[4];
#pragma unroll
          for (int c = 0; c < 4; ++c) w4[c] = *(const uint4*)(wrow + (((c0 + c) ^ (r & 7)) << 4));
          if (!aborted && !mbar_wait(bar_afree + 8 * ab, fpar)) { aborted = true; atomicExch(err, 16); }
          tc_fence_after();
          const uint32_t a_addr = tmem + lane_base + 64 * ab;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint32_t words[4] = {w4[c].x, w4[c].y, w4[c].z, w4[c].w};
            uint32_t regs[16];
#pragma unroll
            for (int w = 0; w < 4; ++w)
#pragma unroll
              for (int q = 0; q < 4; ++q)
                regs[4 * w + q] = lop3_and_or(words[w] >> (4 * q), 0x000F000Fu, 0x43004300u);
            tc_st16(a_addr + 16 * c, regs);
          }
          tc_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_aready + 8 * ab);
          ab += 2;
          if (ab >= kNA) { ab -= kNA; fpar ^= 1; }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + 8 * stage);
        if (++stage == kStages) { stage = 0; par ^= 1; }
      }
    } else {
      // ----------------------------- epilogue -----------------------------
      const int half = (warp - kDqWarps) >> 2;  // tokens 8*half .. 8*half+7 of every group
      const int etid = tid - kDqWarps * 32;     // 0..255
      float out[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) out[i] = 0.f;
      int npend = 0;
      auto flush_tickets = [&]() {
        named_bar_sync(3, kEp);
        if (etid == 32) {
          __threadfence();
          for (int i0 = 0; i0 < npend; i0 += 8) {
            unsigned t[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (i0 + j < npend) t[j] = atomicAdd(&counters[pend[i0 + j]], 1u);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (i0 + j < npend) pend[2 * kMaxPend + i0 + j] = (t[j] == (unsigned)(pend[kMaxPend + i0 + j] - 1));
          }
          __threadfence();
        }
        named_bar_sync(3, kEp);
        for (int i = 0; i < npend; ++i)
          if (pend[2 * kMaxPend + i]) finalize_tile(plan, pieces, counters, y, bias, pend[i], etid, half, r);
        named_bar_sync(3, kEp);
      };

      int stage = 0, nt = (int)(u_begin / sg.cs), kc = (int)(u_begin % sg.cs);
      uint32_t par = 0;
      uint32_t upar = 0;  // parity of the unit inside this CTA's span
      for (unsigned u = u_begin; u < u_end; ++u) {
        if (!aborted && !mbar_wait(bar_full + 8 * stage, par)) { aborted = true; atomicExch(err, 17); }
        const uint8_t* st = stages + stage * kStageBytes;
        const uint4 s8 = *(const uint4*)(st + kWBytes + r * 16);             // the row's 8 scales
        const uint4 b8 = *(const uint4*)(st + kWBytes + kSBBytes + r * 16);  // and 8 biases
        const uint32_t sw[4] = {s8.x, s8.y, s8.z, s8.w}, bw[4] = {b8.x, b8.y, b8.z, b8.w};
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + 8 * stage);  // the scales and biases are in registers
        // every pair of groups: this warp takes its 8 token columns of both accumulators
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t dr[2][8];
          if (!aborted && !mbar_wait(bar_dready + 8 * j, upar)) { aborted = true; atomicExch(err, 14); }
          tc_fence_after();
          tc_ld8_issue(tmem + lane_base + kDCol0 + 32 * j + 8 * half, dr[0]);
          tc_ld8_issue(tmem + lane_base + kDCol0 + 32 * j + 16 + 8 * half, dr[1]);
          tc_ld8_wait(dr[0]);
          tc_ld8_wait(dr[1]);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_dfree + 8 * j);
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int gi = 2 * j + q;
            // groups 2j and 2j+1 share word j of the row's scales: low and high bf16
            const float sc = __uint_as_float(q ? (sw[j] & 0xFFFF0000u) : (sw[j] << 16));
            const float bi = __uint_as_float(q ? (bw[j] & 0xFFFF0000u) : (bw[j] << 16));
            const float bq = fmaf(-128.f, sc, bi);
            const float4* xr = (const float4*)(xs + (kc * 8 + gi) * 16 + 8 * half);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const float4 xv = xr[i];
              out[4 * i + 0] = fmaf(sc, __uint_as_float(dr[q][4 * i + 0]), fmaf(bq, xv.x, out[4 * i + 0]));
              out[4 * i + 1] = fmaf(sc, __uint_as_float(dr[q][4 * i + 1]), fmaf(bq, xv.y, out[4 * i + 1]));
              out[4 * i + 2] = fmaf(sc, __uint_as_float(dr[q][4 * i + 2]), fmaf(bq, xv.z, out[4 * i + 2]));
              out[4 * i + 3] = fmaf(sc, __uint_as_float(dr[q][4 * i + 3]), fmaf(bq, xv.w, out[4 * i + 3]));
            }
          }
        }
        upar ^= 1;
        if (++stage == kStages) { stage = 0; par ^= 1; }

        const bool seg_end = (kc == sg.cs - 1) || (u == u_end - 1);
        if (seg_end) {
          // thread (half, r) holds row r of the tile for token quads 2*half and 2*half+1: nothing to exchange
          const float4 v0 = make_float4(out[0], out[1], out[2], out[3]), v1 = make_float4(out[4], out[5], out[6], out[7]);
#pragma unroll
          for (int i = 0; i < 8; ++i) out[i] = 0.f;
          int total = 0, first_here = 0;
          for (int sl = lane; sl < plan.S; sl += 32) {
            const SlabGeom g2 = slab_geom(plan, sl);
            int f;
            total += tile_pieces(g2, nt, &f);
          }
          total = __reduce_add_sync(0xffffffffu, total);
          tile_pieces(sg, nt, &first_here);
          if (total > 1) {
            float4* base = &pieces[((size_t)(s * plan.maxp + (bl - first_here)) * NT + nt) * kTileF4];
            base[(2 * half) * kRows + r] = v0;
            base[(2 * half + 1) * kRows + r] = v1;
            if (etid == 0) { pend[npend] = nt; pend[kMaxPend + npend] = total; }
            ++npend;
          } else {
            store_rows<__nv_bfloat16>(v0, y, bias, nt * kRows + r, 2 * half, M, N);
            store_rows<__nv_bfloat16>(v1, y, bias, nt * kRows + r, 2 * half + 1, M, N);
          }
          if (npend == kMaxPend) { flush_tickets(); npend = 0; }
        }
        if (++kc == sg.cs) { kc = 0; ++nt; }
      }
      if (npend > 0) flush_tickets();
    }
  }

  // every warp ends here: the accumulator memory goes back before the CTA exits
  tc_fence_before();
  __syncthreads();
  if (warp == kProducerWarp) tmem_dealloc(tmem, kTmemCols);
}

// ------------------------------------------------------------------------------------------------------
namespace {

bool make_plan(int M, int K, int N, int device, int max_blocks, Plan* p) {
  const int C = K / kBK, csmax = kSlabK / kBK;
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
// kind 2: activations bf16 viewed as [K/8][M][8] (a = M, b = K), box 8 x 16 x 256: lands as [k/8][16 tokens][8]
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
  if (kind == 2) {
    cuuint64_t dims[3] = {8, (cuuint64_t)a, (cuuint64_t)(b / 8)};
    cuuint64_t strides[2] = {(cuuint64_t)b * 2, 16};
    cuuint32_t box[3] = {8, 16, (cuuint32_t)(kSlabK / 8)};
    cuuint32_t es[3] = {1, 1, 1};
    r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
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
  }
  if (r != CUDA_SUCCESS) return false;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_maps.size() > 16384) g_maps.clear();
  g_maps.emplace(key, m);
  *out = m;
  return true;
}

}  // namespace

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
  static bool attr_done[64] = {};
  if (!attr_done[device & 63]) {
    cudaError_t e0 = cudaFuncSetAttribute(qmm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e0 != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "cudaFuncSetAttribute(qmm_tc): %s", cudaGetErrorString(e0));
    attr_done[device & 63] = true;
  }
  unsigned* counters = (unsigned*)ws;
  float4* pieces = (float4*)((uint8_t*)ws + counters_bytes());
  cudaError_t e = launch_kernel(qmm_tc_kernel, dim3(plan.slab_cta0[plan.S]), dim3(kThreads), kSmemBytes, st, tw, ts, tb,
                                (const __nv_bfloat16*)x, (const __nv_bfloat16*)bias, (__nv_bfloat16*)y, pieces, counters,
                                plan, device_error_word(device));
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "qmm_tc launch: %s", cudaGetErrorString(e));
  return DFLASH_OK;
}

}  // namespace tc
}  // namespace dflash
