// M<=16 int4 (group 64, bf16) matmul on the 5th-generation tensor cores: tcgen05.mma with the dequantised
// weights as the A operand in TENSOR MEMORY, the activations as the B operand in shared memory and the fp32
// accumulator in tensor memory.  Same contract as qmm_stream_kernel (qmm.cu); replaces the same reference code
// (dflash_mlx/verify_qmm.py:28-331).
//
// Why: the mma.sync kernel spends ~54 warp instructions per 512 weights (fragment shuffling, per-fragment
// scale FMAs, MMA issue by every warp).  Here a thread owns ONE weight row: it reads 32 bytes of nibbles per
// quantisation group, turns them into bf16 (128 + nib) with LOP3 and writes them straight into tensor memory
// (tcgen05.st); one elected thread issues the MMAs (M = 128 rows, N = 16 tokens, K = 16); the per-group
// result comes back with tcgen05.ld and is folded into 16 fp32 registers with the row's scale - a per-thread
// scalar - as   out += s * acc + (b - 128 s) * sum_{k in group} x[k].
//
// Structure of a CTA (1 per SM, persistent over a span of work units):
//   warps 0-15  : 4 sets x 4 warps.  Warp w may touch TMEM lanes 32*(w%4)..+31, so a set covers the 128 rows;
//                 set j handles quantisation groups 2j and 2j+1 of every stage.
//   warp 16     : TMEM allocation and TMA producer (weights: 128B-swizzled boxes; scales, biases; activation slab
//                 as a 3-D map that lands directly in the K-major core-matrix layout the MMA wants).
//   MMA issue   : no dedicated warp.  When a set has finished writing a group's operand, the LAST of its four warps
//                 to get there (a shared-memory ticket) issues that group's four MMAs and the commit, so nothing
//                 waits for a polling thread.
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
constexpr int kSets = 4;
constexpr int kDequantWarps = 16;
constexpr int kDequant = kDequantWarps * 32;  // 512
constexpr int kThreads = kDequant + 32;
constexpr int kStages = 3;
constexpr int kWBytes = kRows * (kBK / 2);    // 32 KB
constexpr int kSBBytes = kRows * 16;          // 2 KB
constexpr int kStageBytes = kWBytes + 2 * kSBBytes;
constexpr int kSlabK = 2048;
constexpr int kXBytes = kSlabK * 32;          // [k/8][16 tok][8] bf16
constexpr int kXsBytes = (kSlabK / kG) * 16 * 4;
constexpr int kRedBytes = kSets * kRows * 16 * 4;
constexpr int kMaxSlabs = 64;
constexpr int kMaxPend = 32;
constexpr int kMaxRowTiles = 16384;
constexpr int kNumBars = 2 * kStages + 1 + 2 * kSets;  // full, empty, x, mma_done[set][2]
constexpr size_t kSmemBytes = 1024 + (size_t)kStages * kStageBytes + kXBytes + kXsBytes + kRedBytes + 8 * kNumBars +
                              3 * kMaxPend * 4 + 2 * kSets * 4 + 64;
constexpr uint32_t kTmemCols = 512;
// TMEM columns: set j owns [96 j, 96 j + 96): A buffers at +0 and +32 (32 columns = 64 k), D buffers at +64, +80.
constexpr uint32_t kSetCols = 96;

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

// Thread `tid` of the CTA that took the last ticket of row tile nt sums that tile's partial tiles in a fixed order.
__device__ __noinline__ void finalize_tile(const Plan& plan, const float4* pieces, unsigned* counters,
                                           __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ bias, int nt,
                                           int tid, int set, int r) {
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s2 = 0; s2 < plan.S; ++s2) {
    const SlabGeom g2 = slab_geom(plan, s2);
    int f;
    const int np = tile_pieces(g2, nt, &f);
    for (int p = 0; p < np; ++p) {
      const float4 a = ld_cg_f4(&pieces[((size_t)(s2 * plan.maxp + p) * plan.NT + nt) * kDequant + tid]);
      v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
    }
  }
  if (tid == 0) counters[nt] = 0;
  store_rows<__nv_bfloat16>(v, y, bias, nt * kRows + r, set, plan.M, plan.N);
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
  float4* red = (float4*)((uint8_t*)xs + kXsBytes);
  uint64_t* bars = (uint64_t*)((uint8_t*)red + kRedBytes);
  volatile int* pend = (volatile int*)(bars + kNumBars);
  int* tickets = (int*)(pend + 3 * kMaxPend);  // [set][buf]: warps of the set that have written the operand
  uint32_t* tmem_holder = (uint32_t*)(tickets + 2 * kSets);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_full = bar0, bar_empty = bar0 + 8 * kStages, bar_x = bar0 + 16 * kStages;
  const uint32_t bar_done = bar_x + 8;  // [set][buf]

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
      mbar_init(bar_empty + 8 * i, kDequantWarps);
    }
    mbar_init(bar_x, 1);
    for (int i = 0; i < 2 * kSets; ++i) {
      mbar_init(bar_done + 8 * i, 1);  // tcgen05.commit
      tickets[i] = 0;
    }
    mbar_fence_init();
  }
  if (warp == kDequantWarps) tmem_alloc(smem_u32(tmem_holder), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_holder;

  if (warp == kDequantWarps) {
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
  } else {
    // ======================= dequant / epilogue warps =======================
    const int set = warp >> 2, r = ((warp & 3) << 5) | lane;  // TMEM lane = weight row inside the tile
    const uint32_t lane_base = (uint32_t)((warp & 3) << 5) << 16;
    const uint32_t xaddr = smem_u32(xbuf);
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
      uint4 v[kXBytes / 16 / kDequant];
#pragma unroll
      for (int j = 0; j < kXBytes / 16 / kDequant; ++j) {
        const int ci = tid + j * kDequant, tok = ci & 15, kb = ci >> 4;
        v[j] = make_uint4(0, 0, 0, 0);
        if (tok < M && kb < kb_lim) v[j] = *(const uint4*)(x + (size_t)tok * plan.K + (size_t)sg.c0 * kBK + kb * 8);
      }
#pragma unroll
      for (int j = 0; j < kXBytes / 16 / kDequant; ++j) {
        uint4 o;
        o.x = prmt(v[j].x, v[j].z, 0x5410); o.y = prmt(v[j].x, v[j].z, 0x7632);
        o.z = prmt(v[j].y, v[j].w, 0x5410); o.w = prmt(v[j].y, v[j].w, 0x7632);
        ((uint4*)xbuf)[tid + j * kDequant] = o;
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    named_bar_sync(1, kDequant);
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
    named_bar_sync(1, kDequant);

    float out[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) out[i] = 0.f;
    // up to two submitted-but-uncollected groups: (scale, folded bias, slab group index)
    float ps[2] = {0.f, 0.f}, pb[2] = {0.f, 0.f};
    int pg[2] = {0, 0};
    unsigned n = 0, ncol = 0;  // groups submitted / collected by this thread (a unit submits two: buffers 0, 1)
    bool primed = false;       // two groups are in flight
    int npend = 0;

    // collect = wait for the MMAs of group `ncol` (buffer `buf`), start the TMEM load of its accumulator ...
    auto collect_begin = [&](const int buf, uint32_t (&dr)[16]) {
      const uint32_t par = (ncol >> 1) & 1;
      if (!aborted && !mbar_wait(bar_done + 8 * (set * 2 + buf), par)) { aborted = true; atomicExch(err, 14); }
      tc_fence_after();
      tc_ld16_issue(tmem + lane_base + set * kSetCols + 64 + 16 * buf, dr);
    };
    // ... and fold it into `out` with that group's scale and bias.
    auto collect_end = [&](const int buf, uint32_t (&dr)[16]) {
      tc_ld16_wait(dr);
      const float sc = ps[buf], bq = pb[buf];
      const float4* xr = (const float4*)(xs + pg[buf] * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 xv = xr[i];
        out[4 * i + 0] = fmaf(sc, __uint_as_float(dr[4 * i + 0]), fmaf(bq, xv.x, out[4 * i + 0]));
        out[4 * i + 1] = fmaf(sc, __uint_as_float(dr[4 * i + 1]), fmaf(bq, xv.y, out[4 * i + 1]));
        out[4 * i + 2] = fmaf(sc, __uint_as_float(dr[4 * i + 2]), fmaf(bq, xv.z, out[4 * i + 2]));
        out[4 * i + 3] = fmaf(sc, __uint_as_float(dr[4 * i + 3]), fmaf(bq, xv.w, out[4 * i + 3]));
      }
      ++ncol;
    };
    auto flush_tickets = [&]() {
      named_bar_sync(1, kDequant);
      if (tid == 32) {
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
      named_bar_sync(1, kDequant);
      for (int i = 0; i < npend; ++i)
        if (pend[2 * kMaxPend + i]) finalize_tile(plan, pieces, counters, y, bias, pend[i], tid, set, r);
      named_bar_sync(1, kDequant);
    };

    int stage = 0, nt = (int)(u_begin / sg.cs), kc = (int)(u_begin % sg.cs);
    uint32_t par = 0;
    for (unsigned u = u_begin; u < u_end; ++u) {
      if (!aborted && !mbar_wait(bar_full + 8 * stage, par)) { aborted = true; atomicExch(err, 15); }
      const uint8_t* st = stages + stage * kStageBytes;
      const uint32_t s2 = *(const uint32_t*)(st + kWBytes + r * 16 + set * 4);
      const uint32_t b2 = *(const uint32_t*)(st + kWBytes + kSBBytes + r * 16 + set * 4);
#pragma unroll
      for (int g2 = 0; g2 < 2; ++g2, ++n) {
        const int buf = g2;
        const int gi = 2 * set + g2;
        const uint8_t* wrow = st + (gi >> 2) * (kRows * 128) + r * 128;
        const int c0 = 2 * (gi & 3);
        // long-latency operations are issued back to back and their waits pushed behind independent work:
        // weights (shared memory) -> previous accumulator (TMEM load) -> dequantise -> TMEM store -> fold -> publish
        const uint4 w0 = *(const uint4*)(wrow + (((c0) ^ (r & 7)) << 4));
        const uint4 w1 = *(const uint4*)(wrow + (((c0 + 1) ^ (r & 7)) << 4));
        uint32_t dr[16];
        if (primed) collect_begin(buf, dr);  // also means A[buf] and D[buf] are free again
        const uint32_t words[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        const uint32_t a_addr = tmem + lane_base + set * kSetCols + 32 * buf;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t regs[16];
#pragma unroll
          for (int w = 0; w < 4; ++w)
#pragma unroll
            for (int p = 0; p < 4; ++p)
              regs[4 * w + p] = lop3_and_or(words[4 * half + w] >> (4 * p), 0x000F000Fu, 0x43004300u);
          tc_st16(a_addr + 16 * half, regs);
        }
        if (primed) collect_end(buf, dr);
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          __threadfence_block();
          const int old = atomicAdd(&tickets[set * 2 + buf], 1);
          if ((old & 3) == 3) {  // the set's operand for this group is complete: issue its MMAs
            __threadfence_block();
            tc_fence_after();
            const int gs = kc * 8 + gi;  // group index inside the slab
            const uint32_t d = tmem + set * kSetCols + 64 + 16 * buf, a = tmem + set * kSetCols + 32 * buf;
#pragma unroll
            for (int i = 0; i < 4; ++i)
              tc_mma(d, a + 8 * i, smem_desc(xaddr + (uint32_t)(gs * 8 + 2 * i) * 256u, 256u, 128u), kIdesc, i > 0);
            tc_commit(bar_done + 8 * (set * 2 + buf));
          }
        }
        const float sc = __uint_as_float((g2 ? (s2 >> 16) : (s2 & 0xFFFFu)) << 16);
        const float bi = __uint_as_float((g2 ? (b2 >> 16) : (b2 & 0xFFFFu)) << 16);
        ps[buf] = sc;
        pb[buf] = fmaf(-128.f, sc, bi);
        pg[buf] = kc * 8 + gi;
      }
      primed = true;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_empty + 8 * stage);
      if (++stage == kStages) { stage = 0; par ^= 1; }

      const bool seg_end = (kc == sg.cs - 1) || (u == u_end - 1);
      if (seg_end) {
        {
          uint32_t d0[16], d1[16];
          collect_begin(0, d0);
          ++ncol;              // the parity of buffer 1's barrier belongs to the next group
          collect_begin(1, d1);
          --ncol;
          collect_end(0, d0);
          collect_end(1, d1);
        }
        primed = false;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          red[(set * 4 + i) * kRows + r] = make_float4(out[4 * i], out[4 * i + 1], out[4 * i + 2], out[4 * i + 3]);
          out[4 * i] = out[4 * i + 1] = out[4 * i + 2] = out[4 * i + 3] = 0.f;
        }
        named_bar_sync(1, kDequant);
        float4 v = red[(0 * 4 + set) * kRows + r];  // tokens 4*set .. 4*set+3 of row r, summed over the 4 sets
#pragma unroll
        for (int s3 = 1; s3 < kSets; ++s3) {
          const float4 a = red[(s3 * 4 + set) * kRows + r];
          v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
        }
        int total = 0, first_here = 0;
        for (int sl = lane; sl < plan.S; sl += 32) {
          const SlabGeom g2 = slab_geom(plan, sl);
          int f;
          total += tile_pieces(g2, nt, &f);
        }
        total = __reduce_add_sync(0xffffffffu, total);
        tile_pieces(sg, nt, &first_here);
        if (total > 1) {
          pieces[((size_t)(s * plan.maxp + (bl - first_here)) * NT + nt) * kDequant + tid] = v;
          if (tid == 0) { pend[npend] = nt; pend[kMaxPend + npend] = total; }
          ++npend;
        } else {
          store_rows<__nv_bfloat16>(v, y, bias, nt * kRows + r, set, M, N);
        }
        named_bar_sync(1, kDequant);
        if (npend == kMaxPend) { flush_tickets(); npend = 0; }
      }
      if (++kc == sg.cs) { kc = 0; ++nt; }
    }
    if (npend > 0) flush_tickets();
  }

  // every warp ends here: the accumulator memory goes back before the CTA exits
  tc_fence_before();
  __syncthreads();
  if (warp == kDequantWarps) tmem_dealloc(tmem, kTmemCols);
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
size_t plan_workspace(const Plan& p) { return counters_bytes() + (size_t)p.S * p.maxp * p.NT * kDequant * sizeof(float4); }

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
