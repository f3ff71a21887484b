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
//   producer warp  : TMEM allocation; TMA loads of a unit's weights, scales, biases and 16 x 512 activation slice.
//   permuter warps : reorder the k of every 8-block of the landed activation slice in place (see above).
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
constexpr int kFin = 2;               // partial tiles whose loads are in flight together in the finalizer
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
// epilogue scratch: per-token factors (one copy per epilogue warp), one tile of residual values (bf16), one tile of the
// other CTAs' summed partial sums (fp32)
constexpr int kEpResOff = 256, kEpOthOff = kEpResOff + 16 * kRows * 2;
constexpr int kEpNwOff = kEpOthOff + 16 * kRows * 4;   // the row's next-norm weight (mode 1), one bf16 per row
constexpr int kEpSmemBytes = kEpNwOff + kRows * 2;
constexpr size_t kSmemBytes = 1024 + (size_t)kStages * kStageBytes + kEpSmemBytes + 8 * kNumBars + 128;
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
// The matmul that follows this one in the stream (dflash_verify_qmm_prefetch_next): its first units per block are pulled
// into L2 while this kernel drains, so the next kernel's pipeline fills at L2 latency instead of a cold HBM ramp.
struct NextPlan {
  int valid, C, NT, ctas;
};
constexpr int kPrefetchUnits = 4;  // units per block of the next matmul (one ring's worth)
// Expert-gathered launches (mixture-of-experts layers): the weights are stacked expert matrices of `block_rows` rows
// and `cpb` K chunks each; only the experts slot_expert[0 .. *n_dev) take part, and their number is known on the device.
//   GATHER 1, rows gathered:   row tile nt reads expert slot nt / block_tiles          (gate|up of the active experts)
//   GATHER 2, chunks gathered: K chunk kc reads expert slot kc / cpb, x chunk kc        (down, summed over the experts)
// Only the weight coordinates and the tile / chunk counts change; the host plans for n_max slots, the block patches
// NT (or C) and the number of working blocks from *n_dev after the wait on the routing kernel.
struct Gather {
  int mode, block_tiles, cpb, block_rows, n_max;
  const int* slot_expert;
  const int* n_dev;
};
constexpr int kMaxSlots = 272;

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
template <int N>
__device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
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

// What the epilogue does with a finished row tile (device-side copy of dflash_qmm_epilogue).
//   mode 0: y = acc * inv (+ bias)
//   mode 1: y = residual + acc (the residual stream, stored in bf16), scaled = y * next_w, out_ssq[(tile, warp)][token] =
//           the sum of y^2 over the warp's 32 rows: the next matmul finishes the RMSNorm from these partial sums
//   mode 2: rows are (gate_j, up_j) interleaved; y[t][j] = silu(gate) * up, both rounded to bf16 first
// inv[token] = rsqrt(sum_p in_ssq[p][token] / in_dim + eps) when in_ssq is given (x then holds h * norm_weight, not
// yet divided by the row's RMS: a per-token factor commutes with the matmul), else 1.
struct Epi {
  int mode, in_parts;
  float in_dim, eps;
  const float* in_ssq;
  const __nv_bfloat16* residual;
  const __nv_bfloat16* next_w;
  __nv_bfloat16* scaled;
  float* out_ssq;
};

// The 16 per-token factors, left in the warp's own 16 floats of shared memory (registers are scarce in this kernel and
// local memory is slow with nearly all of L1 given to shared memory).  The partial sums are added in a fixed order.
__device__ __forceinline__ void token_factors(const Epi& e, int lane, float* inv_sm) {
  if (e.in_ssq == nullptr) {
    if (lane < 16) inv_sm[lane] = 1.f;
    __syncwarp();
    return;
  }
  // entry f of the array seen as float4 = tokens 4 (f % 4) .. + 3 of part f / 4; lane l reads f = l, l + 32, ...
  const float4* src = (const float4*)e.in_ssq;
  const int n4 = e.in_parts * 4;
  float4 acc[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int f0 = lane; f0 < n4; f0 += 128) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = f0 + 32 * u < n4 ? ld_cg_f4(src + f0 + 32 * u) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int u = 0; u < 4; ++u) { acc[u].x += v[u].x; acc[u].y += v[u].y; acc[u].z += v[u].z; acc[u].w += v[u].w; }
  }
  float4 s = make_float4((acc[0].x + acc[1].x) + (acc[2].x + acc[3].x), (acc[0].y + acc[1].y) + (acc[2].y + acc[3].y),
                         (acc[0].z + acc[1].z) + (acc[2].z + acc[3].z), (acc[0].w + acc[1].w) + (acc[2].w + acc[3].w));
#pragma unroll
  for (int m = 4; m <= 16; m <<= 1) {
    s.x += __shfl_xor_sync(0xffffffffu, s.x, m); s.y += __shfl_xor_sync(0xffffffffu, s.y, m);
    s.z += __shfl_xor_sync(0xffffffffu, s.z, m); s.w += __shfl_xor_sync(0xffffffffu, s.w, m);
  }
  const float rd = 1.f / e.in_dim;
  if (lane < 4) {  // lane q holds the token quad q
    inv_sm[4 * lane + 0] = rsqrtf(s.x * rd + e.eps); inv_sm[4 * lane + 1] = rsqrtf(s.y * rd + e.eps);
    inv_sm[4 * lane + 2] = rsqrtf(s.z * rd + e.eps); inv_sm[4 * lane + 3] = rsqrtf(s.w * rd + e.eps);
  }
  __syncwarp();
}

// Row n's residual values of the 16 tokens go to shared memory ([token][row of the tile], read back by the same thread)
// before the accumulators are waited for.
__device__ __forceinline__ void prefetch_row(const Epi& e, int n, int r, int M, int N, unsigned short* res_sm) {
  if (e.mode != 1) return;
  const unsigned short* rs = (const unsigned short*)e.residual;
  unsigned short v[16];
  // the next norm's weight of this row (cold in HBM) rides with the residual values instead of waiting on the tail
  const unsigned short nw = (e.next_w != nullptr && n < N) ? ((const unsigned short*)e.next_w)[n] : (unsigned short)0x3F80;
#pragma unroll
  for (int t = 0; t < 16; ++t) v[t] = (n < N && t < M) ? rs[(size_t)t * N + n] : (unsigned short)0;
#pragma unroll
  for (int t = 0; t < 16; ++t) res_sm[t * kRows + r] = v[t];
  res_sm[(kEpNwOff - kEpResOff) / 2 + r] = nw;
}

// One finished row (all 16 tokens) of row tile nt: v = the accumulators.  Called by whole warps (modes 1 and 2 exchange
// values between the lanes); lanes whose row lies beyond N take part without storing.
__device__ __forceinline__ void finish_row(const Epi& e, const Plan& plan, float (&v)[16], const float* inv_sm,
                                           const unsigned short* res_sm, __nv_bfloat16* y,
                                           const __nv_bfloat16* __restrict__ bias, int nt, int r, int lane) {
  const int n = nt * kRows + r, M = plan.M, N = plan.N;
  const bool live = n < N;
  if (e.mode == 0) {
    if (!live) return;
    const float bv = bias ? __bfloat162float(bias[n]) : 0.f;
#pragma unroll
    for (int t = 0; t < 16; ++t)
      if (t < M) y[(size_t)t * N + n] = __float2bfloat16_rn(v[t] * inv_sm[t] + bv);
    return;
  }
  if (e.mode == 1) {
    const float next_w = __uint_as_float((uint32_t)res_sm[(kEpNwOff - kEpResOff) / 2 + r] << 16);
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      const float res = __uint_as_float((uint32_t)res_sm[t * kRows + r] << 16);
      const __nv_bfloat16 hb = __float2bfloat16_rn(res + v[t] * inv_sm[t]);
      const float h = __bfloat162float(hb);
      v[t] = 0.f;
      if (live && t < M) {
        y[(size_t)t * N + n] = hb;
        if (e.scaled != nullptr) e.scaled[(size_t)t * N + n] = __float2bfloat16_rn(h * next_w);
        v[t] = h * h;
      }
    }
    if (e.out_ssq != nullptr) {
      // 16 sums over the 32 lanes in 16 exchanges: every step halves the values a lane carries
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const int keep = 8 >> s, m = 16 >> s;
        const bool up = (lane & m) != 0;
#pragma unroll
        for (int i = 0; i < keep; ++i) {
          const float send = up ? v[i] : v[i + keep];
          const float mine = up ? v[i + keep] : v[i];
          v[i] = mine + __shfl_xor_sync(0xffffffffu, send, m);
        }
      }
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1);
      const int t = ((lane >> 4) & 1) * 8 + ((lane >> 3) & 1) * 4 + ((lane >> 2) & 1) * 2 + ((lane >> 1) & 1);
      if ((lane & 1) == 0) e.out_ssq[(size_t)(nt * 4 + (r >> 5)) * 16 + t] = v[0];
    }
    return;
  }
  // mode 2: lane pairs hold (gate, up) of output column n / 2; the even lane finishes tokens 0..7, the odd one 8..15
  const int I = N >> 1, j = n >> 1;
  const bool odd = (lane & 1) != 0;
#pragma unroll
  for (int t = 0; t < 16; ++t) {
    const float mine = __bfloat162float(__float2bfloat16_rn(v[t] * inv_sm[t]));
    const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
    const float g = odd ? other : mine, u = odd ? mine : other;
    const bool my_token = odd ? (t >= 8) : (t < 8);
    if (live && my_token && t < M) y[(size_t)t * I + j] = __float2bfloat16_rn(g / (1.f + __expf(-g)) * u);
  }
}

// v += the partial tiles [from, to) of row tile nt, in that order (thread r owns row r); the loads of kFin tiles are
// in flight together.
__device__ __forceinline__ void sum_pieces(const Plan& plan, const float4* pieces, int nt, int from, int to, int r,
                                           float (&o)[16]) {
  float4 v[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) v[q] = make_float4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
  for (int p0 = from; p0 < to; p0 += kFin) {
    float4 a[kFin][4];
#pragma unroll
    for (int i = 0; i < kFin; ++i)
      if (p0 + i < to) {
        const float4* src = &pieces[((size_t)(p0 + i) * plan.NT + nt) * kTileF4 + r];
#pragma unroll
        for (int q = 0; q < 4; ++q) a[i][q] = ld_cg_f4(src + q * kRows);
      }
#pragma unroll
    for (int i = 0; i < kFin; ++i)
      if (p0 + i < to) {
#pragma unroll
        for (int q = 0; q < 4; ++q) { v[q].x += a[i][q].x; v[q].y += a[i][q].y; v[q].z += a[i][q].z; v[q].w += a[i][q].w; }
      }
  }
#pragma unroll
  for (int q = 0; q < 4; ++q) { o[4 * q] = v[q].x; o[4 * q + 1] = v[q].y; o[4 * q + 2] = v[q].z; o[4 * q + 3] = v[q].w; }
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
  static constexpr int kWarps = (kMmaWarp + kMma + 3) / 4 * 4;  // whole warpgroups (the last warp has no role)
  static constexpr int kThreads = kWarps * 32;
  // Registers per thread.  The kernel starts with kRegLaunch everywhere (what __launch_bounds__ lets the compiler use);
  // setmaxnreg then moves registers from the warpgroups that only issue requests to the ones that do arithmetic.  A
  // warpgroup's four warps sit on the four SM sub-partitions, so the budget is per sub-partition: one warp of each.
  static constexpr int kRegLaunch = (65536 / kThreads) / 8 * 8;
  static constexpr int kRegDq = NDQ == 12 ? 80 : 104, kRegEp = 104, kRegX = 56, kRegCtl = 48;  // no spills (ptxas -v)
  static_assert((NDQ / 4) * kRegDq + kRegEp + kRegX + 2 * kRegCtl <= (kWarps / 4) * kRegLaunch,
                "setmaxnreg.inc would wait for registers that never come");
  static constexpr int kSlots = NDQ / 4;                       // pairs being dequantised at the same time
  static constexpr int kClasses = 3;                           // pair classes of the issuing threads (p mod 3)
  static_assert(kNA % kSlots == 0 && kNA % kClasses == 0, "a ring buffer must belong to one slot and one pair class");
};

template <int NDQ, int GATHER>
__global__ void __launch_bounds__(Roles<NDQ>::kThreads, 1)
qmm_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmS,
              const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmX,
              const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* y, float4* __restrict__ pieces,
              unsigned* __restrict__ counters, const __grid_constant__ Plan plan,
              const __grid_constant__ Epi epi, int* __restrict__ err, unsigned long long* __restrict__ stamps,
              const __grid_constant__ CUtensorMap nxW, const __grid_constant__ CUtensorMap nxS,
              const __grid_constant__ CUtensorMap nxB, const __grid_constant__ NextPlan nxt,
              const __grid_constant__ Gather ga) {
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
  uint8_t* ep_smem = stages + kStages * kStageBytes;
  uint64_t* bars = (uint64_t*)(ep_smem + kEpSmemBytes);
  uint32_t* tmem_holder = (uint32_t*)(bars + kNumBars);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_full = bar0, bar_empty = bar_full + 8 * kStages, bar_xraw = bar_empty + 8 * kStages;
  const uint32_t bar_aready = bar_xraw + 8 * kStages, bar_afree = bar_aready + 8 * kNA;
  const uint32_t bar_dready = bar_afree + 8 * kNA, bar_dfree = bar_dready + 8;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int bl = (int)blockIdx.x;
  Plan P = plan;
  __shared__ int s_slots[GATHER != 0 ? kMaxSlots : 1];
  if constexpr (GATHER != 0) {
    pdl_wait();  // the slot list and its length are the routing kernel's output
    int n_act = *ga.n_dev;
    n_act = n_act < 0 ? 0 : (n_act > ga.n_max ? ga.n_max : n_act);
    if (GATHER == 1) P.NT = n_act * ga.block_tiles; else P.C = n_act * ga.cpb;
    const unsigned total_units = (unsigned)P.NT * (unsigned)P.C;
    if (total_units == 0u) {  // no active expert here: the summed output is zero, the gathered rows do not exist
      if (epi.mode != 0 && tid == 0) atomicCAS(err, 0, 19);  // a residual epilogue needs at least one expert (callers keep the shared one)
      if (GATHER == 2)
        for (int i = bl * (int)blockDim.x + tid; i < plan.M * plan.N; i += (int)(gridDim.x * blockDim.x)) y[i] = __float2bfloat16_rn(0.f);
      return;
    }
    P.ctas = total_units < gridDim.x ? (int)total_units : (int)gridDim.x;
  }
  if (bl >= P.ctas) return;  // before any allocation or barrier
  const int C = P.C, NT = P.NT, M = P.M, N = P.N;
  const unsigned units = (unsigned)NT * (unsigned)C;
  const unsigned u_begin = (unsigned)bl * units / P.ctas, u_end = (unsigned)(bl + 1) * units / P.ctas;
  const unsigned npairs = (u_end - u_begin) * 4u;
  const int nt0 = (int)(u_begin / (unsigned)C), nt1 = (int)((u_end - 1) / (unsigned)C);

  // Producer state (one thread): the next stage to fill and the unit it takes.
  int p_stage = 0, p_nt = nt0, p_kc = (int)(u_begin % (unsigned)C);
  uint32_t p_par = 1;
  unsigned p_u = u_begin;
  uint64_t pol_stream = 0, pol_keep = 0;
  auto request_weights = [&]() {  // the weights, scales and biases of unit p_u into stage p_stage
    const uint32_t full = bar_full + 8 * p_stage, dst = smem_u32(stages + p_stage * kStageBytes);
    mbar_arrive_expect_tx(full, kTmaBytes);
    int wy = p_nt * kRows, wx = p_kc * (kBK / 2), sx = p_kc * 8;
    if constexpr (GATHER == 1) {
      const int slot = p_nt / ga.block_tiles;
      wy = s_slots[slot] * ga.block_rows + (p_nt - slot * ga.block_tiles) * kRows;
    }
    if constexpr (GATHER == 2) {
      const int slot = p_kc / ga.cpb, kin = p_kc - slot * ga.cpb;
      wy = s_slots[slot] * ga.block_rows + p_nt * kRows;
      wx = kin * (kBK / 2);
      sx = kin * 8;
    }
    tma_load_2d(dst, &tmW, wx, wy, full, pol_stream);
    tma_load_2d(dst + kRows * 128, &tmW, wx + 128, wy, full, pol_stream);
    tma_load_2d(dst + kWBytes, &tmS, sx, wy, full, pol_keep);
    tma_load_2d(dst + kWBytes + kSBBytes, &tmB, sx, wy, full, pol_keep);
    if (++p_stage == kStages) { p_stage = 0; p_par ^= 1; }
    if (++p_kc == C) { p_kc = 0; ++p_nt; }
    ++p_u;
  };
  if constexpr (GATHER != 0) {
    if (warp == R::kProducerWarp) {  // the slot -> expert table, for the producer thread alone
      const int n_slots = GATHER == 1 ? NT / ga.block_tiles : C / ga.cpb;
      for (int i = lane; i < n_slots && i < kMaxSlots; i += 32) s_slots[i] = ga.slot_expert[i];
      __syncwarp();
    }
  }
  if (warp == R::kProducerWarp && lane == 0) {
    // The producer thread sets the barriers up itself and asks for the first units' weights at once (they are written by
    // no kernel): the requests are on their way while the rest of the block is still being set up.
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
    pol_stream = l2_policy_evict_first();
    pol_keep = l2_policy_evict_last();
    while (p_u < u_end && p_u - u_begin < (unsigned)kEarlyUnits) request_weights();
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmX) : "memory");
  }
  if (warp == R::kWarps - 1) tmem_alloc(smem_u32(tmem_holder), kTmemCols);  // the warp without a role owns the tensor memory
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_holder;
  if (tid == 0) mark(3);

  if (warp >= R::kProducerWarp) reg_dec<R::kRegCtl>();  // two warpgroups: producer, issuing warps, one idle warp
  if (warp == R::kProducerWarp) {
    // ======================= TMA producer =======================
    // Weights are written by no kernel, so they are requested at once, before the wait on the previous kernel.
    if (lane == 0) {
      // x is the previous kernel's output: once the early units' weights are requested (above), the previous kernel is
      // waited for, then every unit's activation tile is requested with (right after) its weights.  Requests are served
      // in order, so an activation tile asked for behind the whole ring of weights would land ~3 us late; behind two
      // units it lands as soon as the MMA could use it.
      unsigned xu = u_begin;  // next unit whose activation tile is still owed
      int xstage = 0, xkc = (int)(u_begin % (unsigned)C);
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
      pdl_wait();
      request_x(p_u);
      while (p_u < u_end) {
        if (!mbar_wait_quiet(bar_empty + 8 * p_stage, p_par)) { TC_TRACE(11, p_u - u_begin); atomicCAS(err, 0, 11 | ((int)(p_u - u_begin) << 8)); break; }
        request_weights();
        request_x(p_u);
      }
      // Everything this block needs is requested; until it exits (the buffered units, the tail) its share of the memory
      // system is idle: pull the next matmul's first units into L2 (a hint: nothing waits for it).
      if (nxt.valid) {
        const unsigned nunits = (unsigned)nxt.NT * (unsigned)nxt.C;
        // (at most two blocks' worth per block: the requests are issued by this one thread, and a small grid ahead of a
        // large one would otherwise spend microseconds issuing them before its block may exit)
        for (int nb = bl, done = 0; nb < nxt.ctas && done < 2; nb += (int)gridDim.x, ++done) {
          const unsigned b0 = (unsigned)nb * nunits / (unsigned)nxt.ctas, b1 = (unsigned)(nb + 1) * nunits / (unsigned)nxt.ctas;
          for (unsigned u = b0; u < b1 && u < b0 + (unsigned)kPrefetchUnits; ++u) {
            const int nt = (int)(u / (unsigned)nxt.C), kc = (int)(u % (unsigned)nxt.C);
            tma_prefetch_2d(&nxW, kc * (kBK / 2), nt * kRows);
            tma_prefetch_2d(&nxW, kc * (kBK / 2) + 128, nt * kRows);
            tma_prefetch_2d(&nxS, kc * 8, nt * kRows);
            tma_prefetch_2d(&nxB, kc * 8, nt * kRows);
          }
        }
      }
    }
  } else if (warp >= R::kMmaWarp) {
    // ======================= MMA issue =======================
    if (lane == 0 && warp < R::kMmaWarp + R::kMma) {
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
    reg_dec<R::kRegX>();
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
    reg_inc<R::kRegDq>();
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
    reg_inc<R::kRegEp>();
    const int r = ((warp & 3) << 5) | lane;  // TMEM lane = weight row inside the tile
    const uint32_t lane_base = (uint32_t)((warp & 3) << 5) << 16;
    const int etid = tid - R::kEpWarp0 * 32;  // 0..127
    bool aborted = false;
    pdl_wait();      // these warps write what a later kernel reads and the previous kernel may still read
    pdl_trigger();
    float* const inv_sm = (float*)ep_smem + (warp & 3) * 16;
    unsigned short* const res_sm = (unsigned short*)(ep_smem + kEpResOff);
    token_factors(epi, lane, inv_sm);
    for (int nt = nt0; nt <= nt1; ++nt) {
      const int seg = nt - nt0;
      prefetch_row(epi, nt * kRows + r, r, M, N, res_sm);
      int first_cta = 0;
      const int total = tile_pieces(P, nt, &first_cta);  // CTAs that share row tile nt
      // A row tile cut over several CTAs is summed from fp32 partial tiles by the tile's FIRST CTA, as (p1 + p2 + ...) +
      // p0 with p0 its own part, which never leaves its registers.  The tile is the end of that CTA's span and the start
      // (or the whole) of the others', so the others are normally done long before: the first CTA waits for their
      // arrivals and sums their parts BEFORE it waits for its own accumulators, which leaves only "add and store" on the
      // kernel's tail.  The others store their part and signal with a release-add; they never wait, so the waits cannot
      // form a cycle (every CTA is resident: at most one per SM is launched).
      float* const oth_sm = (float*)(ep_smem + kEpOthOff);  // [token][row], written and read by the same thread
      const bool owner = total > 1 && bl == first_cta;
      if (owner) {
        unsigned c = 0;
        if (lane == 0) {
          const unsigned* ctr = &counters[nt * 4 + (warp & 3)];
          for (unsigned spins = 0; !aborted; ++spins) {
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(c) : "l"(ctr) : "memory");
            if (c == (unsigned)(total - 1)) break;
            if (spins >= kWaitLimit) { TC_TRACE(18, nt); atomicCAS(err, 0, 18 | (nt << 8)); break; }
            __nanosleep(64);
          }
        }
        c = __shfl_sync(0xffffffffu, c, 0);
        __syncwarp();  // lane 0's acquire before the other lanes' loads
        if (c != (unsigned)(total - 1)) aborted = true;
        float acc[16];
#pragma unroll
        for (int t = 0; t < 16; ++t) acc[t] = 0.f;
        if (!aborted) sum_pieces(P, pieces, nt, 1, total, r, acc);
#pragma unroll
        for (int t = 0; t < 16; ++t) oth_sm[t * kRows + r] = acc[t];
      }
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
      if (total > 1 && !owner) {
        float4* base = &pieces[((size_t)(bl - first_cta) * NT + nt) * kTileF4 + r];
#pragma unroll
        for (int qd = 0; qd < 4; ++qd)
          base[qd * kRows] = make_float4(out[4 * qd], out[4 * qd + 1], out[4 * qd + 2], out[4 * qd + 3]);
        __syncwarp();  // orders the 32 lanes' stores before lane 0's release
        if (lane == 0)
          asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(&counters[nt * 4 + (warp & 3)]) : "memory");
      } else {
        if (owner) {
#pragma unroll
          for (int t = 0; t < 16; ++t) out[t] = oth_sm[t * kRows + r] + out[t];
        }
        finish_row(epi, P, out, inv_sm, res_sm, y, bias, nt, r, lane);
        if (owner && lane == 0) counters[nt * 4 + (warp & 3)] = 0;  // every other part has arrived: ready for the next launch
      }
      if (etid == 0 && nt == nt1) mark(9);
    }
  }

  // every warp ends here: the tensor memory goes back before the CTA exits
  tc_fence_before();
  __syncthreads();
  if (warp == R::kWarps - 1) tmem_dealloc(tmem, kTmemCols);
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
struct NextHint {
  const void* wq; const void* sc; const void* bi; int K, N; bool valid;
};
thread_local NextHint t_next = {};   // dflash_verify_qmm_prefetch_next: consumed by this thread's next launch
bool g_prefetch_next = true;
int g_ndq = 12;  // dequant warps of the launched instantiation (dflash_verify_qmm_set_tc_roles)

bool make_plan(int M, int K, int N, int device, int max_blocks, Plan* p) {
  p->M = M; p->K = K; p->N = N;
  p->C = K / kBK;
  p->NT = (N + kRows - 1) / kRows;
  if (p->NT > kMaxRowTiles || p->C < 1) return false;
  const long long U = (long long)p->NT * p->C;
  // never more CTAs than SMs: a tile's first CTA waits for the others' parts, so all of them must be resident
  long long ctas = sm_count(device);
  if (max_blocks > 0 && max_blocks < ctas) ctas = max_blocks;
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

template <int NDQ, int GATHER = 0>
cudaError_t launch_variant(int grid, cudaStream_t st, int device, const CUtensorMap& tw, const CUtensorMap& ts,
                           const CUtensorMap& tb, const CUtensorMap& tx, const void* bias, void* y, float4* pieces,
                           unsigned* counters, const Plan& plan, const Epi& epi, const CUtensorMap& nw,
                           const CUtensorMap& ns, const CUtensorMap& nb, const NextPlan& nxt, const Gather& ga = Gather{}) {
  auto kern = qmm_tc_kernel<NDQ, GATHER>;
  static bool attr_done[64] = {};
  if (!attr_done[device & 63]) {
    cudaError_t e0 = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e0 != cudaSuccess) return e0;
    // the kernel's setmaxnreg budget assumes the block was given kRegLaunch registers per thread
    cudaFuncAttributes fa;
    e0 = cudaFuncGetAttributes(&fa, kern);
    if (e0 != cudaSuccess) return e0;
    if (fa.numRegs != Roles<NDQ>::kRegLaunch) return cudaErrorLaunchOutOfResources;
    attr_done[device & 63] = true;
  }
  return launch_kernel(kern, dim3(grid), dim3(Roles<NDQ>::kThreads), kSmemBytes, st, tw, ts, tb, tx,
                       (const __nv_bfloat16*)bias, (__nv_bfloat16*)y, pieces, counters, plan, epi,
                       device_error_word(device), g_stamps, nw, ns, nb, nxt, ga);
}

}  // namespace

void set_k_parts(int) {}  // this kernel cuts K only where a CTA's span ends
void set_next(const void* wq, const void* sc, const void* bi, int K, int N) {
  t_next.wq = wq; t_next.sc = sc; t_next.bi = bi; t_next.K = K; t_next.N = N;
  t_next.valid = wq != nullptr && sc != nullptr && bi != nullptr;
}
void set_prefetch_next(int on) { g_prefetch_next = on != 0; }
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

// Consumes this thread's announcement (dflash_verify_qmm_prefetch_next), if any: the announced matmul's tensor maps and
// block -> unit mapping.  The maps are left alone when there is none or it names a shape this kernel does not take.
void take_next_hint(int M, int device, int max_blocks, CUtensorMap* nw, CUtensorMap* ns, CUtensorMap* nb, NextPlan* nxt) {
  if (!t_next.valid) return;
  t_next.valid = false;
  Plan np;
  CUtensorMap a, b, c;
  if (g_prefetch_next && t_next.K % kBK == 0 && make_plan(M, t_next.K, t_next.N, device, max_blocks, &np) &&
      get_map(t_next.wq, t_next.N, t_next.K / 2, 0, &a) && get_map(t_next.sc, t_next.N, t_next.K / kG, 1, &b) &&
      get_map(t_next.bi, t_next.N, t_next.K / kG, 1, &c)) {
    *nw = a; *ns = b; *nb = c;
    nxt->valid = 1; nxt->C = np.C; nxt->NT = np.NT; nxt->ctas = np.ctas;
  }
}

// ---- expert-gathered launches ------------------------------------------------------------------------------------
// The plan of the largest case (n_max active slots) and the largest number of blocks that can share a row tile over
// every possible number of active slots (it sizes the partial-tile workspace).
bool gather_plan(int M, int block_rows, int Kb, int n_max, int mode, int device, int max_blocks, Plan* p) {
  if (block_rows % kRows != 0 || Kb % kBK != 0 || n_max < 1 || n_max > kMaxSlots) return false;
  const int K = mode == 1 ? Kb : n_max * Kb, N = mode == 1 ? n_max * block_rows : block_rows;
  if (!make_plan(M, K, N, device, max_blocks, p)) return false;
  const long long grid = p->ctas;
  long long worst = 1;
  for (int n = 1; n <= n_max; ++n) {
    const long long NT = mode == 1 ? (long long)n * (block_rows / kRows) : block_rows / kRows;
    const long long C = mode == 1 ? Kb / kBK : (long long)n * (Kb / kBK);
    const long long U = NT * C, ctas = U < grid ? U : grid, L = U / ctas;
    long long mp = C > 1 ? (C - 1 + L - 1) / L + 1 : 1;
    if (mp > ctas) mp = ctas;
    if (mp > worst) worst = mp;
  }
  p->maxp = (int)worst;
  return true;
}

size_t gather_workspace_bytes(int M, int block_rows, int Kb, int n_max, int mode, int device, int max_blocks) {
  Plan p;
  if (!gather_plan(M, block_rows, Kb, n_max, mode, device, max_blocks, &p)) return 0;
  return plan_workspace(p);
}

// Returns DFLASH_OK, a negative status, or +1 when this shape is not handled here (the caller then runs qmm.cu).
int launch_gather(const void* x, const void* wq, const void* sc, const void* bi, void* y, int M, int experts, int block_rows,
                  int Kb, int mode, const int* slot_expert, const int* n_dev, int n_max, void* ws, size_t ws_bytes,
                  cudaStream_t st, int device, int max_blocks, const dflash_qmm_epilogue* ep) {
  Plan plan;
  if (!gather_plan(M, block_rows, Kb, n_max, mode, device, max_blocks, &plan)) return 1;
  CUtensorMap tw, ts, tb, tx;
  if (!get_map(wq, experts * block_rows, Kb / 2, 0, &tw) || !get_map(sc, experts * block_rows, Kb / kG, 1, &ts) ||
      !get_map(bi, experts * block_rows, Kb / kG, 1, &tb) || !get_map(x, M, plan.K, 2, &tx))
    return 1;
  const size_t need = plan_workspace(plan);
  if (ws == nullptr || ws_bytes < need)
    return fail(DFLASH_ERR_WORKSPACE, "moe_qmm needs %zu workspace bytes, got %zu", need, ws_bytes);
  unsigned* counters = (unsigned*)ws;
  float4* pieces = (float4*)((uint8_t*)ws + counters_bytes());
  Gather ga{mode, block_rows / kRows, Kb / kBK, block_rows, n_max, slot_expert, n_dev};
  Epi epi = {};
  if (ep != nullptr) {
    epi.mode = ep->mode; epi.in_parts = ep->in_parts; epi.in_dim = ep->in_dim; epi.eps = ep->eps;
    epi.in_ssq = ep->in_ssq; epi.residual = (const __nv_bfloat16*)ep->residual;
    epi.next_w = (const __nv_bfloat16*)ep->next_w; epi.scaled = (__nv_bfloat16*)ep->scaled; epi.out_ssq = ep->out_ssq;
  }
  NextPlan nxt = {};
  CUtensorMap nw = tw, ns = ts, nb = tb;
  take_next_hint(M, device, max_blocks, &nw, &ns, &nb, &nxt);
  cudaError_t e;
  if (g_ndq == 12) {
    e = mode == 1 ? launch_variant<12, 1>(plan.ctas, st, device, tw, ts, tb, tx, nullptr, y, pieces, counters, plan, epi, nw, ns, nb, nxt, ga)
                  : launch_variant<12, 2>(plan.ctas, st, device, tw, ts, tb, tx, nullptr, y, pieces, counters, plan, epi, nw, ns, nb, nxt, ga);
  } else {
    e = mode == 1 ? launch_variant<8, 1>(plan.ctas, st, device, tw, ts, tb, tx, nullptr, y, pieces, counters, plan, epi, nw, ns, nb, nxt, ga)
                  : launch_variant<8, 2>(plan.ctas, st, device, tw, ts, tb, tx, nullptr, y, pieces, counters, plan, epi, nw, ns, nb, nxt, ga);
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "moe_qmm (tcgen05) launch: %s", cudaGetErrorString(e));
  return DFLASH_OK;
}

// Returns DFLASH_OK, a negative status, or +1 when this shape is not handled here (the caller then runs qmm.cu).
int launch(const void* x, const void* wq, const void* sc, const void* bi, const void* bias, void* y, int M, int K, int N,
           void* ws, size_t ws_bytes, cudaStream_t st, int device, int max_blocks, const dflash_qmm_epilogue* ep) {
  if (K % kBK != 0) return 1;
  Epi epi = {};
  if (ep != nullptr) {
    epi.mode = ep->mode; epi.in_parts = ep->in_parts; epi.in_dim = ep->in_dim; epi.eps = ep->eps;
    epi.in_ssq = ep->in_ssq; epi.residual = (const __nv_bfloat16*)ep->residual;
    epi.next_w = (const __nv_bfloat16*)ep->next_w; epi.scaled = (__nv_bfloat16*)ep->scaled; epi.out_ssq = ep->out_ssq;
  }
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
  // the matmul announced to follow this one: its tensor maps and block -> unit mapping ride along as a prefetch hint
  NextPlan nxt = {};
  CUtensorMap nw = tw, ns = ts, nb = tb;
  take_next_hint(M, device, max_blocks, &nw, &ns, &nb, &nxt);
  if (g_ndq == 12) e = launch_variant<12>(grid, st, device, tw, ts, tb, tx, bias, y, pieces, counters, plan, epi, nw, ns, nb, nxt);
  else e = launch_variant<8>(grid, st, device, tw, ts, tb, tx, bias, y, pieces, counters, plan, epi, nw, ns, nb, nxt);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "qmm_tc launch: %s", cudaGetErrorString(e));
  return DFLASH_OK;
}

}  // namespace tc
}  // namespace dflash
