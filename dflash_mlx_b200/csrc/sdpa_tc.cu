// 16-row verify attention on the 5th-generation tensor cores: the partial-softmax pass of csrc/sdpa.cu with K/V moved by
// TMA and both products on tcgen05.  Same contract (q [B,Hq,16,D], k/v [B,Hk,N,D], key n visible to query row i iff
// n <= N-16+i, kernels.py:530; GQA, kernels.py:491) and the same exact two-pass split-KV scheme as the reference's
// `batched_sdpa_2pass_exact` (dflash_mlx/kernels.py:479-637): pass 1 per key range -> (O, max, sum), pass 2 combines.
//
// One CTA = (KV head, 256 consecutive keys).  The Hq/Hk query heads that share the KV head are stacked: 8 heads x 16
// rows = the 128 rows (TMEM lanes) of one MMA tile, so K and V are read once for all of them.
//   S = Q K^T : M128 x N64 x K16 MMAs, A = Q and B = K both K-major from 128B-swizzled shared memory (TMA boxes of 64
//               channels); the four 64-key blocks are issued by four warps into their own 64 accumulator columns.
//   softmax   : S (up to 256 fp32 columns) stays in TENSOR MEMORY, so the pass is exact without rescaling: a thread owns
//               a row, reads it once for the maximum and once more for p = exp2((s - max) * scale), and writes P as
//               bf16 pairs over the front of S (column j/2 is written after column j was read).
//   O = P V   : A = P from tensor memory, B = V straight from the TMA box - rows are keys, 128 bytes of channels each,
//               which is the MN-major 128B-swizzle canonical layout (8 keys = one 1024-byte group) - four warps issue
//               one 64-channel slab each into their own accumulator columns.
// The four K blocks land in four 32 KB buffers (D = 256); as soon as the MMAs of block b are done its buffer takes
// V block b, which therefore streams in while the softmax runs.  Partials: bf16 O + fp32 max / sum; the combine pass is
// the second launch.  Every wait is bounded (device error code 51); no mask array, bf16 only, <= 8 heads per KV head.
#include <atomic>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace dflash {
namespace sdpa_tc {

constexpr int kKeys = 256, kBlk = 64, kBufs = 4, kRows = 128;
constexpr int kSoftWarps = 4, kProducerWarp = 4, kMmaWarp0 = 5, kThreads = 9 * 32;
constexpr uint32_t kTmemCols = 512, kOCol0 = 256;
constexpr int kFuseMaxSplits = 128;   // most key ranges per head the one-launch combine handles

struct Args {
  const float* scale_dummy;
  void* out; __nv_bfloat16* part_o; float* part_m; float* part_l;
  int B, Hq, Hk, N, gqa, splits, keys_per_split;
  float scale_log2;
  const int* n_dev;
  unsigned* counters;   // non-NULL: the blocks of a KV head meet after pass 1 and share pass 2 between them (one launch)
};

// Bounded wait (hardware-suspended polls): gives up after ~2^16 polls of a few microseconds each (a fraction of a second).
#ifndef DFLASH_SDPA_TC_WAIT_POLLS
#define DFLASH_SDPA_TC_WAIT_POLLS (1u << 16)
#endif
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < DFLASH_SDPA_TC_WAIT_POLLS; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(1000u)
        : "memory");
    if (ok) return true;
  }
  return false;
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_holder, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_holder), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D (+)= A (shared memory descriptor) * B (shared memory descriptor)
__device__ __forceinline__ void mma_ss(uint32_t d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accum)
      : "memory");
}
// D (+)= A (tensor memory) * B (shared memory descriptor)
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accum)
      : "memory");
}
__device__ __forceinline__ void ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
      "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n\ttcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
        "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),
        "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// K-major operand, 128B swizzle: rows of 128 bytes (64 channels), 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_sw128(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand, 128B swizzle: a row is one k index holding 64 consecutive n (128 bytes), 8 k = one 1024-byte group
// (stride offset), the next 64 n lie `lbo` bytes further (leading offset).
__device__ __forceinline__ uint64_t desc_mn_sw128(uint32_t addr, uint32_t lbo) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}
// kind::f16 instruction descriptor: D = f32, A = B = bf16, M = 128, N = 64; `b_mn` = B is MN-major.
__device__ __forceinline__ constexpr uint32_t idesc(bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((64u >> 3) << 17) | ((128u >> 4) << 24);
}
__device__ __forceinline__ void tma3(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
               "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tma2(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(map), "r"(x), "r"(y), "r"(bar)
               : "memory");
}

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
sdpa_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const Args a, int* __restrict__ err) {
  constexpr int kSlabs = D / 64;               // 64-channel slabs of a row
  constexpr int kQSlab = kRows * 128;          // bytes of one Q slab
  constexpr int kBufSlab = kBlk * 128;         // bytes of one K / V slab of a 64-key block
  constexpr int kBuf = kSlabs * kBufSlab;      // bytes of one block buffer
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sB = smem + kSlabs * kQSlab;
  uint64_t* bars = (uint64_t*)(sB + kBufs * kBuf);
  uint32_t* tmem_holder = (uint32_t*)(bars + 16);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_q = bar0, bar_kv = bar0 + 8, bar_kfree = bar_kv + 8 * kBufs, bar_s = bar_kfree + 8 * kBufs;
  const uint32_t bar_p = bar_s + 8, bar_o = bar_p + 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, bhk = blockIdx.y, b = bhk / a.Hk, hk = bhk % a.Hk;

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int i = 0; i < kBufs; ++i) { mbar_init(bar_kv + 8 * i, 1); mbar_init(bar_kfree + 8 * i, 1); }
    mbar_init(bar_s, 4);
    mbar_init(bar_p, kSoftWarps);
    mbar_init(bar_o, 4);
    mbar_fence_init();
  }
  if (warp == kProducerWarp) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmQ) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmK) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmV) : "memory");
    }
    tmem_alloc(smem_u32(tmem_holder), kTmemCols);
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = *tmem_holder;
  pdl_wait();      // q and the newest cache rows are the previous kernels' output
  pdl_trigger();
  const int N = a.n_dev ? max(16, min(*a.n_dev, a.N)) : a.N;
  const int k0 = split * a.keys_per_split;
  const int nkeys = max(0, min(a.keys_per_split, N - k0));
  const int nblk = (nkeys + kBlk - 1) / kBlk;

  if (warp == kProducerWarp) {
    if (lane == 0 && nblk > 0) {
      const int qrow0 = (b * a.Hq + hk * a.gqa) * 16;
      mbar_arrive_expect_tx(bar_q, kSlabs * kQSlab);
      for (int s = 0; s < kSlabs; ++s) tma2(smem_u32(sQ + s * kQSlab), &tmQ, 64 * s, qrow0, bar_q);
      for (int blk = 0; blk < nblk; ++blk) {
        mbar_arrive_expect_tx(bar_kv + 8 * blk, kBuf);
        for (int s = 0; s < kSlabs; ++s)
          tma3(smem_u32(sB + blk * kBuf + s * kBufSlab), &tmK, 64 * s, k0 + blk * kBlk, bhk, bar_kv + 8 * blk);
      }
      for (int blk = 0; blk < nblk; ++blk) {   // V block b takes K block b's buffer once its MMAs are done
        if (!wait_bar(bar_kfree + 8 * blk, 0)) { atomicCAS(err, 0, 51 | (1 << 8)); break; }
        mbar_arrive_expect_tx(bar_kv + 8 * blk, kBuf);
        for (int s = 0; s < kSlabs; ++s)
          tma3(smem_u32(sB + blk * kBuf + s * kBufSlab), &tmV, 64 * s, k0 + blk * kBlk, bhk, bar_kv + 8 * blk);
      }
    }
  } else if (warp >= kMmaWarp0) {
    if (lane == 0) {
      const int me = warp - kMmaWarp0;   // key block of S = Q K^T, channel slab of O = P V
      bool ok = true;
      if (me < nblk) {
        ok = wait_bar(bar_q, 0) && wait_bar(bar_kv + 8 * me, 0);
        if (!ok) atomicCAS(err, 0, 51 | (2 << 8));
        fence_after();
        if (ok) {
          const uint32_t d = tmem + 64u * me;
#pragma unroll 1
          for (int s = 0; s < kSlabs; ++s) {
            const uint64_t da = desc_k_sw128(smem_u32(sQ + s * kQSlab));
            const uint64_t db = desc_k_sw128(smem_u32(sB + me * kBuf + s * kBufSlab));
#pragma unroll
            for (int j = 0; j < 4; ++j) mma_ss(d, da + 2 * j, db + 2 * j, idesc(false), (s | j) ? 1u : 0u);
          }
          commit(bar_kfree + 8 * me);
          commit(bar_s);
        }
      }
      if (me >= nblk || !ok) mbar_arrive(bar_s);
      // ---- O slab `me` = P (tensor memory) x V (MN-major) over all keys of this range ----
      if (me < kSlabs && nblk > 0 && ok) {
        if (!wait_bar(bar_p, 0)) { ok = false; atomicCAS(err, 0, 51 | (3 << 8)); }
        fence_after();
        const uint32_t d = tmem + kOCol0 + 64u * me;
        for (int blk = 0; blk < nblk && ok; ++blk) {
          if (!wait_bar(bar_kv + 8 * blk, 1)) { ok = false; atomicCAS(err, 0, 51 | (4 << 8)); break; }
          fence_after();
          const uint64_t dv = desc_mn_sw128(smem_u32(sB + blk * kBuf + me * kBufSlab), kBufSlab);
#pragma unroll
          for (int j = 0; j < 4; ++j)   // 16 keys per MMA = two 1024-byte groups; P: 8 columns (16 bf16) per MMA
            mma_ts(d, tmem + 32u * blk + 8u * j, dv + (uint64_t)(j * (2048 >> 4)), idesc(true), (blk | j) ? 1u : 0u);
        }
        if (ok) commit(bar_o); else mbar_arrive(bar_o);
      } else {
        mbar_arrive(bar_o);
      }
    }
  } else {
    // ---------------- softmax + epilogue: thread = query row (TMEM lane) ----------------
    const int r = warp * 32 + lane, head = r >> 4, i = r & 15;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const bool row_ok = head < a.gqa;
    const int hq = hk * a.gqa + head;
    const int cnt = max(0, min(nkeys, N - 16 + i - k0 + 1));   // keys of this range visible to the row: the first `cnt`
    bool ok = true;
    if (!wait_bar(bar_s, 0)) { ok = false; atomicCAS(err, 0, 51 | (5 << 8)); }
    fence_after();
    float m = -INFINITY, l = 0.f;
    if (nblk > 0 && ok) {
      for (int c0 = 0; c0 < nkeys; c0 += 32) {
        uint32_t v[32];
        ld32(tmem + lane_base + c0, v);
#pragma unroll
        for (int e = 0; e < 32; ++e)
          if (c0 + e < cnt) m = fmaxf(m, __uint_as_float(v[e]));
      }
      const float mref = (m == -INFINITY) ? 0.f : m;
      for (int c0 = 0; c0 < nblk * kBlk; c0 += 32) {
        uint32_t v[32], pk[16];
        ld32(tmem + lane_base + c0, v);
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float p0 = (c0 + e < cnt) ? exp2f((__uint_as_float(v[e]) - mref) * a.scale_log2) : 0.f;
          const float p1 = (c0 + e + 1 < cnt) ? exp2f((__uint_as_float(v[e + 1]) - mref) * a.scale_log2) : 0.f;
          l += p0 + p1;
          __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
          pk[e >> 1] = *(uint32_t*)&h;
        }
        st16(tmem + lane_base + (c0 >> 1), pk);   // column j/2 after column j was read: P overwrites the front of S
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_p);
    if (!wait_bar(bar_o, 0)) { ok = false; atomicCAS(err, 0, 51 | (6 << 8)); }
    fence_after();
    const size_t grow = ((size_t)b * a.Hq + hq) * 16 + i;
    const bool have = nblk > 0 && ok;
    // every lane of the warp takes part in the tensor-memory loads (they are warp-wide instructions); only the stores
    // to global memory depend on whether the lane's row belongs to a real head
    const bool final_out = a.splits == 1;
    const float mul = final_out ? (l == 0.f ? 1.f : 1.f / l) : 1.f;
    __nv_bfloat16* dst = final_out ? (__nv_bfloat16*)a.out + grow * D : a.part_o + (grow * a.splits + split) * D;
    for (int c0 = 0; c0 < D; c0 += 32) {
      uint32_t v[32];
      if (have) ld32(tmem + lane_base + kOCol0 + c0, v);
#pragma unroll
      for (int e = 0; e < 32; e += 8) {
        uint4 w;
        uint32_t* wp = (uint32_t*)&w;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          // O is rounded to bf16 (the partials' type) before it is normalised, with one key range or many: the result
          // then does not depend on how many empty ranges a device-side KV length leaves behind the real ones
          __nv_bfloat162 h = __floats2bfloat162_rn(have ? __uint_as_float(v[e + 2 * q]) : 0.f,
                                                   have ? __uint_as_float(v[e + 2 * q + 1]) : 0.f);
          if (final_out) h = __floats2bfloat162_rn(__bfloat162float(h.x) * mul, __bfloat162float(h.y) * mul);
          wp[q] = *(uint32_t*)&h;
        }
        if (row_ok) *(uint4*)(dst + c0 + e) = w;
      }
    }
    if (row_ok && !final_out) {
      a.part_m[grow * a.splits + split] = (m == -INFINITY) ? -INFINITY : m * a.scale_log2;
      a.part_l[grow * a.splits + split] = l;
    }
    __threadfence();   // the partials are read by other blocks when pass 2 runs inside this launch
  }
  fence_before();
  __syncthreads();
  if (warp == kProducerWarp) tmem_dealloc(tmem, kTmemCols);
  if (a.counters == nullptr || a.splits == 1) return;
  // ---------------- pass 2 inside the same launch ----------------
  // Every block of this KV head has been launched (the host takes this path only when the whole grid is resident: at most
  // one block per SM), so the blocks can wait for each other: arrive on the head's counter, wait (bounded) until all
  // `splits` blocks have, then each block combines its share of the head group's rows (kernels.py:595-637).
  __shared__ float c_w[kThreads / 32][kFuseMaxSplits];   // per warp: the weights of the row it is combining
  __shared__ int c_ok;
  unsigned* arrived = a.counters + 2 * bhk;
  unsigned* done = arrived + 1;
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(arrived, 1u);
    int ok = 0;
    for (unsigned spins = 0; spins < (1u << 22); ++spins) {
      unsigned c;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(c) : "l"(arrived) : "memory");
      if (c >= (unsigned)a.splits) { ok = 1; break; }
      __nanosleep(64);
    }
    if (!ok) atomicCAS(err, 0, 51 | (7 << 8));
    c_ok = ok;
  }
  __syncthreads();
  if (c_ok) {
    // a warp combines one row at a time (no block-wide barrier): lane = 8 channels, 16-byte loads of the bf16 partials
    const int rows_head = a.gqa * 16;
    constexpr int kLanes = D / 8;
    float* w_row = c_w[warp];
    for (int rr = split + warp * a.splits; rr < rows_head; rr += a.splits * (kThreads / 32)) {
      const size_t row = ((size_t)b * a.Hq + hk * a.gqa) * 16 + rr;
      const float* pm = a.part_m + row * a.splits;
      const float* pl = a.part_l + row * a.splits;
      float mx = -INFINITY;
      for (int sidx = lane; sidx < a.splits; sidx += 32) mx = fmaxf(mx, __ldcg(pm + sidx));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float ref = (mx == -INFINITY) ? 0.f : mx;
      float den = 0.f;
      __syncwarp();
      for (int sidx = lane; sidx < a.splits; sidx += 32) {
        const float w = exp2f(__ldcg(pm + sidx) - ref);
        w_row[sidx] = w;
        den += w * __ldcg(pl + sidx);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
      __syncwarp();
      if (lane < kLanes) {
        const uint4* po = (const uint4*)(a.part_o + row * a.splits * D) + lane;
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
        for (int sidx = 0; sidx < a.splits; ++sidx) {   // split order: the same sum as the combine kernel's per channel
          const uint4 v = __ldcg(po + (size_t)sidx * (D / 8));
          const float w = w_row[sidx];
          const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc[2 * e] = fmaf(w, __uint_as_float(u[e] << 16), acc[2 * e]);
            acc[2 * e + 1] = fmaf(w, __uint_as_float(u[e] & 0xFFFF0000u), acc[2 * e + 1]);
          }
        }
        const float inv = den == 0.f ? 1.f : 1.f / den;
        uint4 o4;
        uint32_t* op = (uint32_t*)&o4;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * e] * inv, acc[2 * e + 1] * inv);
          op[e] = *(uint32_t*)&h;
        }
        *((uint4*)((__nv_bfloat16*)a.out + row * D) + lane) = o4;
      }
      __syncwarp();
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned d = atomicAdd(done, 1u);
    if (d == (unsigned)a.splits - 1) {   // the last block to finish: nobody reads the counters any more
      *arrived = 0;
      *done = 0;
    }
  }
}

// pass 2 with bf16 partial outputs: out = sum_s w_s O_s / sum_s w_s l_s, w_s = exp2(m_s - max_s m_s) (kernels.py:595-637)
template <int D>
__global__ void __launch_bounds__(D) combine_kernel(const Args a) {
  __shared__ float sw[1024];
  __shared__ float sred[D / 32];
  __shared__ float sden;
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* pm = a.part_m + (size_t)row * a.splits;
  const float* pl = a.part_l + (size_t)row * a.splits;
  float mx = -INFINITY;
  for (int s = tid; s < a.splits; s += D) mx = fmaxf(mx, pm[s]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) sred[warp] = mx;
  __syncthreads();
  mx = sred[0];
#pragma unroll
  for (int i = 1; i < D / 32; ++i) mx = fmaxf(mx, sred[i]);
  const float ref = (mx == -INFINITY) ? 0.f : mx;
  __syncthreads();
  float den = 0.f;
  for (int s = tid; s < a.splits; s += D) {
    const float w = exp2f(pm[s] - ref);
    sw[s] = w;
    den += w * pl[s];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
  if (lane == 0) sred[warp] = den;
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
    for (int i = 0; i < D / 32; ++i) t += sred[i];
    sden = t;
  }
  __syncthreads();
  const __nv_bfloat16* po = a.part_o + (size_t)row * a.splits * D + tid;
  float acc0 = 0.f, acc1 = 0.f;
  int s = 0;
  for (; s + 2 <= a.splits; s += 2) {
    const float v0 = __bfloat162float(po[(size_t)s * D]), v1 = __bfloat162float(po[(size_t)(s + 1) * D]);
    acc0 = fmaf(sw[s], v0, acc0);
    acc1 = fmaf(sw[s + 1], v1, acc1);
  }
  for (; s < a.splits; ++s) acc0 = fmaf(sw[s], __bfloat162float(po[(size_t)s * D]), acc0);
  const float inv = sden == 0.f ? 1.f : 1.f / sden;   // a row with no visible key yields zeros (kernels.py:630)
  ((__nv_bfloat16*)a.out)[(size_t)row * D + tid] = __float2bfloat16_rn((acc0 + acc1) * inv);
}

// ------------------------------------------------------------------------------------------------------------------
struct MapKey {
  const void* p; long long a, b, c; int kind;
  bool operator==(const MapKey& o) const { return p == o.p && a == o.a && b == o.b && c == o.c && kind == o.kind; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.p) ^ ((size_t)k.a * 1000003u) ^ ((size_t)k.b * 7919u) ^ ((size_t)k.c * 104729u) ^ (size_t)k.kind;
  }
};
std::mutex g_mu;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

// kind 0: q as [rows][D], box 64 x 128.  kind 1: k / v as [B*Hk][N][D] with element strides, box 64 x 64 x 1.
bool get_map(const void* ptr, int kind, long long rows_or_n, int D, long long heads, long long seq_stride, long long head_stride,
             CUtensorMap* out) {
  MapKey key{ptr, rows_or_n * 1024 + D, heads * 4 + kind, seq_stride * 1000003 + head_stride, kind};
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return true; }
  }
  tensormap_encode_fn enc = get_tensormap_encoder();
  if (!enc) return false;
  CUtensorMap m;
  CUresult r;
  cuuint32_t estr[3] = {1, 1, 1};
  if (kind == 0) {
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows_or_n};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)kRows};
    r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)rows_or_n, (cuuint64_t)heads};
    cuuint64_t strides[2] = {(cuuint64_t)seq_stride * 2, (cuuint64_t)head_stride * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)kBlk, 1};
    r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) return false;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps.emplace(key, m);
  *out = m;
  return true;
}

extern int g_split128;
// Keys per block: 256 (the accumulator width); optionally 128 while that still leaves the grid within one block per SM (more
// SMs stream the cache, at the price of twice the partials: measured no faster, so off by default).
int keys_per_split(int N, int heads, int device) {
  const int s128 = (N + 127) / 128;
  return (g_split128 && (long long)s128 * heads <= sm_count(device)) ? 128 : kKeys;
}
int splits_for(int N, int heads, int device) {
  const int kp = keys_per_split(N, heads, device);
  return (N + kp - 1) / kp;
}

// Arrival / completion counters of the one-launch path: kSlots sets of 2 words per KV head, zero when idle (the last
// block of a head resets its pair).  Launches take the sets round robin, so launches in flight on different streams
// do not share one unless more than kSlots are in flight.
constexpr int kSlots = 64, kSlotHeads = 1024;
__device__ unsigned g_counters[kSlots * kSlotHeads * 2];
unsigned* g_counters_ptr[64] = {};
std::atomic<unsigned> g_slot{0};
int g_fuse_combine = 0;
int g_split128 = 0;

size_t workspace_bytes(int B, int Hq, int N, int D) {
  const size_t rows = (size_t)B * Hq * 16, s = (size_t)((N + 127) / 128);   // the finer of the two splittings
  return s > 1 ? rows * s * ((size_t)D * 2 + 8) + 256 : 0;
}

template <int D>
int launch_d(const void* q, const void* k, const void* v, void* out, int B, int Hq, int Hk, int N, long long khs, long long kss,
             long long vhs, long long vss, float scale_log2, const int* n_dev, void* ws, size_t ws_bytes, cudaStream_t st) {
  int device = 0;
  cudaGetDevice(&device);
  CUtensorMap tq, tk, tv;
  if (!get_map(q, 0, (long long)B * Hq * 16, D, 0, 0, 0, &tq) || !get_map(k, 1, N, D, (long long)B * Hk, kss, khs, &tk) ||
      !get_map(v, 1, N, D, (long long)B * Hk, vss, vhs, &tv))
    return 1;
  Args a{};
  a.out = out; a.B = B; a.Hq = Hq; a.Hk = Hk; a.N = N; a.gqa = Hq / Hk;
  a.keys_per_split = keys_per_split(N, B * Hk, device);
  a.splits = splits_for(N, B * Hk, device);
  a.scale_log2 = scale_log2; a.n_dev = n_dev;
  const size_t rows = (size_t)B * Hq * 16;
  if (a.splits > 1) {
    const size_t need = rows * a.splits * ((size_t)D * 2 + 8);
    if (!ws || ws_bytes < need) return fail(DFLASH_ERR_WORKSPACE, "verify_sdpa needs %zu workspace bytes, got %zu", need, ws_bytes);
    if ((uintptr_t)ws & 15) return fail(DFLASH_ERR_MISALIGNED, "verify_sdpa workspace must be 16-byte aligned");
    a.part_o = (__nv_bfloat16*)ws;
    a.part_m = (float*)((uint8_t*)ws + rows * a.splits * D * 2);
    a.part_l = a.part_m + rows * a.splits;
  }
  constexpr size_t smem = (size_t)(D / 64) * kRows * 128 + (size_t)kBufs * (D / 64) * kBlk * 128 + 8 * 16 + 64;
  static bool attr_done[64] = {};
  auto kern = sdpa_tc_kernel<D>;
  if (!attr_done[device & 63]) {
    cudaError_t e0 = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e0 != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e0));
    attr_done[device & 63] = true;
  }
  // pass 2 inside the same launch when every block is resident at once (one block per SM) and the heads fit a counter set
  const bool fuse = g_fuse_combine && a.splits > 1 && a.splits <= kFuseMaxSplits && a.splits * B * Hk <= sm_count(device) && B * Hk <= kSlotHeads &&
                    device >= 0 && device < 64;
  if (fuse) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_counters_ptr[device] == nullptr) {
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, g_counters) != cudaSuccess || p == nullptr) return fail(DFLASH_ERR_LAUNCH, "sdpa: counter symbol");
      g_counters_ptr[device] = (unsigned*)p;
    }
    a.counters = g_counters_ptr[device] + (size_t)(g_slot.fetch_add(1) % kSlots) * kSlotHeads * 2;
  }
  cudaError_t e = launch_kernel(kern, dim3(a.splits, B * Hk), dim3(kThreads), smem, st, tq, tk, tv, a, device_error_word(device));
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "sdpa (tcgen05) launch: %s", cudaGetErrorString(e));
  if (a.splits > 1 && !fuse) {
    e = launch_kernel(combine_kernel<D>, dim3((unsigned)rows), dim3(D), 0, st, a);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "sdpa combine launch: %s", cudaGetErrorString(e));
  }
  return DFLASH_OK;
}

void set_fuse_combine(int on) { g_fuse_combine = on ? 1 : 0; }
void set_split128(int on) { g_split128 = on ? 1 : 0; }

// Returns DFLASH_OK, a negative status, or +1 when the shape is not handled here (the caller then runs csrc/sdpa.cu).
int launch(const void* q, const void* k, const void* v, void* out, int B, int Hq, int Hk, int N, int D, long long khs,
           long long kss, long long vhs, long long vss, float scale_log2, const int* n_dev, void* ws, size_t ws_bytes,
           cudaStream_t st) {
  if (Hq % Hk != 0 || (Hq / Hk) * 16 > kRows || (long long)B * Hk > 65535 || (N + 127) / 128 > 1024) return 1;
  if (D == 256) return launch_d<256>(q, k, v, out, B, Hq, Hk, N, khs, kss, vhs, vss, scale_log2, n_dev, ws, ws_bytes, st);
  if (D == 128) return launch_d<128>(q, k, v, out, B, Hq, Hk, N, khs, kss, vhs, vss, scale_log2, n_dev, ws, ws_bytes, st);
  return 1;
}

}  // namespace sdpa_tc
}  // namespace dflash
