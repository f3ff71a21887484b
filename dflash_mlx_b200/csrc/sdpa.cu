// 16-row verify attention for sm_100a: split-KV partial-softmax pass + combine pass.
//
// Replaces `batched_sdpa_2pass_exact` and the Metal kernels `batched_sdpa_2pass_partials[_mask]`,
// `batched_sdpa_2pass_reduce` (dflash_mlx/kernels.py:658-761, 479-565, 579-638).
//
// q [B,Hq,16,D], k/v [B,Hk,N,D] (N includes the 16 new positions), key n is visible to query row i iff
// n <= N-16+i (kernels.py:530); GQA: head hq reads KV head hq / (Hq/Hk) (kernels.py:491).
//
// Pass 1: one CTA per (KV head, contiguous key range).  The Hq/Hk query heads that share the KV head are
// stacked: warp w owns the 16 rows of query head w, so a K/V block staged once in shared memory is reused by
// every head of the group.  Per 64-key block: S = Q K^T and O += P V on tensor cores (mma.sync m16n8k16, Q
// and K/V fragments via ldmatrix from XOR-swizzled shared memory), online softmax in fp32 registers, K/V
// blocks double-buffered with cp.async.  Each CTA writes un-normalised fp32 (O, max, sum) partials.
// Pass 2: per (head, row) the partials are rescaled by exp2(max_s - max) and summed (kernels.py:595-637).
#include <mutex>

#include "common.cuh"

namespace dflash {
namespace {

constexpr int kBN = 64;  // keys per block
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *(uint32_t*)&v;
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *(uint32_t*)&v;
}
template <typename T> __device__ __forceinline__ float finite_min();
template <> __device__ __forceinline__ float finite_min<__nv_bfloat16>() { return -3.3895313892515355e38f; }
template <> __device__ __forceinline__ float finite_min<__half>() { return -65504.f; }

struct SdpaArgs {
  const void* q; const void* k; const void* v; const void* mask; void* out;
  float* part_o; float* part_m; float* part_l;
  int B, Hq, Hk, N, gqa, splits, blocks_per_split;
  long long k_head_stride, k_seq_stride, v_head_stride, v_seq_stride;  // in elements
  float scale_log2;
  const int* n_dev;  // when not NULL: the KV length lives on the device (N above is then only its upper bound)
};

// Byte offset of 16-byte chunk `chunk` of row `row` in a swizzled tile with `row_bytes` per row.
__device__ __forceinline__ uint32_t swz(int row, int chunk, int row_bytes) {
  return (uint32_t)(row * row_bytes + ((chunk ^ (row & 7)) << 4));
}

template <typename T, int D>
__global__ void __launch_bounds__(256, 1) sdpa_partials_kernel(const SdpaArgs a) {
  using TR = MmaTraits<T>;
  constexpr int RB = D * 2;          // bytes per row
  constexpr int CH = RB / 16;        // 16-byte chunks per row
  constexpr int KS = D / 16;         // k-steps of Q K^T
  constexpr int NT_O = D / 8;        // n-tiles of O
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_wait();
  pdl_trigger();
  const int nwarps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int split = blockIdx.x, bhk = blockIdx.y, b = bhk / a.Hk, hk = bhk % a.Hk;
  const int hq = hk * a.gqa + blockIdx.z * nwarps + warp;  // query head of this warp
  const bool head_ok = (blockIdx.z * nwarps + warp) < a.gqa;

  uint8_t* sQ = smem;
  uint8_t* sK = sQ + nwarps * 16 * RB;
  uint8_t* sV = sK + 2 * kBN * RB;
  const uint32_t uQ = smem_u32(sQ), uK = smem_u32(sK), uV = smem_u32(sV);

  const int N = a.n_dev ? max(16, min(*a.n_dev, a.N)) : a.N;
  const int blk0 = split * a.blocks_per_split;
  const int nblk_total = (N + kBN - 1) / kBN;
  const int blk1 = min(blk0 + a.blocks_per_split, nblk_total);

  const T* kbase = (const T*)a.k + (size_t)bhk * a.k_head_stride;
  const T* vbase = (const T*)a.v + (size_t)bhk * a.v_head_stride;
  auto load_block = [&](int blk, int buf) {
    const int n0 = blk * kBN;
    for (int i = threadIdx.x; i < kBN * CH; i += blockDim.x) {
      const int r = i / CH, ch = i % CH;
      const bool ok = (n0 + r) < N;
      const size_t rr = ok ? (size_t)(n0 + r) : 0;
      cp_async16(uK + buf * kBN * RB + swz(r, ch, RB), kbase + rr * a.k_seq_stride + ch * 8, ok);
      cp_async16(uV + buf * kBN * RB + swz(r, ch, RB), vbase + rr * a.v_seq_stride + ch * 8, ok);
    }
  };

  // Q tile of this CTA's heads (rows of absent heads are zero-filled)
  for (int i = threadIdx.x; i < nwarps * 16 * CH; i += blockDim.x) {
    const int r = i / CH, ch = i % CH;
    const int w = r >> 4, row = r & 15;
    const int h = hk * a.gqa + blockIdx.z * nwarps + w;
    const bool ok = (blockIdx.z * nwarps + w) < a.gqa;
    const T* src = (const T*)a.q + (((size_t)b * a.Hq + (ok ? h : 0)) * 16 + row) * D + ch * 8;
    cp_async16(uQ + swz(r, ch, RB), src, ok);
  }
  if (blk0 < blk1) load_block(blk0, 0);
  cp_async_commit();

  float o[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  const float fmin_t = finite_min<T>();

  for (int blk = blk0; blk < blk1; ++blk) {
    const int buf = (blk - blk0) & 1;
    if (blk + 1 < blk1) load_block(blk + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    // ---- S = Q K^T for this warp's 16 rows x 64 keys ----
    float s[kBN / 8][4];
#pragma unroll
    for (int j = 0; j < kBN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    const uint32_t kb = uK + buf * kBN * RB;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t a0, a1, a2, a3;
      {  // A fragment: rows warp*16 + (lane&15), 16-byte chunk 2*ks + (lane>>4)
        const int r = warp * 16 + (lane & 15);
        ldsm_x4(uQ + swz(r, 2 * ks + (lane >> 4), RB), a0, a1, a2, a3);
      }
#pragma unroll
      for (int jp = 0; jp < kBN / 16; ++jp) {
        // B fragments of two key tiles: matrices (keys 16jp..+7, chunk 2ks), (.., chunk 2ks+1), (keys +8.., 2ks), (.., 2ks+1)
        const int r = jp * 16 + (lane & 7) + ((lane >> 4) << 3);
        const int ch = 2 * ks + ((lane >> 3) & 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(kb + swz(r, ch, RB), b0, b1, b2, b3);
        TR::mma(s[2 * jp], a0, a1, a2, a3, b0, b1);
        TR::mma(s[2 * jp + 1], a0, a1, a2, a3, b2, b3);
      }
    }

    // ---- scale, visibility, online softmax (rows g and g+8 of this warp) ----
    const int n0 = blk * kBN;
    const bool edge = (n0 + kBN > N - 16) || a.mask != nullptr;
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int j = 0; j < kBN / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[j][e] * a.scale_log2;
        if (edge) {
          const int n = n0 + 8 * j + 2 * c + (e & 1);
          const int row = g + ((e >> 1) << 3);
          bool vis = (n < N) && (n <= N - 16 + row);
          if (a.mask != nullptr && vis && head_ok) {
            const float mv = TR::to_float(((const T*)a.mask)[(((size_t)b * a.Hq + hq) * 16 + row) * N + n]);
            vis = mv >= fmin_t;
            v += mv * kLog2e;
          }
          if (!vis) v = -INFINITY;
        }
        s[j][e] = v;
      }
      mx_lo = fmaxf(mx_lo, fmaxf(s[j][0], s[j][1]));
      mx_hi = fmaxf(mx_hi, fmaxf(s[j][2], s[j][3]));
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    // a row that has seen no visible key keeps max = -inf; use 0 as the reference point so exp2 stays finite
    const float ref_lo = (mn_lo == -INFINITY) ? 0.f : mn_lo, ref_hi = (mn_hi == -INFINITY) ? 0.f : mn_hi;
    const float f_lo = exp2f(m_lo - ref_lo), f_hi = exp2f(m_hi - ref_hi);
    m_lo = mn_lo; m_hi = mn_hi;
    float sum_lo = 0.f, sum_hi = 0.f;
    uint32_t p[kBN / 8][2];
#pragma unroll
    for (int j = 0; j < kBN / 8; ++j) {
      const float p0 = exp2f(s[j][0] - ref_lo), p1 = exp2f(s[j][1] - ref_lo);
      const float p2 = exp2f(s[j][2] - ref_hi), p3 = exp2f(s[j][3] - ref_hi);
      sum_lo += p0 + p1;
      sum_hi += p2 + p3;
      p[j][0] = pack2<T>(p0, p1);
      p[j][1] = pack2<T>(p2, p3);
    }
    l_lo = l_lo * f_lo + sum_lo;
    l_hi = l_hi * f_hi + sum_hi;
#pragma unroll
    for (int i = 0; i < NT_O; ++i) {
      o[i][0] *= f_lo; o[i][1] *= f_lo;
      o[i][2] *= f_hi; o[i][3] *= f_hi;
    }

    // ---- O += P V ----
    const uint32_t vb = uV + buf * kBN * RB;
#pragma unroll
    for (int kk = 0; kk < kBN / 16; ++kk) {
      const uint32_t pa0 = p[2 * kk][0], pa1 = p[2 * kk][1], pa2 = p[2 * kk + 1][0], pa3 = p[2 * kk + 1][1];
#pragma unroll
      for (int ip = 0; ip < NT_O / 2; ++ip) {
        // V^T fragments of two d tiles: matrices (keys 16kk..+7, chunk 2ip), (keys +8.., 2ip), (keys .., 2ip+1), (keys +8.., 2ip+1)
        const int r = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        const int ch = 2 * ip + (lane >> 4);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_trans(vb + swz(r, ch, RB), b0, b1, b2, b3);
        TR::mma(o[2 * ip], pa0, pa1, pa2, pa3, b0, b1);
        TR::mma(o[2 * ip + 1], pa0, pa1, pa2, pa3, b2, b3);
      }
    }
    __syncthreads();  // everyone is done with this buffer before the next prefetch overwrites it
  }
  cp_async_wait<0>();

  // ---- row sums across the quad, then write ----
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  if (!head_ok) return;
  const size_t row_lo = ((size_t)b * a.Hq + hq) * 16 + g, row_hi = row_lo + 8;
  if (a.splits == 1) {
    const float inv_lo = l_lo == 0.f ? 1.f : 1.f / l_lo, inv_hi = l_hi == 0.f ? 1.f : 1.f / l_hi;
    T* out = (T*)a.out;
#pragma unroll
    for (int i = 0; i < NT_O; ++i) {
      *(uint32_t*)(out + row_lo * D + 8 * i + 2 * c) = pack2<T>(o[i][0] * inv_lo, o[i][1] * inv_lo);
      *(uint32_t*)(out + row_hi * D + 8 * i + 2 * c) = pack2<T>(o[i][2] * inv_hi, o[i][3] * inv_hi);
    }
    return;
  }
  float* po_lo = a.part_o + (row_lo * a.splits + split) * D;
  float* po_hi = a.part_o + (row_hi * a.splits + split) * D;
#pragma unroll
  for (int i = 0; i < NT_O; ++i) {
    *(float2*)(po_lo + 8 * i + 2 * c) = make_float2(o[i][0], o[i][1]);
    *(float2*)(po_hi + 8 * i + 2 * c) = make_float2(o[i][2], o[i][3]);
  }
  if (c == 0) {
    a.part_m[row_lo * a.splits + split] = m_lo;
    a.part_l[row_lo * a.splits + split] = l_lo;
    a.part_m[row_hi * a.splits + split] = m_hi;
    a.part_l[row_hi * a.splits + split] = l_hi;
  }
}

// One CTA per (head, row), one thread per output channel: out = sum_s w_s O_s / sum_s w_s l_s with
// w_s = exp2(m_s - max_s m_s).  The weights are computed once into shared memory; the channel loop then reads the
// partials with fully coalesced, independent loads.
template <typename T, int D>
__global__ void __launch_bounds__(D) sdpa_combine_kernel(const SdpaArgs a, int rows) {
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
  const float* po = a.part_o + (size_t)row * a.splits * D + tid;
  float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
  int s = 0;
  for (; s + 4 <= a.splits; s += 4) {
    const float v0 = po[(size_t)s * D], v1 = po[(size_t)(s + 1) * D], v2 = po[(size_t)(s + 2) * D], v3 = po[(size_t)(s + 3) * D];
    acc0 = fmaf(sw[s], v0, acc0); acc1 = fmaf(sw[s + 1], v1, acc1);
    acc2 = fmaf(sw[s + 2], v2, acc2); acc3 = fmaf(sw[s + 3], v3, acc3);
  }
  for (; s < a.splits; ++s) acc0 = fmaf(sw[s], po[(size_t)s * D], acc0);
  const float den_all = sden;
  const float inv = den_all == 0.f ? 1.f : 1.f / den_all;  // a row with no visible key yields zeros (kernels.py:630)
  ((T*)a.out)[(size_t)row * D + tid] = MmaTraits<T>::from_float(((acc0 + acc1) + (acc2 + acc3)) * inv);
}

int choose_splits(int N, int ctas_per_split_unit, int device, int requested, int* blocks_per_split) {
  const int nblk = (N + kBN - 1) / kBN;
  int splits = requested > 0 ? requested : sm_count(device) / (ctas_per_split_unit > 0 ? ctas_per_split_unit : 1);
  if (splits < 1) splits = 1;
  if (splits > nblk) splits = nblk;
  if (splits > 1024) splits = 1024;
  const int bps = (nblk + splits - 1) / splits;
  *blocks_per_split = bps;
  return (nblk + bps - 1) / bps;
}

template <typename T, int D>
int launch(SdpaArgs a, void* ws, size_t ws_bytes, int requested_splits, cudaStream_t st) {
  int device = 0;
  cudaGetDevice(&device);
  const int nwarps = a.gqa < 8 ? a.gqa : 8;
  const int zg = (a.gqa + nwarps - 1) / nwarps;
  a.splits = choose_splits(a.N, a.B * a.Hk * zg, device, requested_splits, &a.blocks_per_split);
  const size_t rows = (size_t)a.B * a.Hq * 16;
  if (a.splits > 1) {
    const size_t need = rows * a.splits * (D + 2) * sizeof(float);
    if (!ws || ws_bytes < need) return fail(DFLASH_ERR_WORKSPACE, "verify_sdpa needs %zu workspace bytes, got %zu", need, ws_bytes);
    if ((uintptr_t)ws & 15) return fail(DFLASH_ERR_MISALIGNED, "verify_sdpa workspace must be 16-byte aligned");
    a.part_o = (float*)ws;
    a.part_m = a.part_o + rows * a.splits * D;
    a.part_l = a.part_m + rows * a.splits;
  }
  const size_t smem = (size_t)nwarps * 16 * D * 2 + 4 * (size_t)kBN * D * 2;
  static bool attr_done[64] = {};
  auto kern = sdpa_partials_kernel<T, D>;
  if (!attr_done[device & 63]) {
    cudaError_t e0 = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(8 * 16 * D * 2 + 4 * kBN * D * 2));
    if (e0 != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e0));
    attr_done[device & 63] = true;
  }
  dim3 grid(a.splits, a.B * a.Hk, zg);
  cudaError_t e = launch_kernel(kern, grid, dim3(nwarps * 32), smem, st, a);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "sdpa partials launch: %s", cudaGetErrorString(e));
  if (a.splits > 1) {
    e = launch_kernel(sdpa_combine_kernel<T, D>, dim3((unsigned)rows), dim3(D), 0, st, a, (int)rows);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "sdpa combine launch: %s", cudaGetErrorString(e));
  }
  return DFLASH_OK;
}

}  // namespace
}  // namespace dflash

using namespace dflash;

static int g_sdpa_impl = 0;
/* Kernel choice: 0 (default) = the tcgen05 kernel (csrc/sdpa_tc.cu) where it applies - bf16, no mask array, automatic
 * split count, at most 8 query heads per KV head - else the mma.sync kernel; 1 = the mma.sync kernel always. */
extern "C" void dflash_verify_sdpa_set_impl(int impl) {
  g_sdpa_impl = impl == 1 ? 1 : 0;
  sdpa_tc::set_fuse_combine(impl == 2 ? 1 : 0);   // 2 = the tcgen05 kernel with the combine pass inside the same launch
  sdpa_tc::set_split128(impl == 3 ? 1 : 0);       // 3 = the tcgen05 kernel with 128 keys per block while the grid fits the SMs
}

extern "C" size_t dflash_verify_sdpa_workspace_bytes(int B, int Hq, int Hk, int N, int D, int num_splits) {
  if (B < 1 || Hq < 1 || Hk < 1 || N < 1 || Hq % Hk != 0) return 0;
  int device = 0;
  cudaGetDevice(&device);
  const int gqa = Hq / Hk, nwarps = gqa < 8 ? gqa : 8, zg = (gqa + nwarps - 1) / nwarps;
  int bps;
  const int splits = choose_splits(N, B * Hk * zg, device, num_splits, &bps);
  size_t need = (size_t)B * Hq * 16 * splits * (D + 2) * sizeof(float) + 256;
  if (num_splits == 0) {   // either kernel may run: enough for both
    const size_t tc = sdpa_tc::workspace_bytes(B, Hq, N, D);
    if (tc > need) need = tc;
  }
  return need;
}

static int verify_sdpa_impl(const void* q, const void* k, const void* v, const void* mask, void* out, int B, int Hq,
                            int Hk, int N, int D, long long k_head_stride, long long k_seq_stride,
                            long long v_head_stride, long long v_seq_stride, float scale, int dtype,
                            int num_splits, void* workspace, size_t workspace_bytes, void* stream, const int* n_dev) {
  if (!q || !k || !v || !out) return fail(DFLASH_ERR_BAD_ARG, "verify_sdpa: null operand");
  if (B < 1 || Hq < 1 || Hk < 1 || Hq % Hk != 0) return fail(DFLASH_ERR_BAD_SHAPE, "verify_sdpa: bad head counts");
  if (N < 16) return fail(DFLASH_ERR_BAD_SHAPE, "verify_sdpa: N=%d must include the 16 query positions", N);
  if (D != 128 && D != 256) return fail(DFLASH_ERR_BAD_SHAPE, "verify_sdpa: D=%d not in {128,256}", D);
  if ((long long)B * Hk > 65535) return fail(DFLASH_ERR_BAD_SHAPE, "verify_sdpa: B*Hk too large");
  if (((uintptr_t)q & 15) || ((uintptr_t)k & 15) || ((uintptr_t)v & 15) || ((uintptr_t)out & 15) ||
      (k_seq_stride % 8) || (v_seq_stride % 8) || (k_head_stride % 8) || (v_head_stride % 8))
    return fail(DFLASH_ERR_MISALIGNED, "verify_sdpa: q/k/v/out rows must be 16-byte aligned");
  SdpaArgs a{};
  a.q = q; a.k = k; a.v = v; a.mask = mask; a.out = out;
  a.B = B; a.Hq = Hq; a.Hk = Hk; a.N = N; a.gqa = Hq / Hk;
  a.k_head_stride = k_head_stride; a.k_seq_stride = k_seq_stride;
  a.v_head_stride = v_head_stride; a.v_seq_stride = v_seq_stride;
  a.scale_log2 = scale * kLog2e;
  a.n_dev = n_dev;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == DFLASH_BF16 && mask == nullptr && num_splits == 0 && g_sdpa_impl == 0) {
    const int rc = sdpa_tc::launch(q, k, v, out, B, Hq, Hk, N, D, k_head_stride, k_seq_stride, v_head_stride, v_seq_stride,
                                   a.scale_log2, n_dev, workspace, workspace_bytes, st);
    if (rc <= 0) return rc;
  }
  if (dtype == DFLASH_BF16)
    return D == 128 ? launch<__nv_bfloat16, 128>(a, workspace, workspace_bytes, num_splits, st)
                    : launch<__nv_bfloat16, 256>(a, workspace, workspace_bytes, num_splits, st);
  if (dtype == DFLASH_F16)
    return D == 128 ? launch<__half, 128>(a, workspace, workspace_bytes, num_splits, st)
                    : launch<__half, 256>(a, workspace, workspace_bytes, num_splits, st);
  return fail(DFLASH_ERR_BAD_ARG, "verify_sdpa: dtype %d (want bf16 or f16)", dtype);
}

extern "C" int dflash_verify_sdpa(const void* q, const void* k, const void* v, const void* mask, void* out, int B, int Hq,
                                  int Hk, int N, int D, long long k_head_stride, long long k_seq_stride,
                                  long long v_head_stride, long long v_seq_stride, float scale, int dtype,
                                  int num_splits, void* workspace, size_t workspace_bytes, void* stream) {
  return verify_sdpa_impl(q, k, v, mask, out, B, Hq, Hk, N, D, k_head_stride, k_seq_stride, v_head_stride, v_seq_stride,
                          scale, dtype, num_splits, workspace, workspace_bytes, stream, nullptr);
}

extern "C" int dflash_verify_sdpa_dev_len(const void* q, const void* k, const void* v, void* out, int B, int Hq, int Hk,
                                          int N_max, const int* n_dev, int D, long long k_head_stride,
                                          long long k_seq_stride, long long v_head_stride, long long v_seq_stride,
                                          float scale, int dtype, int num_splits, void* workspace, size_t workspace_bytes,
                                          void* stream) {
  if (!n_dev) return fail(DFLASH_ERR_BAD_ARG, "verify_sdpa_dev_len: n_dev is NULL");
  return verify_sdpa_impl(q, k, v, nullptr, out, B, Hq, Hk, N_max, D, k_head_stride, k_seq_stride, v_head_stride,
                          v_seq_stride, scale, dtype, num_splits, workspace, workspace_bytes, stream, n_dev);
}

// ------------------------------------------------------------------------------------------------
// Variant for callers that must not allocate: the split-KV partials live in a fixed array inside the library.
namespace {
constexpr size_t kStaticScratchBytes = 32u << 20;
static __device__ __align__(256) unsigned char g_sdpa_static_scratch[kStaticScratchBytes];
void* g_static_scratch_ptr[64] = {};  // device address of the array, per device (host code cannot use the symbol itself)
std::mutex g_static_mu;
}  // namespace

extern "C" size_t dflash_verify_sdpa_static_capacity(void) { return kStaticScratchBytes; }

extern "C" int dflash_verify_sdpa_static(const void* q, const void* k, const void* v, const void* mask, void* out, int B,
                                         int Hq, int Hk, int N, int D, long long k_head_stride, long long k_seq_stride,
                                         long long v_head_stride, long long v_seq_stride, float scale, int dtype,
                                         int num_splits, void* stream) {
  if (B < 1 || Hq < 1 || Hk < 1 || Hq % Hk != 0 || N < 16 || (D != 128 && D != 256))
    return fail(DFLASH_ERR_BAD_SHAPE, "verify_sdpa_static: unsupported shape");
  const size_t need = dflash_verify_sdpa_workspace_bytes(B, Hq, Hk, N, D, num_splits);
  if (need > kStaticScratchBytes)
    return fail(DFLASH_ERR_WORKSPACE,
                "verify_sdpa_static: this shape needs %zu bytes of split-KV scratch but the built-in array holds %zu; "
                "pass a smaller num_splits or use dflash_verify_sdpa with a caller workspace",
                need, (size_t)kStaticScratchBytes);
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (device < 0 || device >= 64) return fail(DFLASH_ERR_UNSUPPORTED, "verify_sdpa_static: device index %d", device);
  void* scratch = nullptr;
  {
    // one-time set-up on this device (it is current): resolve the array's device address; the lock makes a first
    // call from two host threads safe
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (g_static_scratch_ptr[device] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_sdpa_static_scratch);
      if (e != cudaSuccess || p == nullptr)
        return fail(DFLASH_ERR_LAUNCH, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
      g_static_scratch_ptr[device] = p;
    }
    scratch = g_static_scratch_ptr[device];
  }
  return dflash_verify_sdpa(q, k, v, mask, out, B, Hq, Hk, N, D, k_head_stride, k_seq_stride, v_head_stride,
                            v_seq_stride, scale, dtype, num_splits, scratch, kStaticScratchBytes, stream);
}
