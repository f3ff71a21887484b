// GatedDeltaNet verify kernels for sm_100a: forward-with-tape (tape record) and tape replay.
//
// Replaces the Metal kernels `gated_delta_tape*` and `tape_replay*` (dflash_mlx/kernels.py:29-105, 244-294).
// Step order (kernels.py:62-99):  S *= g_t ; kv = S k_t ; delta = (v_t - kv) beta_t ; S += delta (x) k_t ;
// y_t = S q_t ; [round S to the state dtype].  Replay (kernels.py:273-288): S *= g_t ; S += delta_t (x) k_t.
//
// Layout: state [B, Hv, Dv, Dk] (row = dv, contiguous in dk).  One warp owns whole state rows: lane l holds
// dk in [NPT*l, NPT*l + NPT) (NPT = Dk/32), so a row is one coalesced 128-bit access per lane for Dk = 128,
// and the two per-step row reductions are warp shuffles.  A CTA of 4 warps owns 16 rows of one (batch, head);
// the step inputs of that head (q, k, gate as fp32, v rows, beta) are staged in shared memory 16 steps at a time.
// The kernels are pure streaming (state in + state out dominate): HBM bound.
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "gdn_step.cuh"

namespace dflash {
namespace {

constexpr int kRowsPerWarp = 4;
constexpr int kWarps = 4;
constexpr int kRowsPerCta = kRowsPerWarp * kWarps;

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <> __device__ __forceinline__ float ldf<__half>(const __half* p) { return __half2float(*p); }
template <typename T> __device__ __forceinline__ T cvt(float v);
template <> __device__ __forceinline__ float cvt<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 cvt<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half cvt<__half>(float v) { return __float2half_rn(v); }
template <typename T> __device__ __forceinline__ float round_to(float v);
template <> __device__ __forceinline__ float round_to<float>(float v) { return v; }
template <> __device__ __forceinline__ float round_to<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
template <> __device__ __forceinline__ float round_to<__half>(float v) { return __half2float(__float2half_rn(v)); }

template <typename ST, int NPT>
__device__ __forceinline__ void load_row(const ST* p, float (&s)[NPT]) {
  if constexpr (sizeof(ST) == 4 && NPT == 4) {
    const float4 v = *(const float4*)p;
    s[0] = v.x; s[1] = v.y; s[2] = v.z; s[3] = v.w;
  } else if constexpr (sizeof(ST) == 4 && NPT == 8) {
    const float4 a = ((const float4*)p)[0], b = ((const float4*)p)[1];
    s[0] = a.x; s[1] = a.y; s[2] = a.z; s[3] = a.w; s[4] = b.x; s[5] = b.y; s[6] = b.z; s[7] = b.w;
  } else {
#pragma unroll
    for (int i = 0; i < NPT; ++i) s[i] = ldf<ST>(p + i);
  }
}
template <typename ST, int NPT>
__device__ __forceinline__ void store_row(ST* p, const float (&s)[NPT]) {
  if constexpr (sizeof(ST) == 4 && NPT == 4) {
    *(float4*)p = make_float4(s[0], s[1], s[2], s[3]);
  } else if constexpr (sizeof(ST) == 4 && NPT == 8) {
    ((float4*)p)[0] = make_float4(s[0], s[1], s[2], s[3]);
    ((float4*)p)[1] = make_float4(s[4], s[5], s[6], s[7]);
  } else {
#pragma unroll
    for (int i = 0; i < NPT; ++i) p[i] = cvt<ST>(s[i]);
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct GdnArgs {
  const void* q; const void* k; const void* v; const float* g; const float* beta; const uint8_t* mask;
  const void* state_in; void* state_out; void* y; float* tape; const float* tape_in;
  const int* steps_dev;
  int B, T, steps, Hk, Hv, Dk, Dv, g_is_vector;
  int vec_ok;  // q and k start on 16-byte boundaries: their rows are staged with 16-byte loads
  int early_state;  // the record kernel may read state_in before it waits for the previous kernel
};

// RECORD = true : forward with tape.  RECORD = false : replay of `steps` tape entries.
template <typename IT, typename ST, int NPT, bool RECORD>
__global__ void __launch_bounds__(kWarps * 32) gdn_kernel(const GdnArgs a) {
  constexpr int Dk = NPT * 32;
  constexpr int kStepChunk = (NPT == 8) ? 8 : 16;  // keeps the static shared memory under 48 KB
  constexpr int kThreads = kWarps * 32;
  constexpr int kElemPerVec = 16 / (int)sizeof(IT), kVecPerRow = Dk / kElemPerVec;   // 16-byte vectors of a q / k row
  constexpr int kVecPerThread = (kStepChunk * kVecPerRow + kThreads - 1) / kThreads;
  constexpr int kValPerThread = (kStepChunk * kRowsPerCta + kThreads - 1) / kThreads;
  pdl_wait();
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y, b = bh / a.Hv, hv = bh % a.Hv, hk = hv / (a.Hv / a.Hk);
  const int row0 = blockIdx.x * kRowsPerCta + warp * kRowsPerWarp;
  int steps = a.steps;
  if (!RECORD && a.steps_dev != nullptr) steps = min(max(*a.steps_dev, 0), a.T);

  __shared__ float sk[kStepChunk][Dk];
  __shared__ float sq[RECORD ? kStepChunk : 1][Dk];
  __shared__ float sgv[kStepChunk][Dk];                 // vector gate only
  __shared__ float sv[kStepChunk][kRowsPerCta];         // v rows (record) or tape rows (replay)
  __shared__ float sg[kStepChunk], sb[kStepChunk];
  __shared__ int sm[kStepChunk];

  float S[kRowsPerWarp][NPT];
  const ST* sin = (const ST*)a.state_in + ((size_t)bh * a.Dv) * Dk;
  ST* sout = (ST*)a.state_out + ((size_t)bh * a.Dv) * Dk;
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    if (row0 + r < a.Dv) load_row<ST, NPT>(sin + (size_t)(row0 + r) * Dk + NPT * lane, S[r]);
    else
#pragma unroll
      for (int i = 0; i < NPT; ++i) S[r][i] = 0.f;
  }

  const IT* qg = (const IT*)a.q;
  const IT* kg = (const IT*)a.k;
  const IT* vg = (const IT*)a.v;
  IT* yg = (IT*)a.y;

  for (int t0 = 0; t0 < steps; t0 += kStepChunk) {
    const int nt = min(kStepChunk, steps - t0);
    __syncthreads();
    // Every global load of the chunk is issued before the first loaded value is used, so the chunk costs one memory
    // latency (a load-convert-store loop pays one per iteration: a warp issues in order and stalls at the convert).
    uint4 kvec[kVecPerThread], qvec[kVecPerThread];
    float vreg[kValPerThread];
    float g_r = 1.f, b_r = 0.f;
    int m_r = 1;
    if (a.vec_ok) {
#pragma unroll
      for (int u = 0; u < kVecPerThread; ++u) {
        const int i = u * kThreads + (int)threadIdx.x;
        if (i < nt * kVecPerRow) {
          const int t = i / kVecPerRow, c = i % kVecPerRow;
          const size_t kq = (((size_t)b * a.T + t0 + t) * a.Hk + hk) * Dk + (size_t)c * kElemPerVec;
          kvec[u] = *(const uint4*)(kg + kq);
          if (RECORD) qvec[u] = *(const uint4*)(qg + kq);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kValPerThread; ++u) {
      const int i = u * kThreads + (int)threadIdx.x;
      const int t = i / kRowsPerCta, r = i % kRowsPerCta;
      const int row = blockIdx.x * kRowsPerCta + r;
      vreg[u] = 0.f;
      if (t < nt && row < a.Dv) {
        const size_t idx = (((size_t)b * a.T + t0 + t) * a.Hv + hv) * a.Dv + row;
        vreg[u] = RECORD ? ldf<IT>(vg + idx) : a.tape_in[idx];
      }
    }
    if (threadIdx.x < nt) {
      const size_t idx = ((size_t)b * a.T + t0 + threadIdx.x) * a.Hv + hv;
      if (!a.g_is_vector) g_r = a.g[idx];
      if (RECORD) b_r = a.beta[idx];
      if (a.mask) m_r = (int)a.mask[(size_t)b * a.T + t0 + threadIdx.x];
    }
    if (a.vec_ok) {
#pragma unroll
      for (int u = 0; u < kVecPerThread; ++u) {
        const int i = u * kThreads + (int)threadIdx.x;
        if (i < nt * kVecPerRow) {
          const int t = i / kVecPerRow, c = i % kVecPerRow;
          const IT* ke = (const IT*)&kvec[u];
          const IT* qe = (const IT*)&qvec[u];
#pragma unroll
          for (int j = 0; j < kElemPerVec; ++j) {
            sk[t][c * kElemPerVec + j] = ldf<IT>(ke + j);
            if (RECORD) sq[t][c * kElemPerVec + j] = ldf<IT>(qe + j);
          }
        }
      }
    } else {
      for (int i = threadIdx.x; i < nt * Dk; i += kThreads) {
        const int t = i / Dk, d = i % Dk;
        const size_t kq = (((size_t)b * a.T + t0 + t) * a.Hk + hk) * Dk + d;
        sk[t][d] = ldf<IT>(kg + kq);
        if (RECORD) sq[t][d] = ldf<IT>(qg + kq);
      }
    }
    if (a.g_is_vector) {
      for (int i = threadIdx.x; i < nt * Dk; i += kThreads) {
        const int t = i / Dk, d = i % Dk;
        sgv[t][d] = a.g[(((size_t)b * a.T + t0 + t) * a.Hv + hv) * Dk + d];
      }
    }
#pragma unroll
    for (int u = 0; u < kValPerThread; ++u) {
      const int i = u * kThreads + (int)threadIdx.x;
      if (i / kRowsPerCta < nt) sv[i / kRowsPerCta][i % kRowsPerCta] = vreg[u];
    }
    if (threadIdx.x < nt) {
      sg[threadIdx.x] = g_r;
      sb[threadIdx.x] = b_r;
      sm[threadIdx.x] = m_r;
    }
    __syncthreads();

    for (int t = 0; t < nt; ++t) {
      const bool on = sm[t] != 0;
      float kk[NPT], gg[NPT];
#pragma unroll
      for (int i = 0; i < NPT; ++i) {
        kk[i] = sk[t][NPT * lane + i];
        gg[i] = a.g_is_vector ? sgv[t][NPT * lane + i] : sg[t];
      }
      if (RECORD) {
        float qq[NPT];
#pragma unroll
        for (int i = 0; i < NPT; ++i) qq[i] = sq[t][NPT * lane + i];
        float kv[kRowsPerWarp], yy[kRowsPerWarp], dl[kRowsPerWarp];
        if (on) {
#pragma unroll
          for (int r = 0; r < kRowsPerWarp; ++r) {
            float p = 0.f;
#pragma unroll
            for (int i = 0; i < NPT; ++i) {
              S[r][i] *= gg[i];
              p = fmaf(S[r][i], kk[i], p);
            }
            kv[r] = p;
          }
#pragma unroll
          for (int r = 0; r < kRowsPerWarp; ++r) kv[r] = warp_sum(kv[r]);
          const float beta = sb[t];
#pragma unroll
          for (int r = 0; r < kRowsPerWarp; ++r) {
            dl[r] = (sv[t][warp * kRowsPerWarp + r] - kv[r]) * beta;
            float p = 0.f;
#pragma unroll
            for (int i = 0; i < NPT; ++i) {
              S[r][i] = fmaf(kk[i], dl[r], S[r][i]);
              p = fmaf(S[r][i], qq[i], p);
            }
            yy[r] = p;
          }
#pragma unroll
          for (int r = 0; r < kRowsPerWarp; ++r) yy[r] = warp_sum(yy[r]);
        } else {
#pragma unroll
          for (int r = 0; r < kRowsPerWarp; ++r) { dl[r] = 0.f; yy[r] = 0.f; }
        }
        // the state is rounded to its storage dtype after every step, masked or not (kernels.py:89-91)
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
          for (int i = 0; i < NPT; ++i) S[r][i] = round_to<ST>(S[r][i]);
        if (lane < kRowsPerWarp) {
          // lane r writes row r (select without dynamic register indexing)
          float yv = yy[0], dv = dl[0];
#pragma unroll
          for (int r = 1; r < kRowsPerWarp; ++r)
            if (lane == r) { yv = yy[r]; dv = dl[r]; }
          const int row = row0 + lane;
          if (row < a.Dv) {
            const size_t idx = (((size_t)b * a.T + t0 + t) * a.Hv + hv) * a.Dv + row;
            yg[idx] = cvt<IT>(yv);
            a.tape[idx] = dv;
          }
        }
      } else {
        if (on) {
#pragma unroll
          for (int r = 0; r < kRowsPerWarp; ++r) {
            const float dl = sv[t][warp * kRowsPerWarp + r];
#pragma unroll
            for (int i = 0; i < NPT; ++i) {
              S[r][i] *= gg[i];
              S[r][i] = fmaf(kk[i], dl, S[r][i]);
              S[r][i] = round_to<ST>(S[r][i]);  // only inside the masked-in branch (kernels.py:274-284)
            }
          }
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r)
    if (row0 + r < a.Dv) store_row<ST, NPT>(sout + (size_t)(row0 + r) * Dk + NPT * lane, S[r]);
}

// ---- tape replay as a pure stream (the common case: scalar gate, no mask, fp32 state, Dk = 128, bf16 k) ----------------
// S = S * g_t + k_t (x) delta_t over the committed steps is element-wise in S: no reductions, so the kernel is a copy of
// the state with 2 x steps flops per element in between.  One block = 64 rows of one (layer, head): 8 warps x 8 rows, a
// lane holds 4 key channels of each of its rows (32 floats), every row a 16-byte load per lane.  The step inputs of the
// head (k as fp32, the 64 tape rows, the gates: 12 KB) are staged once per block.  Arithmetic is the packed fp32 pair
// form (mul.f32x2 / fma.rn.f32x2: IEEE per element, so the bits equal the record kernel's), which halves the issue
// slots - with scalar FMAs the arithmetic would take as long as the memory traffic.
constexpr int kFastRows = 64, kFastWarps = 8, kFastT = 16;

using gdnstep::pack2;
using gdnstep::unpack2;
using gdnstep::mul2;
using gdnstep::fma2;

__global__ void __launch_bounds__(kFastWarps * 32, 4) tape_replay_stream_kernel(const GdnArgs a) {
  constexpr int Dk = 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y, b = bh / a.Hv, hv = bh % a.Hv, hk = hv / (a.Hv / a.Hk);
  const int row_base = blockIdx.x * kFastRows, row0 = row_base + warp * 8;
  __shared__ float sk[kFastT][Dk];
  __shared__ float sd[kFastT][kFastRows];
  __shared__ float sg[kFastT];
  // the state rows are nobody's output in this stream position: requested before the wait on the previous kernel
  const float* sin = (const float*)a.state_in + ((size_t)bh * a.Dv) * Dk;
  float* sout = (float*)a.state_out + ((size_t)bh * a.Dv) * Dk;
  unsigned long long S[8][2];
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row0 + r < a.Dv) v = *(const float4*)(sin + (size_t)(row0 + r) * Dk + 4 * lane);
    S[r][0] = pack2(v.x, v.y);
    S[r][1] = pack2(v.z, v.w);
  }
  pdl_wait();
  pdl_trigger();
  int steps = a.steps;
  if (a.steps_dev != nullptr) steps = min(max(*a.steps_dev, 0), a.T);
  const __nv_bfloat16* kg = (const __nv_bfloat16*)a.k;
  for (int t0 = 0; t0 < steps; t0 += kFastT) {
    const int nt = min(kFastT, steps - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * Dk / 2; i += kFastWarps * 32) {  // two bf16 per load
      const int t = i / (Dk / 2), d2 = i % (Dk / 2);
      const __nv_bfloat162 v = *(const __nv_bfloat162*)(kg + (((size_t)b * a.T + t0 + t) * a.Hk + hk) * Dk + 2 * d2);
      sk[t][2 * d2] = __bfloat162float(v.x);
      sk[t][2 * d2 + 1] = __bfloat162float(v.y);
    }
    for (int i = threadIdx.x; i < nt * kFastRows; i += kFastWarps * 32) {
      const int t = i / kFastRows, r = i % kFastRows, row = row_base + r;
      sd[t][r] = row < a.Dv ? a.tape_in[(((size_t)b * a.T + t0 + t) * a.Hv + hv) * a.Dv + row] : 0.f;
    }
    if (threadIdx.x < nt) sg[threadIdx.x] = a.g[((size_t)b * a.T + t0 + threadIdx.x) * a.Hv + hv];
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float g = sg[t];
      const unsigned long long gg = pack2(g, g);
      const float4 kv = *(const float4*)&sk[t][4 * lane];
      const unsigned long long k01 = pack2(kv.x, kv.y), k23 = pack2(kv.z, kv.w);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float d = sd[t][warp * 8 + r];
        const unsigned long long dd = pack2(d, d);
        S[r][0] = fma2(k01, dd, mul2(S[r][0], gg));   // S *= g ; S += k * delta (kernels.py:273-288), two roundings
        S[r][1] = fma2(k23, dd, mul2(S[r][1], gg));
      }
    }
  }
#pragma unroll
  for (int r = 0; r < 8; ++r)
    if (row0 + r < a.Dv) {
      float4 v;
      unpack2(S[r][0], v.x, v.y);
      unpack2(S[r][1], v.z, v.w);
      *(float4*)(sout + (size_t)(row0 + r) * Dk + 4 * lane) = v;
    }
}

// ---- the same stream, software-pipelined: one persistent block per SM --------------------------------------------------
// The kernel above has nothing in flight while a block computes, so with 4 blocks per SM only about half of the bytes the
// memory system needs outstanding are requested at any time.  Here a producer warp runs kPipeStages tiles ahead with bulk
// copies (cp.async.bulk: a tile's 32 KB of state and its 16 + 16 rows of k and tape land in shared memory and complete
// on an mbarrier), and two groups of 8 warps each take every other tile: registers <- shared memory, the steps, then the
// 16-byte stores.  Same arithmetic, same bits.  Every wait is bounded (device error code 41).
constexpr int kPipeStages = 5, kPipeGroups = 2;
constexpr int kPipeStateBytes = kFastRows * 128 * 4;   // 32 KB
constexpr int kPipeKBytes = kFastT * 128 * 2;          // k of the head, bf16
constexpr int kPipeTapeBytes = kFastT * kFastRows * 4;
constexpr int kPipeStageBytes = kPipeStateBytes + kPipeKBytes + kPipeTapeBytes + 128;  // + gates
constexpr int kPipeThreads = (kPipeGroups * kFastWarps + 1) * 32;
constexpr size_t kPipeSmem = (size_t)kPipeStages * kPipeStageBytes + 16 * kPipeStages;

__device__ __forceinline__ void tma_load_3d_plain(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
               "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
               : "memory");
}

__global__ void __launch_bounds__(kPipeThreads, 1) tape_replay_pipe_kernel(const GdnArgs a, int* __restrict__ err,
                                                                            const __grid_constant__ CUtensorMap tmK,
                                                                            const __grid_constant__ CUtensorMap tmTape) {
  constexpr int Dk = 128;
  extern __shared__ __align__(128) uint8_t smem[];   // used as is: the compiler then knows these are shared-memory loads
  uint64_t* bars = (uint64_t*)(smem + (size_t)kPipeStages * kPipeStageBytes);
  const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * kPipeStages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_blocks = (a.Dv + kFastRows - 1) / kFastRows;
  const int tiles = a.B * a.Hv * row_blocks;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kPipeStages; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, kFastWarps);
    }
    mbar_fence_init();
  }
  __syncthreads();
  if (warp == kPipeGroups * kFastWarps) {
    // ---------------- producer ----------------
    pdl_wait();   // k, tape and gates come from the kernels before this one
    int j = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++j) {
      const int stage = j % kPipeStages;
      const uint32_t par = ((j / kPipeStages) & 1) ^ 1;   // first use of a stage passes at once
      if (!mbar_wait_quiet(bar_empty + 8 * stage, par)) { if (lane == 0) atomicCAS(err, 0, 41 | (j << 8)); break; }
      const int bh = tile / row_blocks, rb = tile % row_blocks;
      const int b = bh / a.Hv, hv = bh % a.Hv, hk = hv / (a.Hv / a.Hk);
      const int row_base = rb * kFastRows, rows = min(kFastRows, a.Dv - row_base);
      uint8_t* st = smem + (size_t)stage * kPipeStageBytes;
      if (lane == 0) {
        const int T = min(a.T, kFastT);
        const uint32_t bytes = (uint32_t)rows * Dk * 4 + (uint32_t)T * (Dk * 2 + kFastRows * 4);
        const uint32_t full = bar_full + 8 * stage;
        mbar_arrive_expect_tx(full, bytes);
        bulk_load_1d(smem_u32(st), (const float*)a.state_in + ((size_t)bh * a.Dv + row_base) * Dk, (uint32_t)rows * Dk * 4, full);
        const __nv_bfloat16* kg = (const __nv_bfloat16*)a.k;
        // the head's k rows and the tile's tape rows of all T steps: one tiled copy each (32 small bulk copies took 8 us
        // of a 52 us launch); columns beyond Dv are filled with zeros
        tma_load_3d_plain(smem_u32(st + kPipeStateBytes), &tmK, 0, hk, b * a.T, full);
        tma_load_3d_plain(smem_u32(st + kPipeStateBytes + kPipeKBytes), &tmTape, row_base, hv, b * a.T, full);
      }
    }
  } else {
    // ---------------- consumers: group = warp / 8 takes this block's tiles j with j % 2 == group ----------------
    const int group = warp / kFastWarps, w = warp % kFastWarps;
    pdl_wait();   // the output buffer may still be read by the kernel before this one; the step count is its output
    pdl_trigger();
    int steps = a.steps;
    if (a.steps_dev != nullptr) steps = min(max(*a.steps_dev, 0), a.T);
    steps = min(steps, kFastT);
    int j = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++j) {
      if (j % kPipeGroups != group) continue;
      const int stage = j % kPipeStages;
      const uint32_t par = (j / kPipeStages) & 1;
      const int bh = tile / row_blocks, rb = tile % row_blocks;
      const int row_base = rb * kFastRows, row0 = row_base + w * 8;
      // lane t fetches the gate of step t (strided scalars: not worth a bulk copy) while the tile is still landing
      const float g_mine = lane < a.T ? a.g[((size_t)(bh / a.Hv) * a.T + lane) * a.Hv + (bh % a.Hv)] : 1.f;
      if (!mbar_wait_quiet(bar_full + 8 * stage, par)) { if (lane == 0) atomicCAS(err, 0, 41 | (j << 8)); break; }
      const uint8_t* st = smem + (size_t)stage * kPipeStageBytes;
      const float* ss = (const float*)st;
      const __nv_bfloat16* skb = (const __nv_bfloat16*)(st + kPipeStateBytes);
      const float* sd = (const float*)(st + kPipeStateBytes + kPipeKBytes);
      // fp32 pairs run ACROSS two rows of the same key channel: the two deltas of a row pair then sit next to each other
      // as they come from shared memory, and only the gate and the four k values have to be duplicated per step
      unsigned long long S[4][4];
#pragma unroll
      for (int rp = 0; rp < 4; ++rp) {
        const float4 va = *(const float4*)(ss + (size_t)(w * 8 + 2 * rp) * Dk + 4 * lane);
        const float4 vb = *(const float4*)(ss + (size_t)(w * 8 + 2 * rp + 1) * Dk + 4 * lane);
        S[rp][0] = pack2(va.x, vb.x); S[rp][1] = pack2(va.y, vb.y); S[rp][2] = pack2(va.z, vb.z); S[rp][3] = pack2(va.w, vb.w);
      }
#pragma unroll 4
      for (int t = 0; t < steps; ++t) {
        const float g = __shfl_sync(0xffffffffu, g_mine, t);
        const unsigned long long gg = pack2(g, g);
        const uint2 kb = *(const uint2*)(skb + t * Dk + 4 * lane);   // four bf16
        const float k0 = __uint_as_float(kb.x << 16), k1 = __uint_as_float(kb.x & 0xFFFF0000u);
        const float k2 = __uint_as_float(kb.y << 16), k3 = __uint_as_float(kb.y & 0xFFFF0000u);
        const unsigned long long kk[4] = {pack2(k0, k0), pack2(k1, k1), pack2(k2, k2), pack2(k3, k3)};
        const float4 d0 = *(const float4*)(sd + t * kFastRows + w * 8), d1 = *(const float4*)(sd + t * kFastRows + w * 8 + 4);
        const unsigned long long dp[4] = {pack2(d0.x, d0.y), pack2(d0.z, d0.w), pack2(d1.x, d1.y), pack2(d1.z, d1.w)};
#pragma unroll
        for (int rp = 0; rp < 4; ++rp)
#pragma unroll
          for (int i = 0; i < 4; ++i)
            S[rp][i] = fma2(kk[i], dp[rp], mul2(S[rp][i], gg));   // S *= g ; S += k * delta (kernels.py:273-288)
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_empty + 8 * stage);   // this warp has read all it needs from the stage
      float* sout = (float*)a.state_out + ((size_t)bh * a.Dv) * Dk;
#pragma unroll
      for (int rp = 0; rp < 4; ++rp) {
        float4 va, vb;
        unpack2(S[rp][0], va.x, vb.x); unpack2(S[rp][1], va.y, vb.y); unpack2(S[rp][2], va.z, vb.z); unpack2(S[rp][3], va.w, vb.w);
        if (row0 + 2 * rp < a.Dv) *(float4*)(sout + (size_t)(row0 + 2 * rp) * Dk + 4 * lane) = va;
        if (row0 + 2 * rp + 1 < a.Dv) *(float4*)(sout + (size_t)(row0 + 2 * rp + 1) * Dk + 4 * lane) = vb;
      }
    }
  }
}

// Tensor maps of the pipelined replay: k as [B*T][Hk][128] bf16 with a box of one head over all T steps, the tape as
// [B*T][Hv][Dv] fp32 with a box of 64 rows of one head over all T steps.  Cached per (pointer, shape).
struct ReplayMapKey {
  const void* p; int a, b, c, kind;
  bool operator==(const ReplayMapKey& o) const { return p == o.p && a == o.a && b == o.b && c == o.c && kind == o.kind; }
};
struct ReplayMapKeyHash {
  size_t operator()(const ReplayMapKey& k) const {
    return std::hash<const void*>()(k.p) ^ ((size_t)k.a * 1000003u) ^ ((size_t)k.b * 7919u) ^ ((size_t)k.c * 104729u) ^ (size_t)k.kind;
  }
};
std::mutex g_replay_mu;
std::unordered_map<ReplayMapKey, CUtensorMap, ReplayMapKeyHash> g_replay_maps;

bool get_replay_map(const void* ptr, int rows_bt, int heads, int inner, int T, int kind, CUtensorMap* out) {
  ReplayMapKey key{ptr, rows_bt, heads, inner * 32 + T, kind};
  {
    std::lock_guard<std::mutex> lk(g_replay_mu);
    auto it = g_replay_maps.find(key);
    if (it != g_replay_maps.end()) { *out = it->second; return true; }
  }
  tensormap_encode_fn enc = get_tensormap_encoder();
  if (!enc) return false;
  const size_t es = kind == 0 ? 2 : 4;
  cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)heads, (cuuint64_t)rows_bt};
  cuuint64_t strides[2] = {(cuuint64_t)inner * es, (cuuint64_t)heads * inner * es};
  cuuint32_t box[3] = {(cuuint32_t)(kind == 0 ? 128 : kFastRows), 1, (cuuint32_t)T};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMap m;
  CUresult r = enc(&m, kind == 0 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(ptr),
                   dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  std::lock_guard<std::mutex> lk(g_replay_mu);
  if (g_replay_maps.size() > 4096) g_replay_maps.clear();
  g_replay_maps.emplace(key, m);
  *out = m;
  return true;
}

// ---- tape record, the common case (scalar gate, no mask, fp32 state, Dk = 128, bf16 inputs, T <= 16) -------------------
// The recurrence is a chain of 16 dependent token steps, so the kernel is bound by the latency and the instruction count
// of one step, not by memory.  Against the general kernel above: (1) a state row is spread over 8 lanes (16 elements
// each) instead of 32, so a row reduction is 3 shuffle levels instead of 5 and a warp advances 4 rows with one
// instruction stream; (2) y_t = S_t q_t is computed as S' q_t + delta_t (k_t . q_t) with S' the decayed state BEFORE the
// update, so both row reductions of a step (S' k_t and S' q_t) run as one interleaved shuffle chain instead of two in
// sequence (k_t . q_t is one scalar per token, computed while the step inputs are staged); (3) packed fp32 pair
// arithmetic.  The state itself goes through the same two roundings per step as everywhere else (S *= g ; S += k delta),
// so a replay of the tape still reproduces it bit for bit.  Lane l = 8 * (row within the warp) + c holds the 16-byte
// chunks c, c + 8, c + 16, c + 24 of its row: global and shared accesses of 8 neighbouring lanes are contiguous.
constexpr int kRecT = 16, kRecRows = 16;
// NORM: the gated RMSNorm that consumes y (runtime.py:445 of dflash-mlx) runs in the same launch.  The Dv / 16 blocks of a
// head form one thread-block cluster and meet once, through distributed shared memory, to add up the 16-row partial
// sums of y^2 per token; out[t, hv*Dv + d] = bf16(bf16(y) * inv_rms * w[d]) * silu(z[t, hv*Dv + d]).
struct GdnNormArgs {
  const __nv_bfloat16* z; long long z_ld; int z_off;
  const __nv_bfloat16* w; __nv_bfloat16* out; long long out_ld; float eps;
};
__device__ __forceinline__ float bf_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <bool NORM>
__global__ void __launch_bounds__(128) gdn_record_fast_kernel(const GdnArgs a, const GdnNormArgs nm) {
  __shared__ __align__(16) float sk[kRecT][128];
  __shared__ __align__(16) float sq[kRecT][128];
  __shared__ float sv[kRecT][kRecRows];
  __shared__ float sg[kRecT], sb[kRecT], skq[kRecT];
  __shared__ float sy[NORM ? kRecT : 1][kRecRows], ssq_part[kRecT], sinv[kRecT];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, rsub = lane >> 3, cg = lane & 7;
  const int bh = blockIdx.y, b = bh / a.Hv, hv = bh % a.Hv, hk = hv / (a.Hv / a.Hk);
  const int row = blockIdx.x * kRecRows + warp * 4 + rsub;
  const bool row_ok = row < a.Dv;
  const int T = a.T;
  const __nv_bfloat16* qg = (const __nv_bfloat16*)a.q;
  const __nv_bfloat16* kg = (const __nv_bfloat16*)a.k;
  const __nv_bfloat16* vg = (const __nv_bfloat16*)a.v;

  // every global load is issued before the first use; when the caller vouches that the kernel launched before this one
  // does not write the state (dflash_gdn_forward_state_is_settled), its rows are requested before the wait on that kernel
  unsigned long long S2[8];
  const float* srow = (const float*)a.state_in + ((size_t)bh * a.Dv + (row_ok ? row : 0)) * 128;
  if (a.early_state) gdnstep::load_row8(srow, cg, row_ok, S2);
  pdl_wait();
  pdl_trigger();
  if (!a.early_state) gdnstep::load_row8(srow, cg, row_ok, S2);
  uint4 kvec[2], qvec[2];
  float vreg[2];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int i = u * 128 + tid, t = i >> 4, c = i & 15;        // 16 vectors of 8 elements per token row
    kvec[u] = make_uint4(0u, 0u, 0u, 0u);
    qvec[u] = make_uint4(0u, 0u, 0u, 0u);
    vreg[u] = 0.f;
    if (t < T) {
      const size_t kq = (((size_t)b * T + t) * a.Hk + hk) * 128 + (size_t)c * 8;
      kvec[u] = *(const uint4*)(kg + kq);
      qvec[u] = *(const uint4*)(qg + kq);
      const int vrow = blockIdx.x * kRecRows + c;                // c doubles as the row of the block for the v tile
      if (vrow < a.Dv) vreg[u] = __bfloat162float(vg[(((size_t)b * T + t) * a.Hv + hv) * a.Dv + vrow]);
    }
  }
  float g_r = 1.f, b_r = 0.f;
  if (tid < T) {
    const size_t idx = ((size_t)b * T + tid) * a.Hv + hv;
    g_r = a.g[idx];
    b_r = a.beta[idx];
  }
  // what the output norm needs from global memory is requested now, behind the recurrence
  float zpre[2] = {0.f, 0.f}, gwpre[2] = {0.f, 0.f};
  if constexpr (NORM) {
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int i = u * 128 + tid, t = i >> 4, vrow = blockIdx.x * kRecRows + (i & 15);
      if (t < T && vrow < a.Dv) {
        zpre[u] = __bfloat162float(nm.z[((size_t)b * T + t) * nm.z_ld + nm.z_off + hv * a.Dv + vrow]);
        gwpre[u] = __bfloat162float(nm.w[vrow]);
      }
    }
  }
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int i = u * 128 + tid, t = i >> 4, c = i & 15;
    const __nv_bfloat16* ke = (const __nv_bfloat16*)&kvec[u];
    const __nv_bfloat16* qe = (const __nv_bfloat16*)&qvec[u];
    float kf[8], qf[8], dot = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      kf[j] = __bfloat162float(ke[j]);
      qf[j] = __bfloat162float(qe[j]);
      dot = fmaf(kf[j], qf[j], dot);
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);   // the 16 lanes of one token row
    if (t < T) {
      *(float4*)&sk[t][c * 8] = make_float4(kf[0], kf[1], kf[2], kf[3]);
      *(float4*)&sk[t][c * 8 + 4] = make_float4(kf[4], kf[5], kf[6], kf[7]);
      *(float4*)&sq[t][c * 8] = make_float4(qf[0], qf[1], qf[2], qf[3]);
      *(float4*)&sq[t][c * 8 + 4] = make_float4(qf[4], qf[5], qf[6], qf[7]);
      sv[t][c] = vreg[u];
      if (c == 0) skq[t] = dot;
    }
  }
  if (tid < T) { sg[tid] = g_r; sb[tid] = b_r; }
  __syncthreads();

  __nv_bfloat16* yg = (__nv_bfloat16*)a.y;
  for (int t = 0; t < T; ++t) {
    float yv;
    const float dl = gdnstep::step(S2, sk[t], sq[t], cg, sg[t], sb[t], sv[t][warp * 4 + rsub], skq[t], yv);
    if (cg == 0) {
      if (row_ok) {
        const size_t idx = (((size_t)b * T + t) * a.Hv + hv) * a.Dv + row;
        if (yg != nullptr) yg[idx] = __float2bfloat16_rn(yv);
        a.tape[idx] = dl;
      }
      if constexpr (NORM) sy[t][warp * 4 + rsub] = row_ok ? bf_round(yv) : 0.f;   // y is a bf16 array in the reference
    }
  }
  if (row_ok) gdnstep::store_row8((float*)a.state_out + ((size_t)bh * a.Dv + row) * 128, cg, S2);
  if constexpr (NORM) {
    __syncthreads();
    if (tid < kRecT) {
      float sum = 0.f;
      if (tid < T) {
#pragma unroll
        for (int r = 0; r < kRecRows; ++r) sum += sy[tid][r] * sy[tid][r];
      }
      ssq_part[tid] = sum;
    }
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (tid < kRecT) {
      float part[8], total = 0.f;
      const uint32_t local = smem_u32(&ssq_part[tid]);
#pragma unroll
      for (unsigned rank = 0; rank < 8; ++rank) {  // all loads in flight together (a cluster has at most 8 blocks)
        part[rank] = 0.f;
        if (rank < gridDim.x) {
          uint32_t remote;
          asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
          asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(part[rank]) : "r"(remote));
        }
      }
#pragma unroll
      for (int rank = 0; rank < 8; ++rank) total += part[rank];  // fixed order: deterministic
      sinv[tid] = rsqrtf(total / (float)a.Dv + nm.eps);
    }
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");  // done reading the others' shared memory
    __syncthreads();
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int i = u * 128 + tid, t = i >> 4, r = i & 15, vrow = blockIdx.x * kRecRows + r;
      if (t < T && vrow < a.Dv) {
        const float n = bf_round(sy[t][r] * sinv[t] * gwpre[u]);
        const float z = zpre[u];
        nm.out[((size_t)b * T + t) * nm.out_ld + hv * a.Dv + vrow] = __float2bfloat16_rn(n * (z / (1.f + __expf(-z))));
      }
    }
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");  // nobody exits while a neighbour may still read
  }
}

template <typename IT, typename ST, bool RECORD>
int launch_npt(const GdnArgs& a, cudaStream_t st) {
  dim3 grid((a.Dv + kRowsPerCta - 1) / kRowsPerCta, a.B * a.Hv);
  cudaError_t e = cudaSuccess;
  switch (a.Dk / 32) {
    case 1: e = launch_kernel(gdn_kernel<IT, ST, 1, RECORD>, grid, dim3(kWarps * 32), 0, st, a); break;
    case 2: e = launch_kernel(gdn_kernel<IT, ST, 2, RECORD>, grid, dim3(kWarps * 32), 0, st, a); break;
    case 4: e = launch_kernel(gdn_kernel<IT, ST, 4, RECORD>, grid, dim3(kWarps * 32), 0, st, a); break;
    case 8: e = launch_kernel(gdn_kernel<IT, ST, 8, RECORD>, grid, dim3(kWarps * 32), 0, st, a); break;
    default: return fail(DFLASH_ERR_BAD_SHAPE, "gdn: Dk=%d not in {32,64,128,256}", a.Dk);
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "gdn launch: %s", cudaGetErrorString(e));
  return DFLASH_OK;
}

template <typename IT, bool RECORD>
int launch_state(const GdnArgs& a, int state_dtype, cudaStream_t st) {
  switch (state_dtype) {
    case DFLASH_F32: return launch_npt<IT, float, RECORD>(a, st);
    case DFLASH_BF16: return launch_npt<IT, __nv_bfloat16, RECORD>(a, st);
    case DFLASH_F16: return launch_npt<IT, __half, RECORD>(a, st);
    default: return fail(DFLASH_ERR_BAD_ARG, "gdn: state dtype %d", state_dtype);
  }
}

template <bool RECORD>
int launch_in(const GdnArgs& a, int in_dtype, int state_dtype, cudaStream_t st) {
  switch (in_dtype) {
    case DFLASH_BF16: return launch_state<__nv_bfloat16, RECORD>(a, state_dtype, st);
    case DFLASH_F16: return launch_state<__half, RECORD>(a, state_dtype, st);
    case DFLASH_F32: return launch_state<float, RECORD>(a, state_dtype, st);
    default: return fail(DFLASH_ERR_BAD_ARG, "gdn: input dtype %d", in_dtype);
  }
}

int check_common(const GdnArgs& a) {
  if (a.B < 1 || a.T < 0 || a.Hk < 1 || a.Hv < 1 || a.Dk < 1 || a.Dv < 1)
    return fail(DFLASH_ERR_BAD_SHAPE, "gdn: non-positive dimension");
  if (a.Hv % a.Hk != 0) return fail(DFLASH_ERR_BAD_SHAPE, "Cannot align K heads %d to V heads %d", a.Hk, a.Hv);
  if (a.Dk % 32 != 0 || a.Dk > 256) return fail(DFLASH_ERR_BAD_SHAPE, "gdn: Dk=%d must be 32, 64, 128 or 256", a.Dk);
  if ((long long)a.B * a.Hv > 65535) return fail(DFLASH_ERR_BAD_SHAPE, "gdn: B*Hv=%d exceeds 65535", a.B * a.Hv);
  if (((uintptr_t)a.state_in & 15) || ((uintptr_t)a.state_out & 15))
    return fail(DFLASH_ERR_MISALIGNED, "gdn: state pointers must be 16-byte aligned");
  return DFLASH_OK;
}

}  // namespace
}  // namespace dflash

using namespace dflash;

static int g_replay_stream = 1;
/* Testing knob: 0 = always the general replay kernel, 1 (default) = the pipelined streaming kernel where it applies,
 * 2 = the plain streaming kernel. */
extern "C" void dflash_tape_replay_set_stream_kernel(int mode) { g_replay_stream = mode < 0 ? 0 : mode > 2 ? 2 : mode; }

static thread_local int t_state_settled = 0;
/* One-shot promise for this thread's next dflash_gdn_forward_tape call: the kernel launched before it in the stream does
 * not write `state_in` (true inside a verify step, where the projection glue runs in between; NOT true when one call's
 * state_out is the next call's state_in).  The record kernel then requests the state rows before it waits for that
 * kernel (programmatic dependent launch), hiding their HBM latency. */
extern "C" void dflash_gdn_forward_state_is_settled(void) { t_state_settled = 1; }

static int g_record_fast = 1;
/* Testing knob: 0 = always the general record kernel, 1 (default) = the low-latency kernel where it applies (scalar
 * gate, no mask, Dk = 128, bf16 inputs, fp32 state, at most 16 tokens). */
extern "C" void dflash_gdn_forward_set_kernel(int mode) { g_record_fast = mode != 0; }

extern "C" int dflash_gdn_forward_tape(const void* q, const void* k, const void* v, const float* g, const float* beta,
                                       const uint8_t* mask, const void* state_in, void* state_out, void* y,
                                       float* tape, int B, int T, int Hk, int Hv, int Dk, int Dv, int g_is_vector,
                                       int in_dtype, int state_dtype, void* stream) {
  const int settled = t_state_settled;  // good for this call only, whatever becomes of it
  t_state_settled = 0;
  if (!q || !k || !v || !g || !beta || !state_in || !state_out || !y || !tape)
    return fail(DFLASH_ERR_BAD_ARG, "gdn_forward_tape: null operand");
  GdnArgs a{q, k, v, g, beta, mask, state_in, state_out, y, tape, nullptr, nullptr, B, T, T, Hk, Hv, Dk, Dv, g_is_vector,
            (((uintptr_t)q | (uintptr_t)k) & 15) == 0, settled};
  if (int rc = check_common(a)) return rc;
  if (g_record_fast && !g_is_vector && mask == nullptr && Dk == 128 && in_dtype == DFLASH_BF16 && state_dtype == DFLASH_F32 &&
      T >= 1 && T <= kRecT && a.vec_ok && ((uintptr_t)v & 1) == 0) {
    cudaError_t e = launch_kernel(gdn_record_fast_kernel<false>, dim3((Dv + kRecRows - 1) / kRecRows, B * Hv), dim3(128), 0,
                                  (cudaStream_t)stream, a, GdnNormArgs{});
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "gdn_forward_tape launch: %s", cudaGetErrorString(e));
    return DFLASH_OK;
  }
  return launch_in<true>(a, in_dtype, state_dtype, (cudaStream_t)stream);
}

extern "C" int dflash_gdn_forward_tape_norm_supported(int T, int Hk, int Hv, int Dk, int Dv, int in_dtype, int state_dtype) {
  return (T >= 1 && T <= kRecT && Hk >= 1 && Hv >= 1 && Hv % Hk == 0 && Dk == 128 && Dv >= kRecRows && Dv % kRecRows == 0 &&
          Dv <= 8 * kRecRows && in_dtype == DFLASH_BF16 && state_dtype == DFLASH_F32) ? 1 : 0;
}

extern "C" int dflash_gdn_forward_tape_norm(const void* q, const void* k, const void* v, const float* g, const float* beta,
                                            const void* state_in, void* state_out, float* tape, const void* z, long long z_ld,
                                            int z_off, const void* norm_w, void* out, long long out_ld, int B, int T, int Hk,
                                            int Hv, int Dk, int Dv, float eps, int in_dtype, int state_dtype, void* stream) {
  const int settled = t_state_settled;
  t_state_settled = 0;
  if (!q || !k || !v || !g || !beta || !state_in || !state_out || !tape || !z || !norm_w || !out)
    return fail(DFLASH_ERR_BAD_ARG, "gdn_forward_tape_norm: null operand");
  if (!dflash_gdn_forward_tape_norm_supported(T, Hk, Hv, Dk, Dv, in_dtype, state_dtype))
    return fail(DFLASH_ERR_BAD_SHAPE, "gdn_forward_tape_norm: needs bf16 inputs, fp32 state, Dk = 128, Dv %% 16 == 0 and <= 128, <= 16 tokens");
  GdnArgs a{q, k, v, g, beta, nullptr, state_in, state_out, nullptr, tape, nullptr, nullptr, B, T, T, Hk, Hv, Dk, Dv, 0,
            (((uintptr_t)q | (uintptr_t)k) & 15) == 0, settled};
  if (int rc = check_common(a)) return rc;
  if (!a.vec_ok) return fail(DFLASH_ERR_MISALIGNED, "gdn_forward_tape_norm: q and k must be 16-byte aligned");
  if (state_in == state_out || out_ld < (long long)Hv * Dv)
    return fail(DFLASH_ERR_BAD_ARG, "gdn_forward_tape_norm: separate state buffers and out_ld >= Hv * Dv are required");
  GdnNormArgs nm{(const __nv_bfloat16*)z, z_ld, z_off, (const __nv_bfloat16*)norm_w, (__nv_bfloat16*)out, out_ld, eps};
  const int nb = Dv / kRecRows;
  cudaError_t e = launch_kernel_cluster(gdn_record_fast_kernel<true>, dim3(nb, B * Hv), dim3(128), nb, 0, (cudaStream_t)stream, a, nm);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "gdn_forward_tape_norm launch: %s", cudaGetErrorString(e));
  return DFLASH_OK;
}

extern "C" int dflash_tape_replay(const float* tape, const void* k, const float* g, const uint8_t* mask,
                                  const void* state_in, void* state_out, int B, int T, int steps, const int* steps_dev,
                                  int Hk, int Hv, int Dk, int Dv, int g_is_vector, int k_dtype, int state_dtype,
                                  void* stream) {
  if (!tape || !k || !g || !state_in || !state_out) return fail(DFLASH_ERR_BAD_ARG, "tape_replay: null operand");
  if (steps < 0 || steps > T) return fail(DFLASH_ERR_BAD_SHAPE, "tape_replay: steps=%d outside 0..T=%d", steps, T);
  GdnArgs a{nullptr, k, nullptr, g, nullptr, mask, state_in, state_out, nullptr, nullptr, tape, steps_dev,
            B, T, steps_dev ? T : steps, Hk, Hv, Dk, Dv, g_is_vector, ((uintptr_t)k & 15) == 0, 0};
  if (int rc = check_common(a)) return rc;
  if (!g_is_vector && mask == nullptr && Dk == 128 && k_dtype == DFLASH_BF16 && state_dtype == DFLASH_F32 && g_replay_stream == 1 &&
      T <= kFastT && Dv % 4 == 0 && ((uintptr_t)tape & 15) == 0 && ((uintptr_t)k & 15) == 0) {
    int device = 0;
    cudaGetDevice(&device);
    static bool attr_done[64] = {};
    if (!attr_done[device & 63]) {
      cudaError_t e0 = cudaFuncSetAttribute(tape_replay_pipe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPipeSmem);
      if (e0 != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "tape_replay: %s", cudaGetErrorString(e0));
      attr_done[device & 63] = true;
    }
    CUtensorMap tmK, tmTape;
    if (get_replay_map(k, B * T, Hk, 128, T, 0, &tmK) && get_replay_map(tape, B * T, Hv, Dv, T, 1, &tmTape)) {
      const int tiles = B * Hv * ((Dv + kFastRows - 1) / kFastRows);
      const int sms = sm_count(device);
      cudaError_t e = launch_kernel(tape_replay_pipe_kernel, dim3(tiles < sms ? tiles : sms), dim3(kPipeThreads), kPipeSmem,
                                    (cudaStream_t)stream, a, device_error_word(device), tmK, tmTape);
      if (e == cudaSuccess) e = cudaGetLastError();
      if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "tape_replay launch: %s", cudaGetErrorString(e));
      return DFLASH_OK;
    }
  }
  if (!g_is_vector && mask == nullptr && Dk == 128 && k_dtype == DFLASH_BF16 && state_dtype == DFLASH_F32 && g_replay_stream) {
    dim3 grid((Dv + kFastRows - 1) / kFastRows, B * Hv);
    cudaError_t e = launch_kernel(tape_replay_stream_kernel, grid, dim3(kFastWarps * 32), 0, (cudaStream_t)stream, a);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "tape_replay launch: %s", cudaGetErrorString(e));
    return DFLASH_OK;
  }
  return launch_in<false>(a, k_dtype, state_dtype, (cudaStream_t)stream);
}
