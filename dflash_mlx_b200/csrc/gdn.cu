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
#include "common.cuh"

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
};

// RECORD = true : forward with tape.  RECORD = false : replay of `steps` tape entries.
template <typename IT, typename ST, int NPT, bool RECORD>
__global__ void __launch_bounds__(kWarps * 32) gdn_kernel(const GdnArgs a) {
  constexpr int Dk = NPT * 32;
  constexpr int kStepChunk = (NPT == 8) ? 8 : 16;  // keeps the static shared memory under 48 KB
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
    for (int i = threadIdx.x; i < nt * Dk; i += kWarps * 32) {
      const int t = i / Dk, d = i % Dk;
      const size_t kq = (((size_t)b * a.T + t0 + t) * a.Hk + hk) * Dk + d;
      sk[t][d] = ldf<IT>(kg + kq);
      if (RECORD) sq[t][d] = ldf<IT>(qg + kq);
      if (a.g_is_vector) sgv[t][d] = a.g[(((size_t)b * a.T + t0 + t) * a.Hv + hv) * Dk + d];
    }
    for (int i = threadIdx.x; i < nt * kRowsPerCta; i += kWarps * 32) {
      const int t = i / kRowsPerCta, r = i % kRowsPerCta;
      const int row = blockIdx.x * kRowsPerCta + r;
      const size_t idx = (((size_t)b * a.T + t0 + t) * a.Hv + hv) * a.Dv + row;
      float val = 0.f;
      if (row < a.Dv) val = RECORD ? ldf<IT>(vg + idx) : a.tape_in[idx];
      sv[t][r] = val;
    }
    if (threadIdx.x < nt) {
      const size_t idx = ((size_t)b * a.T + t0 + threadIdx.x) * a.Hv + hv;
      sg[threadIdx.x] = a.g_is_vector ? 1.f : a.g[idx];
      sb[threadIdx.x] = RECORD ? a.beta[idx] : 0.f;
      sm[threadIdx.x] = a.mask ? (int)a.mask[(size_t)b * a.T + t0 + threadIdx.x] : 1;
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

extern "C" int dflash_gdn_forward_tape(const void* q, const void* k, const void* v, const float* g, const float* beta,
                                       const uint8_t* mask, const void* state_in, void* state_out, void* y,
                                       float* tape, int B, int T, int Hk, int Hv, int Dk, int Dv, int g_is_vector,
                                       int in_dtype, int state_dtype, void* stream) {
  if (!q || !k || !v || !g || !beta || !state_in || !state_out || !y || !tape)
    return fail(DFLASH_ERR_BAD_ARG, "gdn_forward_tape: null operand");
  GdnArgs a{q, k, v, g, beta, mask, state_in, state_out, y, tape, nullptr, nullptr, B, T, T, Hk, Hv, Dk, Dv, g_is_vector};
  if (int rc = check_common(a)) return rc;
  return launch_in<true>(a, in_dtype, state_dtype, (cudaStream_t)stream);
}

extern "C" int dflash_tape_replay(const float* tape, const void* k, const float* g, const uint8_t* mask,
                                  const void* state_in, void* state_out, int B, int T, int steps, const int* steps_dev,
                                  int Hk, int Hv, int Dk, int Dv, int g_is_vector, int k_dtype, int state_dtype,
                                  void* stream) {
  if (!tape || !k || !g || !state_in || !state_out) return fail(DFLASH_ERR_BAD_ARG, "tape_replay: null operand");
  if (steps < 0 || steps > T) return fail(DFLASH_ERR_BAD_SHAPE, "tape_replay: steps=%d outside 0..T=%d", steps, T);
  GdnArgs a{nullptr, k, nullptr, g, nullptr, mask, state_in, state_out, nullptr, nullptr, tape, steps_dev,
            B, T, steps_dev ? T : steps, Hk, Hv, Dk, Dv, g_is_vector};
  if (int rc = check_common(a)) return rc;
  return launch_in<false>(a, k_dtype, state_dtype, (cudaStream_t)stream);
}
