// One GatedDeltaNet layer of a verify step between its input projection and its output projection, in ONE launch:
// causal depthwise conv + SiLU over [conv window ; qkv], per-head RMSNorm and scaling of q and k, gate and beta, the
// gated delta recurrence with tape, the gated RMSNorm of its output (runtime.py:368-445 of dflash-mlx with the kernels of
// dflash_mlx/kernels.py:29-105), plus the rollback tape entries (recurrent_rollback_cache.py:116-127).
// The same arithmetic as dflash_gdn_prep -> dflash_gdn_forward_tape (its low-latency record kernel, whose step function
// is shared) -> dflash_gated_rmsnorm: state, tape and the rollback entries come out bit for bit the same; the per-token
// k . q and the last norm's sum of squares are added in another order (the output differs by fp32 rounding).
//
// Grid (Dv / 16, Hv), 128 threads, the Dv / 16 blocks of a head form one thread-block cluster.  A block owns 16 state
// rows of one value head (a warp 4 rows, 8 lanes a row): it reads them before it waits for the
// previous kernel (nothing of this step writes them), recomputes the head's q and k for the 16 tokens from the
// projection output (cheap, and L2-resident), runs the 16 steps, and meets the other blocks of its head once, to
// finish the output norm.  Restrictions: bf16 activations, fp32 state, Dk = 128, Dv a multiple of 16 up to 128,
// at most 16 tokens, conv kernel up to 8, scalar gate.
#include "common.cuh"
#include "gdn_step.cuh"

namespace dflash {
namespace {

constexpr int kDk = 128, kRowsCta = 16, kTok = 16, kMaxKc = 8;

struct GdnLayerArgs {
  const __nv_bfloat16* proj; long long ld; int z_off, b_off, a_off;
  const __nv_bfloat16* conv_state; const __nv_bfloat16* conv_w; const __nv_bfloat16* conv_b;
  const float* A_log; const float* dt_bias; const __nv_bfloat16* g_norm_w;
  const float* state_in; float* state_out; float* tape; __nv_bfloat16* tape_k; float* tape_g;
  __nv_bfloat16* new_conv_state; __nv_bfloat16* qkv_tape; __nv_bfloat16* out; long long out_ld;
  int T, Hk, Hv, Dv, Kc; float eps;
};

__device__ __forceinline__ float bf(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float ldb(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// 16 sums over the warp's 32 lanes in 16 exchanges (every step halves the values a lane carries); the additions pair up
// exactly as in a butterfly sum of each value.  The even lanes end with the sum of token `token_of_lane(lane)` in v[0].
__device__ __forceinline__ void halving_sum16(float (&v)[kTok], int lane) {
#pragma unroll
  for (int st = 0; st < 4; ++st) {
    const int keepn = 8 >> st, m = 16 >> st;
    const bool up = (lane & m) != 0;
#pragma unroll
    for (int i = 0; i < keepn; ++i) {
      const float send = up ? v[i] : v[i + keepn], mine = up ? v[i + keepn] : v[i];
      v[i] = mine + __shfl_xor_sync(0xffffffffu, send, m);
    }
  }
  v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1);
}
__device__ __forceinline__ int token_of_lane(int lane) {
  return ((lane >> 4) & 1) * 8 + ((lane >> 3) & 1) * 4 + ((lane >> 2) & 1) * 2 + ((lane >> 1) & 1);
}

__global__ void __launch_bounds__(128, 3) gdn_layer_kernel(const GdnLayerArgs a) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, rsub = lane >> 3, cg = lane & 7;
  const int hv = blockIdx.y, rep = a.Hv / a.Hk, hk = hv / rep;
  const int row_base = blockIdx.x * kRowsCta, row = row_base + warp * 4 + rsub;
  const int T = a.T, Kc = a.Kc, keep = Kc - 1, Dv = a.Dv;
  const bool row_ok = row < Dv;
  const int key_dim = a.Hk * kDk, conv_dim = 2 * key_dim + a.Hv * Dv;

  __shared__ __align__(16) float sq[kTok][kDk];
  __shared__ __align__(16) float sk[kTok][kDk];
  __shared__ float sv[kTok][kRowsCta], sy[kTok][kRowsCta];
  __shared__ float sg[kTok], sb[kTok], sinv[kTok];
  __shared__ __align__(16) float red[3][kTok][4];
  __shared__ float ssq_part[kTok];

  // the committed state is written by no kernel of this step: its rows are requested before the wait
  unsigned long long S2[8];
  gdnstep::load_row8(a.state_in + ((size_t)hv * Dv + (row_ok ? row : 0)) * kDk, cg, row_ok, S2);
  pdl_wait();
  pdl_trigger();
  const __nv_bfloat16* proj = a.proj;
  const __nv_bfloat16* cs = a.conv_state;
  const bool writer = blockIdx.x == 0 && hv % rep == 0;  // writes what the blocks of a key head share

  // ---- every global load of the prologue and of the output phase is issued here, before the first use: the block
  // pays one trip to L2 (a warp issues in order and stalls at the first instruction that needs a loaded value) ----
  // q and k of this key head: thread d owns channel d over all tokens (runtime.py:368-397)
  const int cq = hk * kDk + tid, ck = key_dim + cq;
  float wq[kMaxKc], wk[kMaxKc], inq[kTok + kMaxKc - 1], ink[kTok + kMaxKc - 1];
#pragma unroll
  for (int j = 0; j < kMaxKc; ++j) {
    wq[j] = j < Kc ? ldb(a.conv_w + (size_t)cq * Kc + j) : 0.f;
    wk[j] = j < Kc ? ldb(a.conv_w + (size_t)ck * Kc + j) : 0.f;
  }
  const float bq = a.conv_b ? ldb(a.conv_b + cq) : 0.f, bk = a.conv_b ? ldb(a.conv_b + ck) : 0.f;
#pragma unroll
  for (int r = 0; r < kTok + kMaxKc - 1; ++r) {  // rows of [conv window ; qkv]
    inq[r] = 0.f;
    ink[r] = 0.f;
    if (r < T + keep) {
      const __nv_bfloat16* src = r < keep ? cs + (size_t)r * conv_dim : proj + (size_t)(r - keep) * a.ld;
      inq[r] = ldb(src + cq);
      ink[r] = ldb(src + ck);
    }
  }
  // v rows of this block: entry p = (token, row of the block), two per thread
  float xv[2][kMaxKc], wv[2][kMaxKc], bvv[2], zpre[2], gwpre[2];
#pragma unroll
  for (int pp = 0; pp < 2; ++pp) {
    const int p = tid + 128 * pp, t = p >> 4, vrow = row_base + (p & 15);
    const int c = 2 * key_dim + hv * Dv + vrow;
    const bool on = t < T && vrow < Dv;
    bvv[pp] = (on && a.conv_b) ? ldb(a.conv_b + c) : 0.f;
    zpre[pp] = on ? ldb(proj + (size_t)t * a.ld + a.z_off + hv * Dv + vrow) : 0.f;
    gwpre[pp] = on ? ldb(a.g_norm_w + vrow) : 0.f;
#pragma unroll
    for (int j = 0; j < kMaxKc; ++j) {
      xv[pp][j] = 0.f;
      wv[pp][j] = 0.f;
      if (on && j < Kc) {
        const int rr = t + j;
        xv[pp][j] = rr < keep ? ldb(cs + (size_t)rr * conv_dim + c) : ldb(proj + (size_t)(rr - keep) * a.ld + c);
        wv[pp][j] = ldb(a.conv_w + (size_t)c * Kc + j);
      }
    }
  }
  // the new conv window of the block's v channels (rows T .. T+keep-1 of the concatenation): warp 1, one lane per channel
  float ncv[kMaxKc - 1];
  const bool nc_lane = warp == 1 && lane < kRowsCta && row_base + lane < Dv;
  const int nc_c = 2 * key_dim + hv * Dv + row_base + (lane & 15);
#pragma unroll
  for (int r = 0; r < kMaxKc - 1; ++r) {
    ncv[r] = 0.f;
    if (nc_lane && r < keep) {
      const int src = T + r;
      ncv[r] = src < keep ? ldb(cs + (size_t)src * conv_dim + nc_c) : ldb(proj + (size_t)(src - keep) * a.ld + nc_c);
    }
  }
  float gate_a = 0.f, gate_b = 0.f, dtb = 0.f, alog = 0.f;
  if (tid < T) {
    gate_a = ldb(proj + (size_t)tid * a.ld + a.a_off + hv);
    gate_b = ldb(proj + (size_t)tid * a.ld + a.b_off + hv);
    dtb = a.dt_bias[hv];
    alog = a.A_log[hv];
  }

  // ---- conv + SiLU of q and k, their sums of squares ----
  {
    float vq[kTok], vk[kTok];
#pragma unroll
    for (int t = 0; t < kTok; ++t) {
      float aq = bq, ak = bk;
#pragma unroll
      for (int j = 0; j < kMaxKc; ++j)
        if (j < Kc) { aq = fmaf(wq[j], inq[t + j], aq); ak = fmaf(wk[j], ink[t + j], ak); }
      vq[t] = t < T ? bf(silu_f(bf(aq))) : 0.f;
      vk[t] = t < T ? bf(silu_f(bf(ak))) : 0.f;
      sq[t][tid] = vq[t];
      sk[t][tid] = vk[t];
      vq[t] *= vq[t];
      vk[t] *= vk[t];
    }
    if (writer) {
#pragma unroll
      for (int r = 0; r < kTok + kMaxKc - 1; ++r) {
        const __nv_bfloat16 xq = __float2bfloat16_rn(inq[r]), xk = __float2bfloat16_rn(ink[r]);  // exact: bf16 values
        if (r >= keep && r < T + keep) {
          a.qkv_tape[(size_t)(r - keep) * conv_dim + cq] = xq;
          a.qkv_tape[(size_t)(r - keep) * conv_dim + ck] = xk;
        }
        if (r >= T && r < T + keep) {
          a.new_conv_state[(size_t)(r - T) * conv_dim + cq] = xq;
          a.new_conv_state[(size_t)(r - T) * conv_dim + ck] = xk;
        }
      }
    }
    halving_sum16(vq, lane);
    halving_sum16(vk, lane);
    if ((lane & 1) == 0) {
      red[0][token_of_lane(lane)][warp] = vq[0];
      red[1][token_of_lane(lane)][warp] = vk[0];
    }
  }
  // ---- v rows of this block, their tape entries and conv window ----
#pragma unroll
  for (int pp = 0; pp < 2; ++pp) {
    const int p = tid + 128 * pp, t = p >> 4, r = p & 15, vrow = row_base + r;
    float val = 0.f;
    if (t < T && vrow < Dv) {
      const int c = 2 * key_dim + hv * Dv + vrow;
      float acc = bvv[pp], last = 0.f;
#pragma unroll
      for (int j = 0; j < kMaxKc; ++j)
        if (j < Kc) { acc = fmaf(wv[pp][j], xv[pp][j], acc); last = xv[pp][j]; }
      val = bf(silu_f(bf(acc)));
      a.qkv_tape[(size_t)t * conv_dim + c] = __float2bfloat16_rn(last);   // the last tap is the token's own value
    }
    sv[t][r] = val;
  }
  if (nc_lane) {
#pragma unroll
    for (int r = 0; r < kMaxKc - 1; ++r)
      if (r < keep) a.new_conv_state[(size_t)r * conv_dim + nc_c] = __float2bfloat16_rn(ncv[r]);
  }
  // ---- gate and beta (runtime.py:399-403) ----
  if (tid < kTok) {
    float g = 1.f, beta = 0.f;
    if (tid < T) {
      const float xs = bf(gate_a + dtb);
      const float sp = xs > 20.f ? xs : log1pf(expf(xs));
      g = expf(-expf(alog) * sp);
      beta = bf(1.f / (1.f + __expf(-gate_b)));
      if (blockIdx.x == 0) a.tape_g[(size_t)tid * a.Hv + hv] = g;
    }
    sg[tid] = g;
    sb[tid] = beta;
  }
  __syncthreads();
  // ---- per-head RMSNorm of q and k, q scaled by 1/Dk and k by 1/sqrt(Dk); k . q per token for the recurrence ----
  {
    const float isc = rsqrtf((float)kDk);
    float kq[kTok];
#pragma unroll
    for (int t = 0; t < kTok; ++t) {
      const float ssq = (red[0][t][0] + red[0][t][2]) + (red[0][t][1] + red[0][t][3]);
      const float ssk = (red[1][t][0] + red[1][t][2]) + (red[1][t][1] + red[1][t][3]);
      const float nq = bf(sq[t][tid] * rsqrtf(ssq / (float)kDk + a.eps));
      const float nk = bf(sk[t][tid] * rsqrtf(ssk / (float)kDk + a.eps));
      const __nv_bfloat16 kb = __float2bfloat16_rn(nk * isc);
      const float qf = bf(nq * isc * isc), kf = __bfloat162float(kb);
      sq[t][tid] = qf;
      sk[t][tid] = kf;
      kq[t] = qf * kf;
      if (writer && t < T) a.tape_k[((size_t)t * a.Hk + hk) * kDk + tid] = kb;
    }
    halving_sum16(kq, lane);
    if ((lane & 1) == 0) red[2][token_of_lane(lane)][warp] = kq[0];
  }
  __syncthreads();
  // ---- the recurrence (kernels.py:62-99), a state row over 8 lanes ----
  for (int t = 0; t < T; ++t) {
    const float4 kq4 = *(const float4*)red[2][t];
    float yv;
    const float dl = gdnstep::step(S2, sk[t], sq[t], cg, sg[t], sb[t], sv[t][warp * 4 + rsub], (kq4.x + kq4.z) + (kq4.y + kq4.w), yv);
    if (cg == 0) {
      float ys = 0.f;
      if (row_ok) {
        a.tape[((size_t)t * a.Hv + hv) * Dv + row] = dl;
        ys = bf(yv);  // the recurrence's output is a bf16 array in the reference
      }
      sy[t][warp * 4 + rsub] = ys;
    }
  }
  if (row_ok) gdnstep::store_row8(a.state_out + ((size_t)hv * Dv + row) * kDk, cg, S2);
  __syncthreads();
  // ---- gated RMSNorm over the head's Dv outputs (runtime.py:445): 16-row partial sums, one exchange in the cluster ----
  if (tid < kTok) {
    float s = 0.f;
    if (tid < T) {
#pragma unroll
      for (int r = 0; r < kRowsCta; ++r) s += sy[tid][r] * sy[tid][r];
    }
    ssq_part[tid] = s;
  }
  cluster_arrive();
  cluster_wait();
  if (tid < kTok) {
    float total = 0.f, part[8];
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
    sinv[tid] = rsqrtf(total / (float)Dv + a.eps);
  }
  cluster_arrive();  // this block is done reading the others' shared memory
  __syncthreads();
#pragma unroll
  for (int pp = 0; pp < 2; ++pp) {
    const int p = tid + 128 * pp, t = p >> 4, r = p & 15, vrow = row_base + r;
    if (t < T && vrow < Dv) {
      const float n = bf(sy[t][r] * sinv[t] * gwpre[pp]);
      a.out[(size_t)t * a.out_ld + hv * Dv + vrow] = __float2bfloat16_rn(n * silu_f(zpre[pp]));
    }
  }
  cluster_wait();  // nobody exits while a neighbour may still read its partial sums
}

}  // namespace
}  // namespace dflash

using namespace dflash;

extern "C" int dflash_gdn_layer_supported(int T_rows, int Hk, int Hv, int Dk, int Dv, int conv_kernel, int dtype,
                                          int state_dtype) {
  return (T_rows >= 1 && T_rows <= kTok && Hk >= 1 && Hv >= 1 && Hv % Hk == 0 && Hv <= 65535 && Dk == kDk && Dv >= 16 &&
          Dv % kRowsCta == 0 && Dv <= 8 * kRowsCta && conv_kernel >= 1 && conv_kernel <= kMaxKc && dtype == DFLASH_BF16 &&
          state_dtype == DFLASH_F32) ? 1 : 0;
}

extern "C" int dflash_gdn_layer(const void* proj, long long ld, int z_off, int b_off, int a_off, const void* conv_state,
                                const void* conv_w, const void* conv_b, const float* A_log, const float* dt_bias,
                                const void* g_norm_w, const void* state_in, void* state_out, float* tape, void* tape_k,
                                float* tape_g, void* new_conv_state, void* qkv_tape, void* out, long long out_ld,
                                int T_rows, int Hk, int Hv, int Dk, int Dv, int conv_kernel, float eps, int dtype,
                                int state_dtype, void* stream) {
  if (!proj || !conv_state || !conv_w || !A_log || !dt_bias || !g_norm_w || !state_in || !state_out || !tape || !tape_k ||
      !tape_g || !new_conv_state || !qkv_tape || !out)
    return fail(DFLASH_ERR_BAD_ARG, "gdn_layer: null operand");
  if (!dflash_gdn_layer_supported(T_rows, Hk, Hv, Dk, Dv, conv_kernel, dtype, state_dtype))
    return fail(DFLASH_ERR_BAD_SHAPE,
                "gdn_layer: needs bf16 activations, fp32 state, Dk = 128, Dv %% 16 == 0 and <= 128, <= 16 tokens, conv kernel <= 8");
  if (new_conv_state == conv_state || state_in == state_out)
    return fail(DFLASH_ERR_BAD_ARG, "gdn_layer: the new conv window / state must be separate buffers");
  if (((uintptr_t)state_in & 15) || ((uintptr_t)state_out & 15))
    return fail(DFLASH_ERR_MISALIGNED, "gdn_layer: state pointers must be 16-byte aligned");
  if (out_ld < (long long)Hv * Dv) return fail(DFLASH_ERR_BAD_ARG, "gdn_layer: out_ld < Hv * Dv");
  GdnLayerArgs a{(const __nv_bfloat16*)proj, ld, z_off, b_off, a_off, (const __nv_bfloat16*)conv_state,
                 (const __nv_bfloat16*)conv_w, (const __nv_bfloat16*)conv_b, A_log, dt_bias, (const __nv_bfloat16*)g_norm_w,
                 (const float*)state_in, (float*)state_out, tape, (__nv_bfloat16*)tape_k, tape_g,
                 (__nv_bfloat16*)new_conv_state, (__nv_bfloat16*)qkv_tape, (__nv_bfloat16*)out, out_ld,
                 T_rows, Hk, Hv, Dv, conv_kernel, eps};
  const int nb = Dv / kRowsCta;
  cudaError_t e = launch_kernel_cluster(gdn_layer_kernel, dim3(nb, Hv), dim3(128), nb, 0, (cudaStream_t)stream, a);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "gdn_layer launch: %s", cudaGetErrorString(e));
  return DFLASH_OK;
}
