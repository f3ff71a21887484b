// Small fused kernels between the matmuls of a 16-token verify step (sm_100a).
//
// They restate the per-layer dataflow of the reference's target-model hooks: the GatedDeltaNet layer
// (dflash_mlx/runtime.py:351-452), the gated full-attention layer (runtime.py:515-613) and the step driver
// (runtime.py:779-821, 90-108).  Activations are bf16 (or fp16), all arithmetic is fp32.  Every kernel works on
// T <= 64 token rows; they are latency-sized, one CTA (or warp) per row or per (row, head).
#include "common.cuh"

namespace dflash {
namespace {

template <typename T> __device__ __forceinline__ float tof(T v);
template <> __device__ __forceinline__ float tof<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float tof<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T fromf(float v);
template <> __device__ __forceinline__ __nv_bfloat16 fromf<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half fromf<__half>(float v) { return __float2half_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// Block-wide sum for blockDim.x <= 1024 (every thread gets the result).
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? scratch[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + __expf(-x)); }

// h_out = h_in (+ delta);  x = rmsnorm(h_out) * w.  One CTA per token row.
template <typename T>
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(const T* h_in, const T* __restrict__ delta,
                                                          const T* __restrict__ w, T* h_out,
                                                          T* __restrict__ x, int H, float eps) {
  pdl_wait();
  pdl_trigger();
  __shared__ float scratch[32];
  const size_t row = (size_t)blockIdx.x * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = tof<T>(h_in[row + i]);
    if (delta != nullptr) v = tof<T>(fromf<T>(v + tof<T>(delta[row + i])));  // the residual stream is stored in T
    if (h_out != nullptr) h_out[row + i] = fromf<T>(v);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v;
    if (h_out != nullptr) {
      v = tof<T>(h_out[row + i]);  // written by this same thread above (h_out may alias h_in)
    } else {
      v = tof<T>(h_in[row + i]);
      if (delta != nullptr) v = tof<T>(fromf<T>(v + tof<T>(delta[row + i])));
    }
    x[row + i] = fromf<T>(v * inv * tof<T>(w[i]));
  }
}

// Vectorised form for H % 8 == 0: one 16-byte load per thread and operand, values stay in registers.
template <typename T>
__global__ void __launch_bounds__(1024) add_rmsnorm_vec_kernel(const uint4* h_in, const uint4* __restrict__ delta,
                                                               const uint4* __restrict__ w, uint4* h_out,
                                                               uint4* __restrict__ x, int H8, float eps) {
  pdl_wait();
  pdl_trigger();
  __shared__ float scratch[32];
  const size_t row = (size_t)blockIdx.x * H8;
  constexpr int kMaxV = 4;  // vectors per thread (H <= 8 * 4 * blockDim)
  float v[kMaxV][8];
  float ss = 0.f;
  int nv = 0;
  for (int i = threadIdx.x; i < H8 && nv < kMaxV; i += blockDim.x, ++nv) {
    uint4 a = h_in[row + i];
    const T* ap = (const T*)&a;
    if (delta != nullptr) {
      const uint4 d = delta[row + i];
      const T* dp = (const T*)&d;
      T o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) { o[j] = fromf<T>(tof<T>(ap[j]) + tof<T>(dp[j])); v[nv][j] = tof<T>(o[j]); }
      if (h_out != nullptr) h_out[row + i] = *(const uint4*)o;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[nv][j] = tof<T>(ap[j]);
      if (h_out != nullptr && h_out != h_in) h_out[row + i] = a;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += v[nv][j] * v[nv][j];
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)(H8 * 8) + eps);
  int k = 0;
  for (int i = threadIdx.x; i < H8 && k < kMaxV; i += blockDim.x, ++k) {
    const uint4 ww = w[i];
    const T* wp = (const T*)&ww;
    T o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = fromf<T>(v[k][j] * inv * tof<T>(wp[j]));
    x[row + i] = *(const uint4*)o;
  }
}

// y[t, i] = silu(gu[t, i]) * gu[t, I + i]   (SwiGLU on a fused gate|up projection)
template <typename T>
__global__ void __launch_bounds__(256) swiglu_kernel(const T* __restrict__ gu, T* __restrict__ y, int I, int rows) {
  pdl_wait();
  pdl_trigger();
  const size_t n = (size_t)rows * I;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / I, c = i % I;
    const float g = tof<T>(gu[t * 2 * I + c]), u = tof<T>(gu[t * 2 * I + I + c]);
    y[i] = fromf<T>(silu(g) * u);
  }
}

// h[t, :] = table[ids[t], :]
template <typename T>
__global__ void __launch_bounds__(256) embed_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                                    T* __restrict__ h, int H, int V) {
  pdl_wait();
  pdl_trigger();
  int id = ids[blockIdx.x];
  id = min(max(id, 0), V - 1);
  const uint4* src = (const uint4*)(table + (size_t)id * H);
  uint4* dst = (uint4*)(h + (size_t)blockIdx.x * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

// The same, plus what the first fused matmul of a step takes instead of a normalised x: scaled[t, :] = h[t, :] * next_w
// and ssq[t] = sum of h[t, :]^2 (one partial sum per token: in_parts = 1).
template <typename T>
__global__ void __launch_bounds__(256) embed_scaled_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                                           const T* __restrict__ next_w, T* __restrict__ h,
                                                           T* __restrict__ scaled, float* __restrict__ ssq, int H, int V) {
  pdl_wait();
  pdl_trigger();
  __shared__ float scratch[32];
  int id = ids[blockIdx.x];
  id = min(max(id, 0), V - 1);
  const uint4* src = (const uint4*)(table + (size_t)id * H);
  const uint4* wv = (const uint4*)next_w;
  uint4* dst = (uint4*)(h + (size_t)blockIdx.x * H);
  uint4* dsc = (uint4*)(scaled + (size_t)blockIdx.x * H);
  float ss = 0.f;
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    const uint4 a = src[i], w = wv[i];
    uint4 o;
    const T* ap = (const T*)&a;
    const T* wp = (const T*)&w;
    T* op = (T*)&o;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float v = tof<T>(ap[j]);
      ss += v * v;
      op[j] = fromf<T>(v * tof<T>(wp[j]));
    }
    dst[i] = a;
    dsc[i] = o;
  }
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0) ssq[blockIdx.x] = ss;
}

// Acceptance and commit of one speculative cycle in one launch (runtime.py:101-108 and 878-907,
// recurrent_rollback_cache.py:148-171): n = number of leading positions where the drafted tokens block_ids[1..] equal the
// target's greedy tokens posterior[0..]; steps = n + 1 (positions to commit); the cache position advances by steps; and
// every GatedDeltaNet layer's conv window becomes rows steps .. steps+keep-1 of [old window ; this step's qkv rows].
// Every block recomputes n (a few compares); block 0 writes the scalars.  One block per (layer, window row).
template <typename T>
__global__ void __launch_bounds__(256) accept_commit_kernel(const int* __restrict__ block_ids, const int* __restrict__ posterior,
                                                            int n_tokens, int* n_accepted, int* steps, int* offset,
                                                            int* kv_len, int kv_len_extra, const T* __restrict__ conv_old,
                                                            const T* __restrict__ qkv_tape, T* __restrict__ conv_new,
                                                            int layers, int tape_rows, int keep, int conv_dim) {
  pdl_wait();
  pdl_trigger();
  __shared__ int s_n;
  if (threadIdx.x == 0) {
    int n = 0;
    while (n < n_tokens - 1 && block_ids[n + 1] == posterior[n]) ++n;
    s_n = n;
    if (blockIdx.x == 0) {
      *n_accepted = n;
      *steps = n + 1;
      if (offset != nullptr) {
        const int o = *offset + n + 1;
        *offset = o;
        if (kv_len != nullptr) *kv_len = o + kv_len_extra;
      }
    }
  }
  __syncthreads();
  if (layers <= 0 || keep <= 0) return;
  const int st = s_n + 1;
  const int l = blockIdx.x / keep, r = blockIdx.x % keep;
  const int src = st + r;  // row of [old window (keep rows) ; qkv rows]
  const T* from = src < keep ? conv_old + ((size_t)l * keep + src) * conv_dim
                             : qkv_tape + ((size_t)l * tape_rows + (src - keep)) * conv_dim;
  T* to = conv_new + ((size_t)l * keep + r) * conv_dim;
  for (int c = threadIdx.x; c < conv_dim; c += blockDim.x) to[c] = from[c];
}

// out[t] = index of the first maximum of logits[t, :]  (greedy tokens, runtime.py:90-98)
template <typename T>
__global__ void __launch_bounds__(1024) argmax_kernel(const T* __restrict__ logits, const uint8_t* __restrict__ suppress,
                                                      int* __restrict__ out, int V) {
  pdl_wait();
  pdl_trigger();
  __shared__ float sv[32];
  __shared__ int si[32];
  const T* row = logits + (size_t)blockIdx.x * V;
  // a suppressed token's logit counts as -1e9 rounded to the logits' type (greedy_tokens_with_mask, runtime.py:90-98)
  const float floor_v = tof<T>(fromf<T>(-1e9f));
  auto value = [&](float v, int idx) { return (suppress != nullptr && suppress[idx] != 0) ? floor_v : v; };
  float best = -INFINITY;
  int bi = 0x7fffffff;
  // 16-byte loads over the aligned middle of the row, scalar head and tail
  const int head = (int)((((16 - ((uintptr_t)row & 15)) & 15)) / sizeof(T));
  const int h0 = head < V ? head : V;
  const int nvec = (V - h0) / 8;
  for (int i = threadIdx.x; i < h0; i += blockDim.x) {
    const float v = value(tof<T>(row[i]), i);
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
  const uint4* rv = (const uint4*)(row + h0);
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const uint4 a = rv[i];
    const T* ap = (const T*)&a;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int idx = h0 + 8 * i + j;
      const float v = value(tof<T>(ap[j]), idx);
      if (v > best || (v == best && idx < bi)) { best = v; bi = idx; }
    }
  }
  for (int i = h0 + 8 * nvec + threadIdx.x; i < V; i += blockDim.x) {
    const float v = value(tof<T>(row[i]), i);
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    best = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (threadIdx.x == 0) out[blockIdx.x] = bi;
  }
}

// GatedDeltaNet layer, everything between the input projections and the recurrence (runtime.py:368-403):
// depthwise causal conv over [conv_state ; qkv] + SiLU, split into q/k/v heads, q = Dk^-1 rms_norm(q),
// k = Dk^-1/2 rms_norm(k), g = exp(-exp(A_log) softplus(a + dt_bias)), beta = sigmoid(b); also emits the new
// conv window (last Kc-1 rows of the concatenation) and a contiguous copy of qkv for the rollback tape.
// grid (T, 2*Hk + Hv), block = max(Dk, Dv) threads: one thread per channel of one head.
struct GdnPrepArgs {
  const void* proj; long long ld; int z_off, b_off, a_off;
  const void* conv_state; const void* conv_w; const void* conv_b;
  const float* A_log; const float* dt_bias;
  void* q; void* k; void* v; float* g; float* beta; void* new_conv_state; void* qkv_tape;
  int T, Hk, Hv, Dk, Dv, Kc;
  float eps;
};
template <typename T>
__global__ void __launch_bounds__(256) gdn_prep_kernel(const GdnPrepArgs a) {
  __shared__ float scratch[32];
  const int t = blockIdx.x, hb = blockIdx.y, d = threadIdx.x;
  const int key_dim = a.Hk * a.Dk, conv_dim = 2 * key_dim + a.Hv * a.Dv;
  const bool is_v = hb >= 2 * a.Hk;
  const int D = is_v ? a.Dv : a.Dk;
  const int c = is_v ? 2 * key_dim + (hb - 2 * a.Hk) * a.Dv + d : hb * a.Dk + d;
  const bool live = d < D;
  const T* proj = (const T*)a.proj;
  const T* cs = (const T*)a.conv_state;
  const int keep = a.Kc - 1;
  // All global loads are issued before the first loaded value is used (a warp issues in order, so a load placed after
  // a dependent instruction or a store waits for the earlier round trip): the block pays one memory latency.
  constexpr int kMaxTaps = 8;
  T in[kMaxTaps], wv[kMaxTaps];
  T cb = fromf<T>(0.f), carry = fromf<T>(0.f);
  const bool has_carry = live && t < keep;       // this block also writes row t of the new conv window
  float gate_a = 0.f, gate_b = 0.f, dtb = 0.f, alog = 0.f;
  const bool gates = is_v && d == 0;             // one thread per value head also produces the head's gate and beta
  // the layer's constants (written by no kernel, cold in HBM) are requested before the wait on the previous kernel
  if (live) {
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j)
      if (j < a.Kc) wv[j] = ((const T*)a.conv_w)[(size_t)c * a.Kc + j];
    if (a.conv_b) cb = ((const T*)a.conv_b)[c];
  }
  if (gates) {
    dtb = a.dt_bias[hb - 2 * a.Hk];
    alog = a.A_log[hb - 2 * a.Hk];
  }
  pdl_wait();
  pdl_trigger();
  if (live) {
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j) {
      if (j < a.Kc) {
        const int r = t + j;  // row of [conv_state ; qkv]
        in[j] = r < keep ? cs[(size_t)r * conv_dim + c] : proj[(size_t)(r - keep) * a.ld + c];
      }
    }
    if (has_carry) {
      const int src = a.T + t;
      carry = src < keep ? cs[(size_t)src * conv_dim + c] : proj[(size_t)(src - keep) * a.ld + c];
    }
  }
  if (gates) {
    const int hv = hb - 2 * a.Hk;
    gate_a = tof<T>(proj[(size_t)t * a.ld + a.a_off + hv]);
    gate_b = tof<T>(proj[(size_t)t * a.ld + a.b_off + hv]);
  }
  float val = 0.f;
  if (live) {
    float acc = tof<T>(cb);
    T last = in[0];
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j) {
      if (j < a.Kc) {
        acc = fmaf(tof<T>(wv[j]), tof<T>(in[j]), acc);
        last = in[j];
      }
    }
    val = tof<T>(fromf<T>(acc));
    val = tof<T>(fromf<T>(silu(val)));
    ((T*)a.qkv_tape)[(size_t)t * conv_dim + c] = last;      // the last tap is this token's own qkv value
    if (has_carry) ((T*)a.new_conv_state)[(size_t)t * conv_dim + c] = carry;
    for (int r = t + a.T; r < keep; r += a.T) {  // (a window longer than the block: rows T .. T+keep-1 of the concatenation)
      const int src = a.T + r;
      ((T*)a.new_conv_state)[(size_t)r * conv_dim + c] =
          src < keep ? cs[(size_t)src * conv_dim + c] : proj[(size_t)(src - keep) * a.ld + c];
    }
  }
  if (is_v) {
    if (live) ((T*)a.v)[((size_t)t * a.Hv + (hb - 2 * a.Hk)) * a.Dv + d] = fromf<T>(val);
    if (gates) {
      const int hv = hb - 2 * a.Hk;
      const float xs = tof<T>(fromf<T>(gate_a + dtb));
      const float sp = xs > 20.f ? xs : log1pf(expf(xs));
      a.g[(size_t)t * a.Hv + hv] = expf(-expf(alog) * sp);
      a.beta[(size_t)t * a.Hv + hv] = tof<T>(fromf<T>(sigmoidf(gate_b)));
    }
    return;
  }
  const float ss = block_sum(live ? val * val : 0.f, scratch);
  if (!live) return;
  const float inv = rsqrtf(ss / (float)a.Dk + a.eps);
  const float normed = tof<T>(fromf<T>(val * inv));
  const float isc = rsqrtf((float)a.Dk);
  if (hb < a.Hk) ((T*)a.q)[((size_t)t * a.Hk + hb) * a.Dk + d] = fromf<T>(normed * isc * isc);
  else ((T*)a.k)[((size_t)t * a.Hk + (hb - a.Hk)) * a.Dk + d] = fromf<T>(normed * isc);
}

// out[t, hv*Dv + d] = rms_norm(y[t,hv,:])[d] * w[d] * silu(z[t, z_off + hv*Dv + d])   (runtime.py:445)
template <typename T>
__global__ void __launch_bounds__(128) gated_rmsnorm_kernel(const T* __restrict__ y, const T* __restrict__ proj,
                                                            long long ld, int z_off, const T* __restrict__ w,
                                                            T* __restrict__ out, int rows_heads, int Hv, int Dv, float eps) {
  const int rh = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  T wv[8];  // the norm weight (written by no kernel) is requested before the wait on the previous kernel
  if (Dv <= 256) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (lane + 32 * j < Dv) wv[j] = w[lane + 32 * j];
  }
  pdl_wait();
  pdl_trigger();
  if (rh >= rows_heads) return;
  const int t = rh / Hv, hv = rh % Hv;
  const T* yr = y + (size_t)rh * Dv;
  const T* zr = proj + (size_t)t * ld + z_off + hv * Dv;
  T* orow = out + (size_t)t * Hv * Dv + hv * Dv;
  if (Dv <= 256) {
    // every load is issued before the first use: one memory latency per row instead of one per 32 channels
    T yv[8], zv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int d = lane + 32 * j;
      if (d < Dv) { yv[j] = yr[d]; zv[j] = zr[d]; }
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (lane + 32 * j < Dv) { const float v = tof<T>(yv[j]); ss += v * v; }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)Dv + eps);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int d = lane + 32 * j;
      if (d < Dv) {
        const float n = tof<T>(fromf<T>(tof<T>(yv[j]) * inv * tof<T>(wv[j])));
        orow[d] = fromf<T>(n * silu(tof<T>(zv[j])));
      }
    }
    return;
  }
  float ss = 0.f;
  for (int d = lane; d < Dv; d += 32) { const float v = tof<T>(yr[d]); ss += v * v; }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)Dv + eps);
  for (int d = lane; d < Dv; d += 32) {
    const float n = tof<T>(fromf<T>(tof<T>(yr[d]) * inv * tof<T>(w[d])));
    orow[d] = fromf<T>(n * silu(tof<T>(zr[d])));
  }
}

// Full-attention layer between the projections and the attention kernel (runtime.py:527-555):
// per-head RMSNorm of q and k (with weights), rotary embedding of the first `rope_dims` channels at position
// offset + t, q written as [Hq, T, D], k and v appended to the cache at row offset + t.
// proj row: [ (query D | gate D) x Hq | k (Hk*D) | v (Hk*D) ].  One warp per (token, head).
struct AttnPrepArgs {
  const void* proj; long long ld; int k_off, v_off;
  const void* q_norm_w; const void* k_norm_w;
  void* q; void* kcache; void* vcache; long long cache_head_stride;
  int T, Hq, Hk, D, rope_dims, offset;
  float eps, rope_base;
  const int* offset_dev;  // when not NULL the cache offset is read on the device
  int capacity;           // rows per head the caches hold: a position at or beyond it is not stored
  int* err;               // device error word (code 31: cache position out of range)
};
template <typename T>
__global__ void __launch_bounds__(128) attn_prep_kernel(const AttnPrepArgs a) {
  const int idx = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int heads = a.Hq + 2 * a.Hk;
  const int t = idx / heads, h = idx % heads;
  // the norm weights (written by no kernel) are requested before the wait on the previous kernel
  T wv[8], wpv[8];
  if (idx < a.T * heads && h < a.Hq + a.Hk && a.D <= 256) {
    const T* w0 = (const T*)(h < a.Hq ? a.q_norm_w : a.k_norm_w);
    const int half0 = a.rope_dims / 2;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int d = lane + 32 * j;
      if (d < a.D) {
        wv[j] = w0[d];
        if (d < a.rope_dims) wpv[j] = w0[d < half0 ? d + half0 : d - half0];
      }
    }
  }
  pdl_wait();
  pdl_trigger();
  if (idx >= a.T * heads) return;
  const T* row = (const T*)a.proj + (size_t)t * a.ld;
  const int pos = (a.offset_dev ? *a.offset_dev : a.offset) + t;
  // A stale or mis-advanced device offset must not become a store into a neighbouring allocation: the row is dropped
  // and the device error word says so (the queries are still written: they live in their own buffer).
  const bool in_cache = pos >= 0 && pos < a.capacity;
  if (!in_cache && lane == 0 && h >= a.Hq) atomicCAS(a.err, 0, 31 | (t << 8));
  if (h >= a.Hq + a.Hk) {  // value head: plain copy into the cache
    if (!in_cache) return;
    const int hk = h - a.Hq - a.Hk;
    T* dst = (T*)a.vcache + (size_t)hk * a.cache_head_stride + (size_t)pos * a.D;
    if (a.D <= 256) {   // loads first, then stores: one memory latency for the row
      T vv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (lane + 32 * j < a.D) vv[j] = row[a.v_off + hk * a.D + lane + 32 * j];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (lane + 32 * j < a.D) dst[lane + 32 * j] = vv[j];
      return;
    }
    for (int d = lane; d < a.D; d += 32) dst[d] = row[a.v_off + hk * a.D + d];
    return;
  }
  const bool is_q = h < a.Hq;
  const T* src = is_q ? row + (size_t)h * 2 * a.D : row + a.k_off + (h - a.Hq) * a.D;
  const T* w = (const T*)(is_q ? a.q_norm_w : a.k_norm_w);
  T* dst = is_q ? (T*)a.q + ((size_t)h * a.T + t) * a.D
                : (T*)a.kcache + (size_t)(h - a.Hq) * a.cache_head_stride + (size_t)pos * a.D;
  const int half = a.rope_dims / 2;
  if (a.D <= 256) {
    // Every load (the row, the norm weights, the rotation partners) is issued before the first use, and the rotation
    // angles - double-precision pow / sincos, independent of the data - are computed while the loads are in flight.
    T xv[8], xpv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int d = lane + 32 * j;
      if (d < a.D) {
        xv[j] = src[d];
        if (d < a.rope_dims) xpv[j] = src[d < half ? d + half : d - half];
      }
    }
    float cs_[8], sn_[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int d = lane + 32 * j;
      cs_[j] = 1.f;
      sn_[j] = 0.f;
      if (d < a.D && d < a.rope_dims) {
        const int i = d < half ? d : d - half;
        const double theta = (double)pos * pow((double)a.rope_base, -2.0 * (double)i / (double)a.rope_dims);
        double sn, cs;
        sincos(theta, &sn, &cs);
        cs_[j] = (float)cs;
        sn_[j] = (float)sn;
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (lane + 32 * j < a.D) { const float v = tof<T>(xv[j]); ss += v * v; }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)a.D + a.eps);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int d = lane + 32 * j;
      if (d < a.D) {
        const float x = tof<T>(fromf<T>(tof<T>(xv[j]) * inv * tof<T>(wv[j])));
        float o = x;
        if (d < a.rope_dims) {
          const float xp = tof<T>(fromf<T>(tof<T>(xpv[j]) * inv * tof<T>(wpv[j])));
          o = d < half ? x * cs_[j] - xp * sn_[j] : xp * sn_[j] + x * cs_[j];
        }
        if (is_q || in_cache) dst[d] = fromf<T>(o);
      }
    }
    return;
  }
  float ss = 0.f;
  for (int d = lane; d < a.D; d += 32) { const float v = tof<T>(src[d]); ss += v * v; }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)a.D + a.eps);
  for (int d = lane; d < a.D; d += 32) {
    const float x = tof<T>(fromf<T>(tof<T>(src[d]) * inv * tof<T>(w[d])));
    float o = x;
    if (d < a.rope_dims) {
      const int i = d < half ? d : d - half;
      const int pd = d < half ? d + half : d - half;
      const float xp = tof<T>(fromf<T>(tof<T>(src[pd]) * inv * tof<T>(w[pd])));
      const double theta = (double)pos * pow((double)a.rope_base, -2.0 * (double)i / (double)a.rope_dims);
      double sn, cs;
      sincos(theta, &sn, &cs);
      o = d < half ? x * (float)cs - xp * (float)sn : xp * (float)sn + x * (float)cs;
    }
    if (is_q || in_cache) dst[d] = fromf<T>(o);
  }
}

// out[t, hq*D + d] = o[hq, t, d] * sigmoid(gate[t, hq, d])   (runtime.py:611-612)
template <typename T>
__global__ void __launch_bounds__(256) attn_post_kernel(const T* __restrict__ o, const T* __restrict__ proj, long long ld,
                                                        T* __restrict__ out, long long out_ld, int Tn, int Hq, int D) {
  pdl_wait();
  pdl_trigger();
  const size_t n = (size_t)Tn * Hq * D;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int d = (int)(i % D), hq = (int)((i / D) % Hq), t = (int)(i / ((size_t)D * Hq));
    const float gate = tof<T>(proj[(size_t)t * ld + (size_t)hq * 2 * D + D + d]);
    out[(size_t)t * out_ld + (size_t)hq * D + d] = fromf<T>(tof<T>(o[((size_t)hq * Tn + t) * D + d]) * sigmoidf(gate));
  }
}


// ---- mixture of experts: routing --------------------------------------------------------------------------------
// One CTA, one warp per token.  logits [T, E + 1] (column E is the shared expert's gate).  Per token: the top_k routed
// experts by logit (ties to the lower index) and their softmax weights over those top_k (= softmax over all experts
// renormalised on the chosen ones, mlx-lm / Qwen `norm_topk_prob`).  Then the experts any token chose that lie in
// [e_lo, e_hi) are numbered in ascending id order into `slot_expert` as indices into this rank's expert stack
// (e - e_lo); with `with_shared` the shared expert (stack index e_hi - e_lo) takes the last slot with weight
// sigmoid(logit[t, E]).  wdense[t, slot] is token t's weight for that slot (0 if not routed).
template <typename T, int kPer>  // kPer = experts per lane: 8 covers E <= 256, 32 covers E <= 1024
__global__ void __launch_bounds__(1024) moe_route_kernel(const T* __restrict__ logits, int T_rows, int E, int top_k, int e_lo,
                                                         int e_hi, int with_shared, int n_max, int* __restrict__ slot_expert,
                                                         int* __restrict__ n_out, float* __restrict__ wdense,
                                                         int* __restrict__ topk_ids, float* __restrict__ topk_w) {
  pdl_wait();
  pdl_trigger();
  __shared__ int chosen[1024];     // expert -> 1 if some token chose it
  __shared__ int slot_of[1024];    // expert -> slot (or -1)
  __shared__ int warp_cnt[32];
  __shared__ int s_ids[32][16];
  __shared__ float s_w[32][16];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  for (int i = threadIdx.x; i < 1024; i += blockDim.x) { chosen[i] = 0; slot_of[i] = -1; }
  for (int i = threadIdx.x; i < T_rows * n_max; i += blockDim.x) wdense[i] = 0.f;
  __syncthreads();
  if (warp < T_rows) {
    const T* row = logits + (size_t)warp * (E + 1);
    float v[kPer];
    const int per = (E + 31) / 32;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const int e = lane + 32 * i;
      v[i] = (i < per && e < E) ? tof<T>(row[e]) : -INFINITY;
    }
    float mx0 = 0.f, den = 0.f;
    for (int k = 0; k < top_k; ++k) {
      float best = -INFINITY;
      int bi = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < kPer; ++i)
        if (i < per && v[i] > best) { best = v[i]; bi = lane + 32 * i; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      if (k == 0) mx0 = best;
      const float w = __expf(best - mx0);
      den += w;
      if (lane == 0) { s_ids[warp][k] = bi; s_w[warp][k] = w; chosen[bi] = 1; }
      if ((bi & 31) == lane) {
#pragma unroll
        for (int i = 0; i < kPer; ++i)
          if (i == (bi >> 5)) v[i] = -INFINITY;
      }
    }
    if (lane == 0)
      for (int k = 0; k < top_k; ++k) {
        s_w[warp][k] /= den;
        if (topk_ids != nullptr) { topk_ids[warp * top_k + k] = s_ids[warp][k]; topk_w[warp * top_k + k] = s_w[warp][k]; }
      }
  }
  __syncthreads();
  // number the chosen local experts in ascending order: thread e owns expert e (E <= blockDim.x is checked by the host)
  const int e = threadIdx.x;
  const int mine = (e < E && e >= e_lo && e < e_hi && chosen[e]) ? 1 : 0;
  const unsigned bal = __ballot_sync(0xffffffffu, mine);
  if (lane == 0) warp_cnt[warp] = __popc(bal);
  __syncthreads();
  int before = 0;
  for (int w = 0; w < warp; ++w) before += warp_cnt[w];
  int total = 0;
  for (int w = 0; w < nwarp; ++w) total += warp_cnt[w];
  if (mine) {
    const int slot = before + __popc(bal & ((1u << lane) - 1u));
    if (slot < n_max) { slot_expert[slot] = e - e_lo; slot_of[e] = slot; }  // index inside this rank's stack
  }
  int n = total < n_max ? total : n_max;
  int shared_slot = -1;
  if (with_shared && n < n_max) { shared_slot = n; ++n; }
  if (threadIdx.x == 0) {
    if (shared_slot >= 0) slot_expert[shared_slot] = e_hi - e_lo;  // the shared expert follows the rank's experts
    *n_out = n;
  }
  __syncthreads();
  if (warp < T_rows) {
    if (lane < top_k) {
      const int sl = slot_of[s_ids[warp][lane]];
      if (sl >= 0) wdense[warp * n_max + sl] = s_w[warp][lane];
    }
    if (lane == 0 && shared_slot >= 0)
      wdense[warp * n_max + shared_slot] = sigmoidf(tof<T>(logits[(size_t)warp * (E + 1) + E]));
  }
}

// act[t, slot * I + i] = w[t, slot] * silu(gu[t, slot * 2I + i]) * gu[t, slot * 2I + I + i]  for slot < *n  (the input of
// the chunk-gathered down projection; rows of tokens that did not choose the expert are written as zeros)
template <typename T>
__global__ void __launch_bounds__(256) moe_swiglu_kernel(const T* __restrict__ gu, const float* __restrict__ wdense,
                                                         const int* __restrict__ n_dev, T* __restrict__ act, int T_rows, int I,
                                                         int n_max) {
  pdl_wait();
  pdl_trigger();
  const int slot = blockIdx.x, t = blockIdx.y;
  if (slot >= *n_dev) return;
  const float w = wdense[t * n_max + slot];
  const T* g = gu + ((size_t)t * n_max + slot) * 2 * I;
  T* o = act + ((size_t)t * n_max + slot) * I;
  if ((I & 7) == 0 && (((uintptr_t)gu | (uintptr_t)act) & 15) == 0) {   // 16-byte vectors: 8 channels per thread and trip
    for (int i8 = threadIdx.x; i8 < (I >> 3); i8 += blockDim.x) {
      const uint4 gv = *(const uint4*)(g + 8 * i8), uv = *(const uint4*)(g + I + 8 * i8);
      const T* ge = (const T*)&gv;
      const T* ue = (const T*)&uv;
      T r[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        r[j] = (w == 0.f) ? fromf<T>(0.f) : fromf<T>(w * tof<T>(fromf<T>(silu(tof<T>(ge[j])) * tof<T>(ue[j]))));
      *(uint4*)(o + 8 * i8) = *(const uint4*)r;
    }
    return;
  }
  for (int i = threadIdx.x; i < I; i += blockDim.x)
    o[i] = (w == 0.f) ? fromf<T>(0.f) : fromf<T>(w * tof<T>(fromf<T>(silu(tof<T>(g[i])) * tof<T>(g[I + i]))));
}

}  // namespace
}  // namespace dflash

using namespace dflash;

#define DFLASH_DISPATCH(dtype, CALL)                                                  \
  do {                                                                                \
    if ((dtype) == DFLASH_BF16) { using T = __nv_bfloat16; CALL; }                    \
    else if ((dtype) == DFLASH_F16) { using T = __half; CALL; }                       \
    else return fail(DFLASH_ERR_BAD_ARG, "%s: dtype %d (want bf16 or f16)", __func__, (int)(dtype)); \
    cudaError_t e_ = cudaGetLastError();                                              \
    if (e_ != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "%s: %s", __func__, cudaGetErrorString(e_)); \
    return DFLASH_OK;                                                                 \
  } while (0)

extern "C" int dflash_add_rmsnorm(const void* h_in, const void* delta, const void* w, void* h_out, void* x, int T_rows,
                                  int H, float eps, int dtype, void* stream) {
  if (!h_in || !w || !x || T_rows < 1 || H < 1) return fail(DFLASH_ERR_BAD_ARG, "add_rmsnorm: bad argument");
  cudaStream_t st = (cudaStream_t)stream;
  auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  if (H % 8 == 0 && H <= 8 * 4 * 1024 && al(h_in) && al(delta) && al(w) && al(h_out) && al(x)) {
    int threads = (H / 8 + 31) / 32 * 32;
    if (threads > 1024) threads = 1024;
    DFLASH_DISPATCH(dtype, (launch_kernel(add_rmsnorm_vec_kernel<T>, dim3(T_rows), dim3(threads), 0, st, (const uint4*)h_in, (const uint4*)delta, (const uint4*)w, (uint4*)h_out, (uint4*)x, H / 8, eps)));
  }
  DFLASH_DISPATCH(dtype, (launch_kernel(add_rmsnorm_kernel<T>, dim3(T_rows), dim3(256), 0, st, (const T*)h_in, (const T*)delta, (const T*)w,
                                                                          (T*)h_out, (T*)x, H, eps)));
}

extern "C" int dflash_swiglu(const void* gate_up, void* y, int T_rows, int I, int dtype, void* stream) {
  if (!gate_up || !y || T_rows < 1 || I < 1) return fail(DFLASH_ERR_BAD_ARG, "swiglu: bad argument");
  cudaStream_t st = (cudaStream_t)stream;
  const int blocks = (int)(((size_t)T_rows * I + 255) / 256);
  DFLASH_DISPATCH(dtype, (launch_kernel(swiglu_kernel<T>, dim3(blocks < 2048 ? blocks : 2048), dim3(256), 0, st, (const T*)gate_up, (T*)y, I, T_rows)));
}

extern "C" int dflash_embed(const int* ids, const void* table, void* h, int T_rows, int H, int V, int dtype, void* stream) {
  if (!ids || !table || !h || T_rows < 1 || H % 8 != 0) return fail(DFLASH_ERR_BAD_ARG, "embed: bad argument (H %% 8 == 0)");
  cudaStream_t st = (cudaStream_t)stream;
  DFLASH_DISPATCH(dtype, (launch_kernel(embed_kernel<T>, dim3(T_rows), dim3(256), 0, st, ids, (const T*)table, (T*)h, H, V)));
}

extern "C" int dflash_embed_scaled(const int* ids, const void* table, const void* next_w, void* h, void* scaled, float* ssq,
                                   int T_rows, int H, int V, int dtype, void* stream) {
  if (!ids || !table || !next_w || !h || !scaled || !ssq || T_rows < 1 || T_rows > 16 || H % 8 != 0)
    return fail(DFLASH_ERR_BAD_ARG, "embed_scaled: bad argument (1..16 rows, H %% 8 == 0)");
  cudaStream_t st = (cudaStream_t)stream;
  DFLASH_DISPATCH(dtype, (launch_kernel(embed_scaled_kernel<T>, dim3(T_rows), dim3(256), 0, st, ids, (const T*)table, (const T*)next_w,
                                        (T*)h, (T*)scaled, ssq, H, V)));
}

extern "C" int dflash_argmax(const void* logits, int* out, int T_rows, int V, int dtype, void* stream) {
  if (!logits || !out || T_rows < 1 || V < 1) return fail(DFLASH_ERR_BAD_ARG, "argmax: bad argument");
  cudaStream_t st = (cudaStream_t)stream;
  DFLASH_DISPATCH(dtype, (launch_kernel(argmax_kernel<T>, dim3(T_rows), dim3(1024), 0, st, (const T*)logits, (const uint8_t*)nullptr, out, V)));
}

extern "C" int dflash_argmax_masked(const void* logits, const uint8_t* suppress, int* out, int T_rows, int V, int dtype,
                                    void* stream) {
  if (!logits || !out || T_rows < 1 || V < 1) return fail(DFLASH_ERR_BAD_ARG, "argmax_masked: bad argument");
  cudaStream_t st = (cudaStream_t)stream;
  DFLASH_DISPATCH(dtype, (launch_kernel(argmax_kernel<T>, dim3(T_rows), dim3(1024), 0, st, (const T*)logits, suppress, out, V)));
}

extern "C" int dflash_accept_commit(const int* block_ids, const int* posterior, int n_tokens, int* n_accepted, int* steps,
                                    int* offset, int* kv_len, int kv_len_extra, const void* conv_old, const void* qkv_tape,
                                    void* conv_new, int layers, int tape_rows, int keep, int conv_dim, int dtype, void* stream) {
  if (!block_ids || !posterior || !n_accepted || !steps || n_tokens < 1 || n_tokens > 64)
    return fail(DFLASH_ERR_BAD_ARG, "accept_commit: bad argument (1..64 tokens)");
  if (layers > 0 && (!conv_old || !qkv_tape || !conv_new || keep < 0 || conv_dim < 1 || tape_rows < n_tokens || conv_old == conv_new))
    return fail(DFLASH_ERR_BAD_ARG, "accept_commit: bad conv window arguments");
  cudaStream_t st = (cudaStream_t)stream;
  const int rows = layers > 0 ? layers * (keep > 0 ? keep : 1) : 1;
  DFLASH_DISPATCH(dtype, (launch_kernel(accept_commit_kernel<T>, dim3(rows), dim3(256), 0, st, block_ids, posterior, n_tokens,
                                        n_accepted, steps, offset, kv_len, kv_len_extra, (const T*)conv_old, (const T*)qkv_tape,
                                        (T*)conv_new, layers, tape_rows, keep, conv_dim)));
}

extern "C" int dflash_gdn_prep(const void* proj, long long ld, int z_off, int b_off, int a_off, const void* conv_state,
                               const void* conv_w, const void* conv_b, const float* A_log, const float* dt_bias, void* q,
                               void* k, void* v, float* g, float* beta, void* new_conv_state, void* qkv_tape, int T_rows,
                               int Hk, int Hv, int Dk, int Dv, int conv_kernel, float eps, int dtype, void* stream) {
  if (!proj || !conv_state || !conv_w || !A_log || !dt_bias || !q || !k || !v || !g || !beta || !new_conv_state || !qkv_tape)
    return fail(DFLASH_ERR_BAD_ARG, "gdn_prep: null operand");
  if (T_rows < 1 || Dk > 256 || Dv > 256 || conv_kernel < 1 || conv_kernel > 8 || new_conv_state == conv_state)
    return fail(DFLASH_ERR_BAD_SHAPE, "gdn_prep: unsupported shape (Dk,Dv <= 256; conv kernel 1..8; separate conv buffers)");
  GdnPrepArgs a{proj, ld, z_off, b_off, a_off, conv_state, conv_w, conv_b, A_log, dt_bias, q, k, v, g, beta,
                new_conv_state, qkv_tape, T_rows, Hk, Hv, Dk, Dv, conv_kernel, eps};
  const int D = Dk > Dv ? Dk : Dv;
  const int threads = (D + 31) / 32 * 32;
  dim3 grid(T_rows, 2 * Hk + Hv);
  cudaStream_t st = (cudaStream_t)stream;
  DFLASH_DISPATCH(dtype, (launch_kernel(gdn_prep_kernel<T>, dim3(grid), dim3(threads), 0, st, a)));
}

extern "C" int dflash_gated_rmsnorm(const void* y, const void* proj, long long ld, int z_off, const void* w, void* out,
                                    int T_rows, int Hv, int Dv, float eps, int dtype, void* stream) {
  if (!y || !proj || !w || !out || T_rows < 1) return fail(DFLASH_ERR_BAD_ARG, "gated_rmsnorm: bad argument");
  cudaStream_t st = (cudaStream_t)stream;
  const int rh = T_rows * Hv;
  DFLASH_DISPATCH(dtype, (launch_kernel(gated_rmsnorm_kernel<T>, dim3((rh + 3) / 4), dim3(128), 0, st, (const T*)y, (const T*)proj, ld, z_off,
                                                                                 (const T*)w, (T*)out, rh, Hv, Dv, eps)));
}

static int attn_prep_impl(const void* proj, long long ld, int k_off, int v_off, const void* q_norm_w,
                          const void* k_norm_w, void* q, void* kcache, void* vcache, long long cache_head_stride,
                          int T_rows, int Hq, int Hk, int D, int rope_dims, int offset, float eps, float rope_base,
                          int dtype, void* stream, const int* offset_dev, int capacity) {
  if (!proj || !q_norm_w || !k_norm_w || !q || !kcache || !vcache) return fail(DFLASH_ERR_BAD_ARG, "attn_prep: null operand");
  if (T_rows < 1 || rope_dims < 0 || rope_dims > D || rope_dims % 2 != 0 || offset < 0)
    return fail(DFLASH_ERR_BAD_SHAPE, "attn_prep: bad rope_dims/offset");
  if (capacity < 1 || (long long)capacity * D > cache_head_stride)
    return fail(DFLASH_ERR_BAD_SHAPE, "attn_prep: cache capacity %d does not fit the head stride", capacity);
  if (!offset_dev && offset + T_rows > capacity)
    return fail(DFLASH_ERR_BAD_SHAPE, "attn_prep: rows %d..%d exceed the cache capacity %d", offset, offset + T_rows - 1, capacity);
  int device = 0;
  cudaGetDevice(&device);
  AttnPrepArgs a{proj, ld, k_off, v_off, q_norm_w, k_norm_w, q, kcache, vcache, cache_head_stride,
                 T_rows, Hq, Hk, D, rope_dims, offset, eps, rope_base, offset_dev, capacity, device_error_word(device)};
  const int n = T_rows * (Hq + 2 * Hk);
  cudaStream_t st = (cudaStream_t)stream;
  DFLASH_DISPATCH(dtype, (launch_kernel(attn_prep_kernel<T>, dim3((n + 3) / 4), dim3(128), 0, st, a)));
}

extern "C" int dflash_attn_prep(const void* proj, long long ld, int k_off, int v_off, const void* q_norm_w,
                                const void* k_norm_w, void* q, void* kcache, void* vcache, long long cache_head_stride,
                                int cache_capacity, int T_rows, int Hq, int Hk, int D, int rope_dims, int offset, float eps,
                                float rope_base, int dtype, void* stream) {
  return attn_prep_impl(proj, ld, k_off, v_off, q_norm_w, k_norm_w, q, kcache, vcache, cache_head_stride, T_rows, Hq, Hk, D,
                        rope_dims, offset, eps, rope_base, dtype, stream, nullptr, cache_capacity);
}

extern "C" int dflash_attn_prep_dev_offset(const void* proj, long long ld, int k_off, int v_off, const void* q_norm_w,
                                           const void* k_norm_w, void* q, void* kcache, void* vcache,
                                           long long cache_head_stride, int cache_capacity, int T_rows, int Hq, int Hk,
                                           int D, int rope_dims, const int* offset_dev, float eps, float rope_base,
                                           int dtype, void* stream) {
  if (!offset_dev) return fail(DFLASH_ERR_BAD_ARG, "attn_prep_dev_offset: offset_dev is NULL");
  return attn_prep_impl(proj, ld, k_off, v_off, q_norm_w, k_norm_w, q, kcache, vcache, cache_head_stride, T_rows, Hq, Hk, D,
                        rope_dims, 0, eps, rope_base, dtype, stream, offset_dev, cache_capacity);
}

extern "C" int dflash_attn_post(const void* o, const void* proj, long long ld, void* out, long long out_ld, int T_rows,
                                int Hq, int D, int dtype, void* stream) {
  if (!o || !proj || !out || T_rows < 1 || out_ld < (long long)Hq * D) return fail(DFLASH_ERR_BAD_ARG, "attn_post: bad argument");
  cudaStream_t st = (cudaStream_t)stream;
  const int blocks = (int)(((size_t)T_rows * Hq * D + 255) / 256);
  DFLASH_DISPATCH(dtype, (launch_kernel(attn_post_kernel<T>, dim3(blocks), dim3(256), 0, st, (const T*)o, (const T*)proj, ld, (T*)out, out_ld, T_rows, Hq, D)));
}

extern "C" int dflash_moe_route(const void* logits, int T_rows, int experts, int top_k, int e_lo, int e_hi, int with_shared,
                                int n_max, int* slot_expert, int* n_active, float* wdense, int* topk_ids, float* topk_w,
                                int dtype, void* stream) {
  if (!logits || !slot_expert || !n_active || !wdense) return fail(DFLASH_ERR_BAD_ARG, "moe_route: null operand");
  if (T_rows < 1 || T_rows > 32 || experts < 1 || experts > 1024 || top_k < 1 || top_k > 16 || top_k > experts || n_max < 1 ||
      e_lo < 0 || e_hi > experts || e_lo > e_hi || (topk_ids != nullptr) != (topk_w != nullptr))
    return fail(DFLASH_ERR_BAD_SHAPE, "moe_route: T <= 32, experts <= 1024, top_k <= 16, 0 <= e_lo <= e_hi <= experts");
  int threads = (experts + 31) / 32 * 32;
  if (threads < 32 * T_rows) threads = 32 * T_rows;
  cudaStream_t st = (cudaStream_t)stream;
  if (experts <= 256)
    DFLASH_DISPATCH(dtype, (launch_kernel(moe_route_kernel<T, 8>, dim3(1), dim3(threads), 0, st, (const T*)logits, T_rows,
                                          experts, top_k, e_lo, e_hi, with_shared, n_max, slot_expert, n_active, wdense,
                                          topk_ids, topk_w)));
  DFLASH_DISPATCH(dtype, (launch_kernel(moe_route_kernel<T, 32>, dim3(1), dim3(threads), 0, st, (const T*)logits, T_rows, experts,
                                        top_k, e_lo, e_hi, with_shared, n_max, slot_expert, n_active, wdense, topk_ids, topk_w)));
}

extern "C" int dflash_moe_swiglu(const void* gate_up, const float* wdense, const int* n_active, void* act, int T_rows, int I,
                                 int n_max, int dtype, void* stream) {
  if (!gate_up || !wdense || !n_active || !act || T_rows < 1 || I < 1 || n_max < 1)
    return fail(DFLASH_ERR_BAD_ARG, "moe_swiglu: bad argument");
  cudaStream_t st = (cudaStream_t)stream;
  const int threads = (I & 7) == 0 ? (I / 8 >= 256 ? 256 : (I / 8 + 31) / 32 * 32) : 256;
  DFLASH_DISPATCH(dtype, (launch_kernel(moe_swiglu_kernel<T>, dim3(n_max, T_rows), dim3(threads), 0, st, (const T*)gate_up, wdense,
                                        n_active, (T*)act, T_rows, I, n_max)));
}
