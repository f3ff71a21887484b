// One token step of the gated delta recurrence in the low-latency layout, shared by the record kernel (gdn.cu) and the
// one-launch layer kernel (gdn_layer.cu) so that both produce the same bits.
//
// A state row (128 key channels) is spread over 8 neighbouring lanes: lane c of the group holds the 16-byte chunks
// c, c + 8, c + 16, c + 24 of the row as 8 packed fp32 pairs.  Per step (kernels.py:62-99 of dflash-mlx):
//   S *= g ; kv = S k ; delta = (v - kv) beta ; S += delta (x) k ; y = S q
// with y evaluated as S' q + delta (k . q), S' the decayed state before the update: the two row reductions (S' k, S' q)
// then form one interleaved shuffle chain of 3 levels.  The state goes through the same two roundings per step as in
// the replay kernels (mul, then fma), so a replay of the tape reproduces it bit for bit.
#pragma once
#include <cuda_runtime.h>

namespace dflash {
namespace gdnstep {

__device__ __forceinline__ unsigned long long pack2(float a, float b) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ unsigned long long mul2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

// The lane's part of the row from / to global memory (row = pointer to the row's 128 floats, cg = lane & 7).
__device__ __forceinline__ void load_row8(const float* row, int cg, bool ok, unsigned long long (&S2)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 v = ok ? *(const float4*)(row + 4 * (cg + 8 * i)) : make_float4(0.f, 0.f, 0.f, 0.f);
    S2[2 * i] = pack2(v.x, v.y);
    S2[2 * i + 1] = pack2(v.z, v.w);
  }
}
__device__ __forceinline__ void store_row8(float* row, int cg, const unsigned long long (&S2)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float4 o;
    unpack2(S2[2 * i], o.x, o.y);
    unpack2(S2[2 * i + 1], o.z, o.w);
    *(float4*)(row + 4 * (cg + 8 * i)) = o;
  }
}

// One step for the lane's row.  k_row / q_row: the token's 128 key / query channels as fp32 in shared memory (16-byte
// aligned).  Returns delta (identical on the 8 lanes of the row); y = the row's output for this token.
__device__ __forceinline__ float step(unsigned long long (&S2)[8], const float* k_row, const float* q_row, int cg, float g,
                                      float beta, float v, float kq, float& y) {
  unsigned long long k2[8], q2[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 kk = *(const float4*)(k_row + 4 * (cg + 8 * i));
    const float4 qq = *(const float4*)(q_row + 4 * (cg + 8 * i));
    k2[2 * i] = pack2(kk.x, kk.y); k2[2 * i + 1] = pack2(kk.z, kk.w);
    q2[2 * i] = pack2(qq.x, qq.y); q2[2 * i + 1] = pack2(qq.z, qq.w);
  }
  const unsigned long long g2 = pack2(g, g);
  unsigned long long ak0 = 0ull, ak1 = 0ull, aq0 = 0ull, aq1 = 0ull;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    S2[2 * i] = mul2(S2[2 * i], g2);
    S2[2 * i + 1] = mul2(S2[2 * i + 1], g2);
    ak0 = fma2(S2[2 * i], k2[2 * i], ak0);
    ak1 = fma2(S2[2 * i + 1], k2[2 * i + 1], ak1);
    aq0 = fma2(S2[2 * i], q2[2 * i], aq0);
    aq1 = fma2(S2[2 * i + 1], q2[2 * i + 1], aq1);
  }
  float a0, a1, a2, a3;
  unpack2(ak0, a0, a1); unpack2(ak1, a2, a3);
  float pk = (a0 + a1) + (a2 + a3);
  unpack2(aq0, a0, a1); unpack2(aq1, a2, a3);
  float pq = (a0 + a1) + (a2 + a3);
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) {
    pk += __shfl_xor_sync(0xffffffffu, pk, o);
    pq += __shfl_xor_sync(0xffffffffu, pq, o);
  }
  const float dl = (v - pk) * beta;
  const unsigned long long d2 = pack2(dl, dl);
#pragma unroll
  for (int i = 0; i < 8; ++i) S2[i] = fma2(k2[i], d2, S2[i]);
  y = fmaf(dl, kq, pq);
  return dl;
}

}  // namespace gdnstep
}  // namespace dflash
