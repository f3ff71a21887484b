/* CPU restatement of the int4 affine quantised matmul (TEST INFRASTRUCTURE, also the timed CPU baseline).
 *
 * Follows the semantic of `mx.quantized_matmul(transpose=True)` that dflash_mlx/verify_qmm.py:276-280 falls
 * back to, with the bit layout of verify_qmm.py:70-75: nibble i of word j of row n is element k = 8j+i,
 * w_hat = nib * scale[n, k/G] + bias[n, k/G], y[m, n] = sum_k x[m, k] * w_hat[n, k], fp32 accumulate.
 * Inputs/outputs use bf16 bit patterns (uint16) for x, scales, biases; y is fp32.
 * Parallel over output columns with OpenMP; per group the dot product is factored as
 *   s * sum(nib * x) + b * sum(x)   (same algebra as the reference's result, fewer multiplies).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bf16_to_f32(uint16_t v) {
  uint32_t u = (uint32_t)v << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

int qmm_ref_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* x: [M,K] bf16 bits; wq: [N,K/8]; s,b: [N,K/G] bf16 bits; y: [M,N] fp32.  M <= 64. */
void qmm_ref(const uint16_t* x, const uint32_t* wq, const uint16_t* s, const uint16_t* b, float* y, int M, int K,
             int N, int G) {
  float* xf = (float*)malloc((size_t)M * K * sizeof(float));
  float* xsum = (float*)malloc((size_t)M * (K / G) * sizeof(float));
  for (size_t i = 0; i < (size_t)M * K; ++i) xf[i] = bf16_to_f32(x[i]);
  for (int m = 0; m < M; ++m)
    for (int g = 0; g < K / G; ++g) {
      float t = 0.f;
      for (int k = 0; k < G; ++k) t += xf[(size_t)m * K + g * G + k];
      xsum[(size_t)m * (K / G) + g] = t;
    }
  const int words_per_group = G / 8, groups = K / G;
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    float acc[64];
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    const uint32_t* wrow = wq + (size_t)n * (K / 8);
    for (int g = 0; g < groups; ++g) {
      const float sc = bf16_to_f32(s[(size_t)n * groups + g]), bi = bf16_to_f32(b[(size_t)n * groups + g]);
      float nib[128];
      for (int j = 0; j < words_per_group; ++j) {
        const uint32_t w = wrow[g * words_per_group + j];
        for (int i = 0; i < 8; ++i) nib[8 * j + i] = (float)((w >> (4 * i)) & 0xF);
      }
      for (int m = 0; m < M; ++m) {
        const float* xr = xf + (size_t)m * K + g * G;
        float t = 0.f;
        for (int k = 0; k < G; ++k) t += nib[k] * xr[k];
        acc[m] += sc * t + bi * xsum[(size_t)m * groups + g];
      }
    }
    for (int m = 0; m < M; ++m) y[(size_t)m * N + n] = acc[m];
  }
  free(xf);
  free(xsum);
}
