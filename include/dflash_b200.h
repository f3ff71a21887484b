/* C ABI of libdflash_b200: the B200 (sm_100a) implementation of the dflash-mlx target-verify
 * hot path.  Plain pointers and sizes only; every pointer named `*_dev` / documented as device
 * memory must be a CUDA device pointer on the current device.  Every entry point returns a
 * dflash_status (0 = ok, <0 = error, message via dflash_last_error_string()), enqueues its work on
 * `stream` (a cudaStream_t passed as void*, NULL = the legacy default stream), never synchronises
 * the host and never allocates device memory unless stated.
 *
 * Citations are to files of the dflash-mlx project (the interface each entry point replaces).
 */
#ifndef DFLASH_B200_H_
#define DFLASH_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define DFLASH_API __attribute__((visibility("default")))
#else
#define DFLASH_API
#endif

typedef enum dflash_status {
  DFLASH_OK = 0,
  DFLASH_ERR_BAD_ARG = -1,      /* null pointer, negative size, unknown enum value */
  DFLASH_ERR_BAD_SHAPE = -2,    /* shape outside what the kernel supports */
  DFLASH_ERR_MISALIGNED = -3,   /* pointer or stride not aligned as documented */
  DFLASH_ERR_WORKSPACE = -4,    /* workspace missing or too small */
  DFLASH_ERR_LAUNCH = -5,       /* CUDA reported an error at launch */
  DFLASH_ERR_DEVICE_WAIT = -6,  /* a kernel gave up on a bounded wait (see dflash_device_error) */
  DFLASH_ERR_UNSUPPORTED = -7
} dflash_status;

typedef enum dflash_dtype { DFLASH_BF16 = 0, DFLASH_F16 = 1, DFLASH_F32 = 2 } dflash_dtype;

/* Library version (major*10000 + minor*100 + patch). */
DFLASH_API int dflash_version(void);
/* Message of the last error on the calling thread ("" if none). */
DFLASH_API const char* dflash_last_error_string(void);
/* Reads (and clears) the device-side status word of `device`; non-zero means a kernel abandoned a
 * bounded wait.  This call synchronises the device. */
DFLASH_API int dflash_device_error(int device);

/* ---------------------------------------------------------------------------------------------
 * verify_qmm: y[M,N] = x[M,K] . dequant(w_q)[N,K]^T (+ bias[N]),  M <= 16.
 * Replaces the Metal kernels `verify_mma2big` / `verify_mma2big_pipe` and their dispatcher
 * `verify_matmul` (dflash_mlx/verify_qmm.py:28-127, 130-243, 266-331).
 *   x        device, dtype[M,K] row-major, 16-byte aligned
 *   w_q      device, uint32[N,K/8]; nibble i of word j is element k=8j+i (verify_qmm.py:70-75)
 *   scales   device, dtype[N,K/G];  biases likewise;  w_hat = nib*scale + bias
 *   bias     device, dtype[N] or NULL (the linear layer's additive bias, verify_linear.py:113-128)
 *   y        device, dtype[M,N]
 *   dtype    DFLASH_BF16 or DFLASH_F16;  group_size G in {32,64,128};  K % G == 0, K % 32 == 0
 *   workspace: dflash_verify_qmm_workspace_bytes() bytes of device memory, ZERO-FILLED ONCE by the
 *   caller before its first use and then left alone (the kernel restores the zeros it relies on).
 *   One workspace must not be used by two launches that can overlap on the GPU.
 * Shapes with K % (8*G) != 0 or a misaligned operand run a slower general kernel.
 */
DFLASH_API size_t dflash_verify_qmm_workspace_bytes(int M, int K, int N, int group_size);
DFLASH_API int dflash_verify_qmm(const void* x, const void* w_q, const void* scales, const void* biases, const void* bias,
                      void* y, int M, int K, int N, int group_size, int dtype, void* workspace,
                      size_t workspace_bytes, void* stream);
/* Tuning/testing knob: caps the number of thread blocks the fast kernel uses (0 = one per SM). */
DFLASH_API void dflash_verify_qmm_set_max_blocks(int max_blocks);
/* Introspection for host-side tests (needs no GPU): writes the streaming kernel's work partition for a
 * shape as ints {row_tiles, slabs, max_pieces, blocks, slab_chunk0[slabs+1], slab_block0[slabs+1]} and
 * returns how many ints were written (<0 on error). */
DFLASH_API int dflash_verify_qmm_plan(int M, int K, int N, int group_size, int* out, int capacity);

#ifdef __cplusplus
}
#endif
#endif /* DFLASH_B200_H_ */
