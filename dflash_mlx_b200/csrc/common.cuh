// Shared device/host helpers for the dflash B200 kernels (sm_100a only).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dflash_b200.h"

namespace dflash {

// ---- host side error plumbing ------------------------------------------------------------
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);

// Device-side status word: kernels that give up on a bounded wait store a non-zero code here.
int* device_error_word(int device);

// Driver entry point for cuTensorMapEncodeTiled, resolved once (no link-time libcuda dependency).
typedef CUresult (*tensormap_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                        const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                        CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
tensormap_encode_fn get_tensormap_encoder();

int sm_count(int device);

// Programmatic dependent launch: when on, every kernel of this library is launched with the stream-serialisation
// attribute, so its blocks may start (prologue, loads of data no earlier kernel writes) while the previous kernel of
// the stream drains; every kernel executes pdl_wait() before it touches anything an earlier kernel may write or read.
bool pdl_enabled_for_next_launch();

// tcgen05 implementation of the bf16 / group-64 verify matmul (qmm_tc.cu)
namespace tc {
size_t workspace_bytes(int M, int K, int N, int device, int max_blocks);
int launch(const void* x, const void* wq, const void* sc, const void* bi, const void* bias, void* y, int M, int K, int N,
           void* ws, size_t ws_bytes, cudaStream_t st, int device, int max_blocks,
           const dflash_qmm_epilogue* epilogue = nullptr);
size_t gather_workspace_bytes(int M, int block_rows, int Kb, int n_max, int mode, int device, int max_blocks);
int launch_gather(const void* x, const void* wq, const void* sc, const void* bi, void* y, int M, int experts, int block_rows,
                  int Kb, int mode, const int* slot_expert, const int* n_dev, int n_max, void* ws, size_t ws_bytes,
                  cudaStream_t st, int device, int max_blocks, const dflash_qmm_epilogue* epilogue = nullptr);
void set_roles(int dequant_warps, int issuing_threads);
void set_k_parts(int k_parts);
void set_stamps(void* dev);
void set_next(const void* wq, const void* sc, const void* bi, int K, int N);
void set_prefetch_next(int on);
}  // namespace tc

namespace sdpa_tc {
void set_fuse_combine(int on);
void set_split128(int on);
size_t workspace_bytes(int B, int Hq, int N, int D);
int launch(const void* q, const void* k, const void* v, void* out, int B, int Hq, int Hk, int N, int D, long long khs,
           long long kss, long long vhs, long long vss, float scale_log2, const int* n_dev, void* ws, size_t ws_bytes,
           cudaStream_t st);
}  // namespace sdpa_tc

#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_as(bool dependent, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr = {};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = dependent ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Args&&>(args)...);
}
// The same with thread-block clusters of `cluster_x` consecutive blocks along x (gridDim.x % cluster_x == 0).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, int cluster_x, size_t smem,
                                         cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2] = {};
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled_for_next_launch() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Args&&>(args)...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                 Args&&... args) {
  return launch_kernel_as(pdl_enabled_for_next_launch(), kernel, grid, block, smem, st, static_cast<Args&&>(args)...);
}

// ---- device helpers -----------------------------------------------------------------------
#ifndef DFLASH_WAIT_LIMIT
#define DFLASH_WAIT_LIMIT (1u << 22)
#endif
constexpr uint32_t kWaitLimit = DFLASH_WAIT_LIMIT;  // polls before a wait gives up (a fraction of a second)
#ifndef DFLASH_SPIN_POLLS
#define DFLASH_SPIN_POLLS 2
#endif
#ifndef DFLASH_SPIN_SLEEP_NS
#define DFLASH_SPIN_SLEEP_NS 32
#endif
constexpr int kSpinPolls = DFLASH_SPIN_POLLS;      // failed polls before the waiting thread starts to sleep between polls
constexpr int kSpinSleepNs = DFLASH_SPIN_SLEEP_NS;

// Blocks until every kernel this one depends on has completed and its writes are visible (no-op for a plain launch).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel of the stream start its blocks as soon as every block of this one has got here (or exited).
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: returns false (and leaves the barrier alone) after kWaitLimit polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i >= (uint32_t)kSpinPolls) __nanosleep(i > 2048 ? 64 : kSpinSleepNs);
  }
  return false;
}
// The same wait for warps that may wait long next to warps that compute: every poll lets the hardware suspend the thread
// for up to ~1 us (it resumes as soon as the phase completes), so a waiting warp issues almost nothing.  Bounded:
// kWaitLimit / 4 polls of at most that long.
__device__ __forceinline__ bool mbar_wait_quiet(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kWaitLimit / 4; ++i) {
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

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// 2-D tiled TMA load, completion counted on an mbarrier, with an L2 cache-policy hint.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar,
                                            uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar), "l"(policy)
      : "memory");
}
// 2-D tiled TMA prefetch into L2 (no shared-memory destination, no completion): the box of the tensor map at {x, y}.
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y) : "memory");
}
// 3-D tiled TMA load (x innermost), completion counted on an mbarrier, with an L2 cache-policy hint.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar,
                                            uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar), "l"(policy)
      : "memory");
}
// 1-D bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

template <typename T>
struct MmaTraits;
template <>
struct MmaTraits<__nv_bfloat16> {
  static constexpr uint32_t kMagic = 0x43004300u;  // bf16 pair (128.0, 128.0): OR-ing a nibble gives 128+nib exactly
  static constexpr float kMagicValue = 128.0f;
  static constexpr uint32_t kOnes = 0x3F803F80u;   // (1.0, 1.0)
  __device__ static __forceinline__ void mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
  __device__ static __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
  __device__ static __forceinline__ float bits_to_float(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
};
template <>
struct MmaTraits<__half> {
  static constexpr uint32_t kMagic = 0x64006400u;  // fp16 pair (1024.0, 1024.0)
  static constexpr float kMagicValue = 1024.0f;
  static constexpr uint32_t kOnes = 0x3C003C00u;
  __device__ static __forceinline__ void mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
  __device__ static __forceinline__ float to_float(__half v) { return __half2float(v); }
  __device__ static __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
  __device__ static __forceinline__ float bits_to_float(uint16_t b) {
    return __half2float(__ushort_as_half(b));
  }
};

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));
  return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ float4 ld_cg_f4(const float4* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
#endif  // __CUDACC__

}  // namespace dflash
