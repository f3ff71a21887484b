// Row-parallel reduction fused with the residual add and RMSNorm that consume it, over peer-mapped memory (NVLink).
//
// The reference's only collective is one `mx.distributed.all_sum` on the GatedDeltaNet output projection
// (dflash_mlx/runtime.py:449-450); here every row-parallel projection (out_proj, o_proj, down) of a tensor-parallel
// verify step ends in the same pattern: sum the [T, H] block over the ranks, add it to the residual stream, normalise.
// One kernel does all three.  One CTA per token row:
//   1. push    : the CTA writes its row of this rank's partial block into slot `rank` of every OTHER rank's inbox as
//                8-byte entries {two elements, sequence number} (plain stores through peer pointers).  An 8-byte store
//                is indivisible, so data and "ready" arrive together: no fence, no separate flag, one NVLink latency.
//   2. wait    : every thread polls ITS entries of its own inbox until they carry the row's sequence number.  The wait
//                is bounded: after a set number of polls the row records an error and writes nothing.
//   3. reduce  : h_out = h_in + sum over ranks (fixed order, fp32) of the rows; x = rmsnorm(h_out) * w.
// Rows are independent, so there is no grid-wide step.  Inboxes are double buffered on the parity of the sequence
// number: a rank can be at most one reduction ahead of a peer (it needs that peer's push to finish its own), so a slot
// is never overwritten while a peer still reads it, and an entry left from two reductions ago carries another number.
// The sequence numbers live on the device (one per row, behind the "flags" buffer, advanced by the kernel), so a
// captured CUDA graph can be replayed.  No multicast, no TMA: plain loads and stores.
#include "common.cuh"

namespace dflash {
namespace {

constexpr int kMaxWorld = 8;
uint32_t g_wait_polls = 1u << 22;
int g_protocol = 0;  // 0: by rank count (entries for <= 4 ranks, flags above), 1: entries, 2: flags
// (every rank of a job must use the same protocol)  // polls before a row gives up; with the back-off below a few seconds

struct PeerArgs {
  const uint4* delta;        // this rank's partial block [T, H8]
  uint4* inbox[kMaxWorld];   // inbox of every rank (peer mapped): [2 slots][world][T][H8]
  unsigned* flags[kMaxWorld];  // flag array of every rank: [2 slots][world][T]
  unsigned* seq;             // this rank's per-row sequence numbers [T]
  const uint4* h_in;
  const uint4* w;
  uint4* h_out;
  uint4* x;
  int rank, world, T, H8;
  float eps;
  uint32_t wait_polls;
  int* err;
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T>
__device__ __forceinline__ float tof(T v);
template <>
__device__ __forceinline__ float tof<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float tof<__half>(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T fromf(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 fromf<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half fromf<__half>(float v) { return __float2half_rn(v); }

// Variant for more than four ranks: 16-byte vector pushes, one system-scope fence, one flag per (rank, row) that a single
// thread per rank polls.  With 8 ranks the 8-byte entries of the kernel below cost more NVLink packets and polling
// traffic than they save in latency (measured, dense step: 8 ranks 6.97 ms with flags, 8.32 ms with entries; 4 ranks 5.76
// vs 5.46 ms, 2 ranks 8.91 vs 8.51 ms: the entries win up to 4 ranks).
template <typename T>
__global__ void __launch_bounds__(1024) peer_reduce_flags_kernel(const PeerArgs a) {
  pdl_wait();
  pdl_trigger();
  __shared__ float scratch[32];
  __shared__ int s_fail;
  const int row = blockIdx.x, tid = threadIdx.x;
  constexpr int kMaxV = 2;  // vectors per thread (H <= 8 * 2 * blockDim)
  const unsigned seq = a.seq[row] + 1u;  // sequence number of this reduction for this row (never 0)
  const int slot = (int)(seq & 1u);
  if (tid == 0) s_fail = 0;

  // 1. push this rank's row to every rank's inbox
  const size_t slot_row = ((size_t)(slot * a.world + a.rank) * a.T + row) * a.H8;
  for (int i = tid; i < a.H8; i += blockDim.x) {
    const uint4 v = a.delta[(size_t)row * a.H8 + i];
    for (int p = 0; p < a.world; ++p) a.inbox[p][slot_row + i] = v;
  }
  __threadfence_system();  // the row's stores are ordered before the flags below
  __syncthreads();
  if (tid < a.world) st_release_sys(&a.flags[tid][(slot * a.world + a.rank) * a.T + row], seq);

  // 2. wait for every rank's row (thread q watches rank q)
  if (tid < a.world) {
    const unsigned* f = &a.flags[a.rank][(slot * a.world + tid) * a.T + row];
    bool ok = false;
    for (uint32_t it = 0; it < a.wait_polls; ++it) {
      if (ld_acquire_sys(f) == seq) { ok = true; break; }
      if (it > 64) __nanosleep(it > 4096 ? 400 : 40);
    }
    if (!ok) { atomicExch(&s_fail, 1); atomicExch(a.err, 21); }
  }
  __syncthreads();
  if (tid == 0) a.seq[row] = seq;  // advanced even on failure, so that the ranks stay in step afterwards
  if (s_fail) return;

  // 3. h_out = h_in + sum of the ranks' rows; x = rmsnorm(h_out) * w
  float v[kMaxV][8];
  float ss = 0.f;
  int nv = 0;
  const uint4* mine = a.inbox[a.rank];
  for (int i = tid; i < a.H8 && nv < kMaxV; i += blockDim.x, ++nv) {
    const uint4 hv = a.h_in[(size_t)row * a.H8 + i];
    const T* hp = (const T*)&hv;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int q = 0; q < a.world; ++q) {
      const uint4 d = __ldcg(&mine[((size_t)(slot * a.world + q) * a.T + row) * a.H8 + i]);
      const T* dp = (const T*)&d;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += tof<T>(dp[j]);
    }
    T o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      o[j] = fromf<T>(tof<T>(hp[j]) + acc[j]);
      v[nv][j] = tof<T>(o[j]);
      ss += v[nv][j] * v[nv][j];
    }
    a.h_out[(size_t)row * a.H8 + i] = *(const uint4*)o;
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) scratch[tid >> 5] = ss;
  __syncthreads();
  float tot = (tid & 31) < ((blockDim.x + 31) >> 5) ? scratch[tid & 31] : 0.f;
  tot = warp_sum(tot);
  const float inv = rsqrtf(tot / (float)(a.H8 * 8) + a.eps);
  int k = 0;
  for (int i = tid; i < a.H8 && k < kMaxV; i += blockDim.x, ++k) {
    const uint4 ww = a.w[i];
    const T* wp = (const T*)&ww;
    T o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = fromf<T>(v[k][j] * inv * tof<T>(wp[j]));
    a.x[(size_t)row * a.H8 + i] = *(const uint4*)o;
  }
}

__device__ __forceinline__ void st_entry(uint2* p, uint32_t data, uint32_t seq) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(data), "r"(seq) : "memory");
}
__device__ __forceinline__ uint2 ld_entry(const uint2* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}

template <typename T>
__global__ void __launch_bounds__(1024) peer_reduce_add_rmsnorm_kernel(const PeerArgs a) {
  pdl_wait();
  pdl_trigger();
  __shared__ float scratch[32];
  __shared__ int s_fail;
  const int row = blockIdx.x, tid = threadIdx.x;
  constexpr int kMaxV = 2;  // 16-byte vectors per thread (H <= 8 * 2 * blockDim)
  const unsigned seq = a.seq[row] + 1u;  // sequence number of this reduction for this row (never 0)
  const int slot = (int)(seq & 1u);
  if (tid == 0) s_fail = 0;
  __syncthreads();
  const size_t epr = (size_t)a.H8 * 4;  // 8-byte entries per row: {two elements, sequence number}

  // 1. push: every 32-bit pair of this rank's row goes to slot `rank` of every OTHER rank's inbox together with the
  //    sequence number, in one 8-byte store - data and "ready" arrive together, no fence, no separate flag
  uint4 mine[kMaxV];
  int nv = 0;
  for (int i = tid; i < a.H8 && nv < kMaxV; i += blockDim.x, ++nv) {
    const uint4 v = a.delta[(size_t)row * a.H8 + i];
    mine[nv] = v;
    const size_t e0 = ((size_t)(slot * a.world + a.rank) * a.T + row) * epr + (size_t)i * 4;
    for (int p = 0; p < a.world; ++p) {
      if (p == a.rank) continue;
      uint2* dst = (uint2*)a.inbox[p] + e0;
      st_entry(dst + 0, v.x, seq);
      st_entry(dst + 1, v.y, seq);
      st_entry(dst + 2, v.z, seq);
      st_entry(dst + 3, v.w, seq);
    }
  }

  // 2. + 3. every thread waits for its own entries of the other ranks' rows (bounded), sums them in rank order in fp32,
  //    adds the residual; then x = rmsnorm(h_out) * w
  float v[kMaxV][8];
  float ss = 0.f;
  nv = 0;
  const uint2* inbox = (const uint2*)a.inbox[a.rank];
  for (int i = tid; i < a.H8 && nv < kMaxV; i += blockDim.x, ++nv) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int q = 0; q < a.world; ++q) {
      uint32_t w4[4];
      if (q == a.rank) {
        w4[0] = mine[nv].x; w4[1] = mine[nv].y; w4[2] = mine[nv].z; w4[3] = mine[nv].w;
      } else {
        const uint2* src = inbox + ((size_t)(slot * a.world + q) * a.T + row) * epr + (size_t)i * 4;
        bool ok = false;
        for (uint32_t it = 0; it < a.wait_polls; ++it) {
          const uint2 e0 = ld_entry(src), e1 = ld_entry(src + 1), e2 = ld_entry(src + 2), e3 = ld_entry(src + 3);
          if (e0.y == seq && e1.y == seq && e2.y == seq && e3.y == seq) {
            w4[0] = e0.x; w4[1] = e1.x; w4[2] = e2.x; w4[3] = e3.x;
            ok = true;
            break;
          }
          if (*(volatile int*)&s_fail) break;  // another thread of the row already gave up
          if (it > 64) __nanosleep(it > 4096 ? 400 : 40);
        }
        if (!ok) {
          if (atomicExch(&s_fail, 1) == 0) atomicExch(a.err, 21);
          w4[0] = w4[1] = w4[2] = w4[3] = 0u;
        }
      }
      const T* dp = (const T*)w4;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += tof<T>(dp[j]);
    }
    const uint4 hv = a.h_in[(size_t)row * a.H8 + i];
    const T* hp = (const T*)&hv;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[nv][j] = tof<T>(fromf<T>(tof<T>(hp[j]) + acc[j]));  // the residual stream is stored in T
      ss += v[nv][j] * v[nv][j];
    }
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) scratch[tid >> 5] = ss;
  __syncthreads();
  if (tid == 0) a.seq[row] = seq;  // advanced even on failure, so that the ranks stay in step afterwards
  if (s_fail) return;              // a row that gave up writes nothing
  float tot = (tid & 31) < ((blockDim.x + 31) >> 5) ? scratch[tid & 31] : 0.f;
  tot = warp_sum(tot);
  const float inv = rsqrtf(tot / (float)(a.H8 * 8) + a.eps);
  int k = 0;
  for (int i = tid; i < a.H8 && k < kMaxV; i += blockDim.x, ++k) {
    const uint4 ww = a.w[i];
    const T* wp = (const T*)&ww;
    T ho[8], xo[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      ho[j] = fromf<T>(v[k][j]);
      xo[j] = fromf<T>(v[k][j] * inv * tof<T>(wp[j]));
    }
    a.h_out[(size_t)row * a.H8 + i] = *(const uint4*)ho;
    a.x[(size_t)row * a.H8 + i] = *(const uint4*)xo;
  }
}

}  // namespace
}  // namespace dflash

using namespace dflash;

extern "C" size_t dflash_peer_inbox_bytes(int world, int T_rows, int H) {
  if (world < 1 || world > kMaxWorld || T_rows < 1 || H < 8 || H % 8 != 0) return 0;
  return (size_t)2 * world * T_rows * H * 4;  // 8-byte entries {two elements, sequence number}, two slots
}
extern "C" size_t dflash_peer_flags_bytes(int world, int T_rows) {
  if (world < 1 || world > kMaxWorld || T_rows < 1) return 0;
  return ((size_t)2 * world * T_rows * sizeof(unsigned) + 255) / 256 * 256 + (size_t)T_rows * sizeof(unsigned);
}

extern "C" void dflash_peer_set_protocol(int protocol) { g_protocol = (protocol == 1 || protocol == 2) ? protocol : 0; }
extern "C" void dflash_peer_set_wait_polls(unsigned polls) { g_wait_polls = polls < 1024u ? 1024u : polls; }

extern "C" int dflash_peer_alloc(size_t bytes, void** dev_ptr) {
  if (!dev_ptr || bytes == 0) return fail(DFLASH_ERR_BAD_ARG, "peer_alloc: bad argument");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) {
    if (p) cudaFree(p);
    return fail(DFLASH_ERR_LAUNCH, "peer_alloc(%zu): %s", bytes, cudaGetErrorString(e));
  }
  *dev_ptr = p;
  return DFLASH_OK;
}
extern "C" int dflash_peer_free(void* dev_ptr) {
  if (dev_ptr && cudaFree(dev_ptr) != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "peer_free failed");
  return DFLASH_OK;
}
extern "C" int dflash_peer_export(void* dev_ptr, unsigned char* handle64) {
  if (!dev_ptr || !handle64) return fail(DFLASH_ERR_BAD_ARG, "peer_export: bad argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, dev_ptr);
  if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  memcpy(handle64, &h, 64);
  return DFLASH_OK;
}
extern "C" int dflash_peer_open(const unsigned char* handle64, void** dev_ptr) {
  if (!handle64 || !dev_ptr) return fail(DFLASH_ERR_BAD_ARG, "peer_open: bad argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
  *dev_ptr = p;
  return DFLASH_OK;
}
extern "C" int dflash_peer_close(void* dev_ptr) {
  if (dev_ptr && cudaIpcCloseMemHandle(dev_ptr) != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "cudaIpcCloseMemHandle failed");
  return DFLASH_OK;
}

extern "C" int dflash_peer_reduce_add_rmsnorm(const void* delta, void* const* inbox_ptrs, void* const* flag_ptrs, int rank,
                                              int world, const void* h_in, const void* w, void* h_out, void* x, int T_rows,
                                              int H, float eps, int dtype, void* stream) {
  if (!delta || !inbox_ptrs || !flag_ptrs || !h_in || !w || !h_out || !x)
    return fail(DFLASH_ERR_BAD_ARG, "peer_reduce_add_rmsnorm: null operand");
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || T_rows < 1 || H % 8 != 0 || H > 8 * 2 * 1024)
    return fail(DFLASH_ERR_BAD_SHAPE, "peer_reduce_add_rmsnorm: world 1..8, H %% 8 == 0, H <= 16384");
  auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  if (!al(delta) || !al(h_in) || !al(w) || !al(h_out) || !al(x))
    return fail(DFLASH_ERR_MISALIGNED, "peer_reduce_add_rmsnorm: operands must be 16-byte aligned");
  int device = 0;
  cudaGetDevice(&device);
  PeerArgs a;
  a.delta = (const uint4*)delta;
  for (int p = 0; p < kMaxWorld; ++p) { a.inbox[p] = nullptr; a.flags[p] = nullptr; }
  for (int p = 0; p < world; ++p) {
    if (!inbox_ptrs[p] || !flag_ptrs[p] || !al(inbox_ptrs[p])) return fail(DFLASH_ERR_BAD_ARG, "peer_reduce_add_rmsnorm: bad peer pointer %d", p);
    a.inbox[p] = (uint4*)inbox_ptrs[p];
    a.flags[p] = (unsigned*)flag_ptrs[p];
  }
  // this rank's sequence numbers sit behind its own flag array
  a.seq = (unsigned*)((uint8_t*)flag_ptrs[rank] + ((size_t)2 * world * T_rows * sizeof(unsigned) + 255) / 256 * 256);
  a.h_in = (const uint4*)h_in; a.w = (const uint4*)w; a.h_out = (uint4*)h_out; a.x = (uint4*)x;
  a.rank = rank; a.world = world; a.T = T_rows; a.H8 = H / 8; a.eps = eps;
  a.wait_polls = g_wait_polls;
  a.err = device_error_word(device);
  int threads = (a.H8 + 31) / 32 * 32;
  if (threads > 1024) threads = 1024;
  if (threads < 32 * ((world + 31) / 32)) threads = 32;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  const bool entries = g_protocol == 1 || (g_protocol == 0 && world <= 4);
  if (dtype == DFLASH_BF16)
    e = entries ? launch_kernel(peer_reduce_add_rmsnorm_kernel<__nv_bfloat16>, dim3(T_rows), dim3(threads), 0, st, a)
                : launch_kernel(peer_reduce_flags_kernel<__nv_bfloat16>, dim3(T_rows), dim3(threads), 0, st, a);
  else if (dtype == DFLASH_F16)
    e = entries ? launch_kernel(peer_reduce_add_rmsnorm_kernel<__half>, dim3(T_rows), dim3(threads), 0, st, a)
                : launch_kernel(peer_reduce_flags_kernel<__half>, dim3(T_rows), dim3(threads), 0, st, a);
  else return fail(DFLASH_ERR_BAD_ARG, "peer_reduce_add_rmsnorm: dtype %d (want bf16 or f16)", dtype);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "peer_reduce_add_rmsnorm: %s", cudaGetErrorString(e));
  return DFLASH_OK;
}
