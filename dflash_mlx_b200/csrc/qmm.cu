// M<=16 int4 affine quantised matmul for sm_100a:  y[M,N] = x[M,K] . (nib*scale + bias)[N,K]^T.
//
// Replaces dflash_mlx/verify_qmm.py (Metal kernels `verify_mma2big`, `verify_mma2big_pipe`).
//
// Design (weight streaming, HBM bound):
//   * one persistent CTA per SM: 8 consumer warps + 1 TMA producer warp;
//   * the weight matrix is cut into units of 64 rows x (8 quantisation groups); one unit is one
//     pipeline stage (packed nibbles via 128B-swizzled TMA boxes + its scales + its biases);
//   * K is cut into slabs of <= 2048 columns.  A CTA works inside ONE slab, so its 16 x slabK slice of
//     the activations is loaded once into shared memory and stays there.  The units of a slab are
//     ordered row-tile-major and dealt out to the slab's CTAs as equal contiguous spans (stream-K),
//     so every SM streams the same number of weight bytes;
//   * inside a stage warp w owns quantisation group w for all 64 rows.  The packed words go straight
//     from shared memory to registers; a nibble becomes the bf16 number 128+nib with one LOP3 (the
//     exponent trick) and feeds mma.sync.m16n8k16 as the A operand (16 weight rows x 16 k), the
//     activations are the B operand (16 k x 8 tokens).  The k order inside an MMA is permuted so that
//     one 32-bit word of weights and one 128-bit load of activations line up without shuffles;
//   * scale and bias are applied to the fp32 accumulator once per group:
//         out += s * acc_g + (b - 128 s) * sum_{k in g} x[k]
//     (the group sums of x come from one extra MMA against a matrix of ones), so weights enter the
//     tensor core as exact integers and there is no per-weight FMA;
//   * at the end of a (slab, row tile) segment the 8 warps reduce through shared memory.  If the
//     segment is the tile's only contribution the result is stored directly; otherwise it is written
//     as an fp32 piece to the workspace and the LAST contributor (atomic ticket) sums all pieces in a
//     fixed order - deterministic, no inter-CTA waiting.
#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "common.cuh"

namespace dflash {
namespace {

constexpr int kBN = 64;             // weight rows per unit
constexpr int kConsumerWarps = 8;   // = quantisation groups per unit
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = 2 * kConsumers;  // two workers of 8 warps; thread 0 of a worker also issues its TMA loads
constexpr int kRedBytes = 4 * 8 * 32 * 16;     // per worker: [4 warps][quad][lane] float4
constexpr int kMaxSlabs = 64;
constexpr int kMaxRowTiles = 16384;  // ticket counters kept in a fixed prefix of the workspace

struct QmmPlan {
  int M, K, N, NT, S, maxp;
  int pend_cap;  // partial tiles one worker may write: sizes its list in the workspace (tickets are taken after its last unit)
  int slab_chunk0[kMaxSlabs + 1];
  int slab_cta0[kMaxSlabs + 1];
};

// Expert-gathered variants (mixture-of-experts layers): the weights are E stacked matrices of `block_rows` rows and
// one or more K chunks each, and only the experts listed in slot_expert[0 .. *n_dev) take part.
//   mode 1: ROWS gathered.  y[M, slot * block_rows + r] = x[M,K] . W[slot_expert[slot]][r, :]   (fused gate|up of every
//           active expert; row tile nt reads expert slot nt / block_tiles)
//   mode 2: CHUNKS gathered.  y[M, r] = sum over slots of x[M, slot * Kb .. +Kb) . W[slot_expert[slot]][r, :]   (the
//           experts' down projections, routing weights already folded into x; K chunk c reads expert slot c / cpb)
// The number of active slots is only known on the device, so the work partition is made there (by one thread, into
// shared memory) with the same rules as make_plan().
struct GatherArgs {
  const int* slot_expert;
  const int* n_dev;
  int mode, block_rows, block_tiles, cpb, csmax, blocks;
};

template <int G>
struct Cfg {
  static constexpr int BK = 8 * G;
  static constexpr int kWRowBytes = BK / 2;
  static constexpr int kBoxes = kWRowBytes / 128;
  static constexpr int kWBytes = kBN * kWRowBytes;
  static constexpr int kSBBytes = kBN * 16;
  static constexpr int kStageBytes = kWBytes + 2 * kSBBytes;
  static constexpr int kStages = (G == 128) ? 2 : (G == 64 ? 3 : 5);  // per worker
  static constexpr int WPT = G / 32;  // packed words per thread per weight row
  static constexpr int kSlabKMax = (G == 128) ? 1024 : 2048;
  static constexpr int kXRowBytes = kSlabKMax * 2 + 16;  // +16 B: rows land on different banks
  static constexpr int kXBytes = 16 * kXRowBytes;
  static constexpr size_t kSmemBytes =
      1024 + (size_t)2 * kStages * kStageBytes + kXBytes + 2 * kRedBytes + 8 * (4 * kStages + 1) + 64;
};

// Which weight row of a 16-row tile half a lane group reads: chosen per group size so that the
// swizzled shared-memory reads of a quarter/half warp fall on distinct banks.
template <int G>
__device__ __forceinline__ int row_perm(int g) {
  if (G == 64) return ((g & 3) << 1) | (g >> 2);
  if (G == 128) return (g >> 1) | ((g & 1) << 2);
  return g;
}

// Which CTA of a slab owns unit u when `units` units are dealt out as equal contiguous spans.  The host
// guarantees (units + 1) * ctas < 2^31, so 32-bit arithmetic is exact.
__device__ __forceinline__ int cta_of(unsigned u, unsigned units, unsigned ctas) {
  return (int)(((u + 1u) * ctas - 1u) / units);
}

struct SlabGeom {
  int c0, cs, cta0, ctas;
  unsigned units;
};
__device__ __forceinline__ SlabGeom slab_geom(const QmmPlan& p, int s) {
  SlabGeom g;
  g.c0 = p.slab_chunk0[s];
  g.cs = p.slab_chunk0[s + 1] - g.c0;
  g.cta0 = p.slab_cta0[s];
  g.units = (unsigned)p.NT * (unsigned)g.cs;
  const unsigned ctas = (unsigned)(p.slab_cta0[s + 1] - g.cta0);
  g.ctas = (int)(ctas < g.units ? ctas : g.units);
  return g;
}
// How many CTAs of slab s contribute to row tile nt, and the first of them (slab-local index).
__device__ __forceinline__ int tile_pieces(const SlabGeom& g, int nt, int* first) {
  int a = cta_of((unsigned)nt * g.cs, g.units, g.ctas);
  int b = cta_of((unsigned)(nt + 1) * g.cs - 1u, g.units, g.ctas);
  *first = a;
  return b - a + 1;
}

// make_plan() for a size known only on the device (see GatherArgs); `base` carries M and the padded strides K, N.
__device__ void device_plan(const QmmPlan& base, const GatherArgs& ga, int n, QmmPlan* p) {
  p->M = base.M; p->K = base.K; p->N = base.N;
  int C;
  if (ga.mode == 1) { p->NT = n * ga.block_tiles; C = base.slab_chunk0[base.S]; }
  else { p->NT = base.NT; C = n * ga.cpb; }
  p->S = (C + ga.csmax - 1) / ga.csmax;
  for (int i = 0; i <= p->S; ++i) p->slab_chunk0[i] = (int)((long long)i * C / p->S);
  const long long U = (long long)p->NT * C;
  long long blocks = ga.blocks;
  if (2 * blocks > U + 1) blocks = (U + 1) / 2;
  if (blocks < p->S) blocks = p->S;
  for (int i = 0; i <= p->S; ++i) p->slab_cta0[i] = 2 * (int)(blocks * p->slab_chunk0[i] / C);
  for (int i = 1; i <= p->S; ++i)
    if (p->slab_cta0[i] < p->slab_cta0[i - 1] + 2) p->slab_cta0[i] = p->slab_cta0[i - 1] + 2;
  p->slab_cta0[p->S] = 2 * (int)blocks;
  for (int i = p->S - 1; i >= 1; --i)
    if (p->slab_cta0[i] > p->slab_cta0[i + 1] - 2) p->slab_cta0[i] = p->slab_cta0[i + 1] - 2;
  p->maxp = base.maxp;  // the host's bounds for the largest case (they size the workspace)
  p->pend_cap = base.pend_cap;
}

// Output element ownership after the cross-warp reduction: consumer thread (warp, lane) holds, for row
// tile nt, weight rows n_lo = 64 nt + 16 (warp>>1) + rp and n_lo + 8, tokens tok = 8 (warp&1) + 2 c and tok+1.
template <typename T>
__device__ __forceinline__ void store_tile(const float4& v, T* __restrict__ y, const T* __restrict__ bias, int nt,
                                           int warp, int rp, int c, int M, int N) {
  using TR = MmaTraits<T>;
  const int n_lo = nt * kBN + 16 * (warp >> 1) + rp, n_hi = n_lo + 8;
  const int tok = 8 * (warp & 1) + 2 * c;
  float bl0 = 0.f, bh0 = 0.f;
  if (bias != nullptr) {
    if (n_lo < N) bl0 = TR::to_float(bias[n_lo]);
    if (n_hi < N) bh0 = TR::to_float(bias[n_hi]);
  }
  if (n_lo < N) {
    if (tok < M) y[(size_t)tok * N + n_lo] = TR::from_float(v.x + bl0);
    if (tok + 1 < M) y[(size_t)(tok + 1) * N + n_lo] = TR::from_float(v.y + bl0);
  }
  if (n_hi < N) {
    if (tok < M) y[(size_t)tok * N + n_hi] = TR::from_float(v.z + bh0);
    if (tok + 1 < M) y[(size_t)(tok + 1) * N + n_hi] = TR::from_float(v.w + bh0);
  }
}

// Run by the CTA that took the last ticket of row tile nt: sum the fp32 pieces in a fixed order.
template <typename T>
__device__ __noinline__ void finalize_tile(const QmmPlan& plan, const float4* pieces, unsigned* counters,
                                           T* __restrict__ y, const T* __restrict__ bias, int nt, int ctid, int warp,
                                           int rp, int c) {
  // First the slot list (integer divisions only), then the loads eight at a time so that their latencies overlap,
  // then the sum in slot order (fixed order: deterministic).
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  int s2 = 0, p = 0, np = 0;
  {
    int f;
    np = tile_pieces(slab_geom(plan, 0), nt, &f);
  }
  bool more = true;
  while (more) {
    const float4* src[8];
    int n = 0;
    while (n < 8) {
      if (p >= np) {
        if (++s2 >= plan.S) { more = false; break; }
        int f;
        np = tile_pieces(slab_geom(plan, s2), nt, &f);
        p = 0;
        continue;
      }
      src[n++] = &pieces[((size_t)(s2 * plan.maxp + p) * plan.NT + nt) * kConsumers + ctid];
      ++p;
    }
    float4 a[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < n) a[i] = ld_cg_f4(src[i]);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < n) { v.x += a[i].x; v.y += a[i].y; v.z += a[i].z; v.w += a[i].w; }
  }
  if (ctid == 0) counters[nt] = 0;  // ready for the next launch
  store_tile<T>(v, y, bias, nt, warp, rp, c, plan.M, plan.N);
}

// Variant for products with many K slabs (the chunk-gathered expert product: dozens of pieces per row tile), run by
// the worker (256 threads) that took the last ticket of row tile nt; same summation order as finalize_tile.
// The list of pieces (integer divisions per K slab) is built once, by the lanes of the worker's first warp in parallel,
// into `scratch` (shared memory, >= 4 * (1 + S * maxp) bytes); then every thread sums its element over the list, eight
// loads in flight at a time.  Order = slab-major, then piece index: deterministic.
template <typename T>
__device__ __noinline__ void finalize_tile_coop(const QmmPlan& plan, const float4* pieces, unsigned* counters,
                                           T* __restrict__ y, const T* __restrict__ bias, int nt, int ctid, int warp,
                                           int rp, int c, int* scratch, int bar_id) {
  const int lane = ctid & 31;
  if (warp == 0) {
    int base = 0;
    for (int s0 = 0; s0 < plan.S; s0 += 32) {
      const int s2 = s0 + lane;
      int np = 0;
      if (s2 < plan.S) {
        int f;
        np = tile_pieces(slab_geom(plan, s2), nt, &f);
      }
      int incl = np;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      const int excl = base + incl - np;
      for (int p = 0; p < np; ++p) scratch[1 + excl + p] = s2 * plan.maxp + p;
      base += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) scratch[0] = base;
  }
  named_bar_sync(bar_id, kConsumers);
  const int P = scratch[0];
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int k0 = 0; k0 < P; k0 += 8) {
    float4 a[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (k0 + i < P) a[i] = ld_cg_f4(&pieces[((size_t)scratch[1 + k0 + i] * plan.NT + nt) * kConsumers + ctid]);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (k0 + i < P) { v.x += a[i].x; v.y += a[i].y; v.z += a[i].z; v.w += a[i].w; }
  }
  if (ctid == 0) counters[nt] = 0;  // ready for the next launch
  store_tile<T>(v, y, bias, nt, warp, rp, c, plan.M, plan.N);
  named_bar_sync(bar_id, kConsumers);  // `scratch` may be rebuilt for the next tile
}

template <typename T, int G, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
qmm_stream_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmS,
                  const __grid_constant__ CUtensorMap tmB, const T* __restrict__ x, const T* __restrict__ bias,
                  T* __restrict__ y, float4* __restrict__ pieces, unsigned* __restrict__ counters,
                  const __grid_constant__ QmmPlan base_plan, int* __restrict__ err, const int dependent,
                  const __grid_constant__ GatherArgs ga, int* __restrict__ pend_ws) {
  using C = Cfg<G>;
  using TR = MmaTraits<T>;
  extern __shared__ uint8_t smem_raw[];
  const QmmPlan* plan_ptr = &base_plan;
  if constexpr (MODE != 0) {
    // the partition depends on the number of active expert slots, which the routing kernel left on the device
    __shared__ QmmPlan dyn_plan;
    __shared__ int dyn_n;
    pdl_wait();  // n_dev and slot_expert are written by an earlier kernel of the stream
    if (threadIdx.x == 0) {
      const int n = *ga.n_dev;
      dyn_n = n;
      if (n > 0) device_plan(base_plan, ga, n, &dyn_plan);
    }
    __syncthreads();
    if (dyn_n <= 0) {  // no active expert on this rank: a chunk-gathered product is all zeros, a row-gathered one is empty
      if (MODE == 2)
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)base_plan.M * base_plan.N;
             i += (size_t)gridDim.x * blockDim.x)
          y[i] = TR::from_float(0.f);
      return;
    }
    plan_ptr = &dyn_plan;
  }
  const QmmPlan& plan = *plan_ptr;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Two independent workers share the CTA (and its activation slab): warps 0-7 are worker 0, warps 8-15
  // worker 1.  Each owns a span of units, a ring of stages and its barriers; its first thread issues the
  // TMA loads (kStages-1 units ahead), so all 16 warps compute and each SM sub-partition holds 4 warps.
  const int worker = warp >> 3;
  const int wwarp = warp & 7;  // warp index inside the worker

  uint8_t* stages = smem + (size_t)worker * C::kStages * C::kStageBytes;
  uint8_t* xbuf = smem + (size_t)2 * C::kStages * C::kStageBytes;
  float4* red = (float4*)(xbuf + C::kXBytes + (size_t)worker * kRedBytes);
  uint64_t* bars = (uint64_t*)(xbuf + C::kXBytes + 2 * kRedBytes);
  const uint32_t bar_full = smem_u32(bars) + worker * 16 * C::kStages, bar_empty = bar_full + 8 * C::kStages;
  const uint32_t bar_x = smem_u32(bars) + 32 * C::kStages;

  // ---- which slab, which span of its units (virtual CTA = 2 * blockIdx.x + worker) ----
  const int vcta = 2 * (int)blockIdx.x + worker;
  int s = 0;
  while (s + 1 < plan.S && 2 * (int)blockIdx.x >= plan.slab_cta0[s + 1]) ++s;  // slab starts are even
  const SlabGeom sg = slab_geom(plan, s);
  const int bl = vcta - sg.cta0;
  const bool has_work = bl < sg.ctas;
  if (2 * (int)blockIdx.x - sg.cta0 >= sg.ctas) return;  // neither worker has units
  const unsigned u_begin = has_work ? (unsigned)bl * sg.units / sg.ctas : 0u;
  const unsigned u_end = has_work ? (unsigned)(bl + 1) * sg.units / sg.ctas : 0u;
  const int NT = plan.NT, M = plan.M, K = plan.K, N = plan.N;
  const int slabK = sg.cs * C::BK;

  if (threadIdx.x == 0) {
    for (int w = 0; w < 2; ++w)
      for (int i = 0; i < C::kStages; ++i) {
        mbar_init(smem_u32(bars) + w * 16 * C::kStages + 8 * i, 1);                                   // full
        mbar_init(smem_u32(bars) + w * 16 * C::kStages + 8 * C::kStages + 8 * i, kConsumerWarps);     // empty
      }
    mbar_init(bar_x, 1);
    mbar_fence_init();
  }
  __syncthreads();

  // =============================== consumers ===============================
  const int ctid = threadIdx.x & (kConsumers - 1);  // 0..255 inside the worker
  const int g = lane >> 2, c = lane & 3;
  const int rp = row_perm<G>(g);
  const int bar_id = 1 + worker;
  bool aborted = false;
  // Row tiles for which this worker has written a partial tile but not yet taken its ticket.  Tickets are
  // taken in batches (one gpu-scope fence per batch, normally one per kernel at the end of the span, when no
  // loads are in flight), by a thread that does not issue TMA loads.
  // this worker's list of written partial tiles, in the workspace: [row tile | contributors | last?] x pend_cap
  const int kMaxPend = plan.pend_cap;
  volatile int* pend = (volatile int*)pend_ws + (size_t)vcta * 3 * kMaxPend;
  int npend = 0;
  auto flush_tickets = [&]() {
    named_bar_sync(bar_id, kConsumers);  // every pending partial-tile store has been issued
    if (ctid == 32) {
      __threadfence();  // cumulative over the worker's stores (observed through the barrier)
      for (int i0 = 0; i0 < npend; i0 += 8) {  // 8 tickets in flight at a time
        unsigned t[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (i0 + j < npend) t[j] = atomicAdd(&counters[pend[i0 + j]], 1u);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (i0 + j < npend) pend[2 * kMaxPend + i0 + j] = (t[j] == (unsigned)(pend[kMaxPend + i0 + j] - 1));
      }
      __threadfence();
    }
    named_bar_sync(bar_id, kConsumers);
    for (int i = 0; i < npend; ++i)
      if (pend[2 * kMaxPend + i]) {
        // many K slabs: build the list of pieces cooperatively; few: every thread walks the slabs itself
        if (plan.S > 4) finalize_tile_coop<T>(plan, pieces, counters, y, bias, pend[i], ctid, wwarp, rp, c, (int*)red, bar_id);
        else finalize_tile<T>(plan, pieces, counters, y, bias, pend[i], ctid, wwarp, rp, c);
      }
    named_bar_sync(bar_id, kConsumers);
  };

  // ---- TMA issue (thread 0 of the worker): the classic producer sequence, run kStages-1 units ahead ----
  const uint64_t pol_stream = l2_policy_evict_first(), pol_keep = l2_policy_evict_last();
  int pstage = 0, pnt = (int)(u_begin / sg.cs), pkc = (int)(u_begin % sg.cs);
  uint32_t ppar = 1;
  unsigned pu = u_begin;
  auto issue_one = [&]() {
    if (pu >= u_end) return;
    if (!mbar_wait(bar_empty + 8 * pstage, ppar)) { atomicExch(err, 1); pu = u_end; return; }
    const uint32_t full = bar_full + 8 * pstage;
    const uint32_t dst = smem_u32(stages + pstage * C::kStageBytes);
    mbar_arrive_expect_tx(full, C::kStageBytes);
    int wrow = pnt * kBN, wchunk = sg.c0 + pkc;  // first weight row and K chunk of the unit inside the stacked weights
    if constexpr (MODE == 1) {
      wrow = (ga.slot_expert[pnt / ga.block_tiles] * ga.block_tiles + pnt % ga.block_tiles) * kBN;
    } else if constexpr (MODE == 2) {
      wrow = ga.slot_expert[wchunk / ga.cpb] * ga.block_rows + pnt * kBN;
      wchunk = wchunk % ga.cpb;
    }
#pragma unroll
    for (int j = 0; j < C::kBoxes; ++j)
      tma_load_2d(dst + j * (kBN * 128), &tmW, wchunk * C::kWRowBytes + 128 * j, wrow, full, pol_stream);
    tma_load_2d(dst + C::kWBytes, &tmS, wchunk * 8, wrow, full, pol_keep);
    tma_load_2d(dst + C::kWBytes + C::kSBBytes, &tmB, wchunk * 8, wrow, full, pol_keep);
    if (++pstage == C::kStages) { pstage = 0; ppar ^= 1; }
    if (++pkc == sg.cs) { pkc = 0; ++pnt; }
    ++pu;
  };
  // A dependent launch (blocks may start while the previous kernel of the stream drains) requests its first weight
  // stages - written by no kernel - before it waits for that kernel, and the activations (its output) after; every
  // store of this kernel comes after the wait too.  An ordinary launch asks for the small, L2-resident activation
  // slab first so that it does not queue behind the weight stages.
  auto issue_x = [&]() {
    mbar_arrive_expect_tx(bar_x, (uint32_t)(M * slabK * 2));
    for (int r = 0; r < M; ++r)
      bulk_load_1d(smem_u32(xbuf + r * C::kXRowBytes), x + (size_t)r * K + (size_t)sg.c0 * C::BK,
                   (uint32_t)(slabK * 2), bar_x);
  };
  if (!dependent && threadIdx.x == 0) issue_x();
  if (ctid == 0) {
#pragma unroll 1
    for (int j = 0; j < C::kStages - 1; ++j) issue_one();
  }
  if (dependent) {
    pdl_wait();
    pdl_trigger();
    if (threadIdx.x == 0) issue_x();
  }

  // rows >= M of the activation slab are zeros (all 512 threads take part)
  for (int r = M; r < 16; ++r)
    for (int i = threadIdx.x; i < slabK * 2 / 16; i += 2 * kConsumers)
      ((uint4*)(xbuf + r * C::kXRowBytes))[i] = make_uint4(0, 0, 0, 0);
  named_bar_sync(3, 2 * kConsumers);
  if (!has_work) return;
  if (!mbar_wait(bar_x, 0)) { aborted = true; atomicExch(err, 2); }

  float out[4][2][4];
#pragma unroll
  for (int t = 0; t < 4; ++t)
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int j = 0; j < 4; ++j) out[t][h][j] = 0.f;

  // position of this warp's group inside a stage row: box, first 16-byte chunk
  constexpr int kGroupBytes = G / 2;
  const int box = (wwarp * kGroupBytes) >> 7;
  const int lbyte = ((wwarp * kGroupBytes) & 127) + c * 4 * C::WPT;  // logical byte inside the 128-byte box row
  const int phys = ((((lbyte >> 4) ^ rp) << 4) | (lbyte & 15));      // 128B swizzle: chunk ^= (row & 7)

  int stage = 0;
  uint32_t par = 0;
  int nt = (int)(u_begin / sg.cs), kc = (int)(u_begin % sg.cs);
  for (unsigned u = u_begin; u < u_end; ++u) {
    if (ctid == 0) issue_one();  // refills the stage that unit u-1 used
    __syncwarp();
    if (!aborted && !mbar_wait(bar_full + 8 * stage, par)) { aborted = true; atomicExch(err, 3); }
    const uint8_t* st = stages + stage * C::kStageBytes;

    // ---- activation fragments (B operand) of this warp's group, both token halves ----
    uint32_t xb[2][2 * C::WPT][2];
    float xs[2][4];
    {
      const uint8_t* xcol = xbuf + (size_t)(kc * C::BK + wwarp * G + c * 8 * C::WPT) * 2;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint4* p = (const uint4*)(xcol + (g + 8 * h) * C::kXRowBytes);
#pragma unroll
        for (int i = 0; i < C::WPT; ++i) {
          const uint4 X = p[i];
          xb[h][2 * i][0] = prmt(X.x, X.z, 0x5410);      // (k0, k4)
          xb[h][2 * i][1] = prmt(X.x, X.z, 0x7632);      // (k1, k5)
          xb[h][2 * i + 1][0] = prmt(X.y, X.w, 0x5410);  // (k2, k6)
          xb[h][2 * i + 1][1] = prmt(X.y, X.w, 0x7632);  // (k3, k7)
        }
        xs[h][0] = xs[h][1] = xs[h][2] = xs[h][3] = 0.f;
      }
#pragma unroll
      for (int m = 0; m < 2 * C::WPT; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          TR::mma(xs[h], TR::kOnes, TR::kOnes, TR::kOnes, TR::kOnes, xb[h][m][0], xb[h][m][1]);
    }

    const uint16_t* S16 = (const uint16_t*)(st + C::kWBytes);
    const uint16_t* B16 = (const uint16_t*)(st + C::kWBytes + C::kSBBytes);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int r_lo = 16 * t + rp;
      const uint8_t* wl = st + box * (kBN * 128) + r_lo * 128 + phys;
      const uint8_t* wh = wl + 8 * 128;
      uint32_t U[C::WPT], V[C::WPT];
      if constexpr (C::WPT == 1) {
        U[0] = *(const uint32_t*)wl;
        V[0] = *(const uint32_t*)wh;
      } else if constexpr (C::WPT == 2) {
        const uint2 a = *(const uint2*)wl, b = *(const uint2*)wh;
        U[0] = a.x; U[1] = a.y;
        V[0] = b.x; V[1] = b.y;
      } else {
        const uint4 a = *(const uint4*)wl, b = *(const uint4*)wh;
        U[0] = a.x; U[1] = a.y; U[2] = a.z; U[3] = a.w;
        V[0] = b.x; V[1] = b.y; V[2] = b.z; V[3] = b.w;
      }
      const float s_lo = TR::bits_to_float(S16[r_lo * 8 + wwarp]), s_hi = TR::bits_to_float(S16[(r_lo + 8) * 8 + wwarp]);
      const float b_lo = TR::bits_to_float(B16[r_lo * 8 + wwarp]), b_hi = TR::bits_to_float(B16[(r_lo + 8) * 8 + wwarp]);
      const float bq_lo = fmaf(-TR::kMagicValue, s_lo, b_lo), bq_hi = fmaf(-TR::kMagicValue, s_hi, b_hi);

      float acc[2][4];
#pragma unroll
      for (int h = 0; h < 2; ++h) acc[h][0] = acc[h][1] = acc[h][2] = acc[h][3] = 0.f;
#pragma unroll
      for (int i = 0; i < C::WPT; ++i) {
        uint32_t PU[4], PV[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          PU[q] = lop3_and_or(U[i] >> (4 * q), 0x000F000Fu, TR::kMagic);  // (nib q, nib q+4) as 128+nib
          PV[q] = lop3_and_or(V[i] >> (4 * q), 0x000F000Fu, TR::kMagic);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) TR::mma(acc[h], PU[0], PV[0], PU[1], PV[1], xb[h][2 * i][0], xb[h][2 * i][1]);
#pragma unroll
        for (int h = 0; h < 2; ++h)
          TR::mma(acc[h], PU[2], PV[2], PU[3], PV[3], xb[h][2 * i + 1][0], xb[h][2 * i + 1][1]);
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        out[t][h][0] = fmaf(s_lo, acc[h][0], fmaf(bq_lo, xs[h][0], out[t][h][0]));
        out[t][h][1] = fmaf(s_lo, acc[h][1], fmaf(bq_lo, xs[h][1], out[t][h][1]));
        out[t][h][2] = fmaf(s_hi, acc[h][2], fmaf(bq_hi, xs[h][0], out[t][h][2]));
        out[t][h][3] = fmaf(s_hi, acc[h][3], fmaf(bq_hi, xs[h][1], out[t][h][3]));
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_empty + 8 * stage);
    if (++stage == C::kStages) { stage = 0; par ^= 1; }

    const bool seg_end = (kc == sg.cs - 1) || (u == u_end - 1);
    if (seg_end) {
      // ---- reduce the 8 warps' partial tiles through shared memory, in two rounds of 16 KB ----
      if (wwarp >= 4) {
#pragma unroll
        for (int q = 0; q < 8; ++q)
          red[((wwarp - 4) * 8 + q) * 32 + lane] =
              make_float4(out[q >> 1][q & 1][0], out[q >> 1][q & 1][1], out[q >> 1][q & 1][2], out[q >> 1][q & 1][3]);
      }
      named_bar_sync(bar_id, kConsumers);
      if (wwarp < 4) {  // warp w folds warp w+4's tile into its own and puts the sum back in the same slots
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float4 a = red[(wwarp * 8 + q) * 32 + lane];
          red[(wwarp * 8 + q) * 32 + lane] =
              make_float4(out[q >> 1][q & 1][0] + a.x, out[q >> 1][q & 1][1] + a.y, out[q >> 1][q & 1][2] + a.z,
                          out[q >> 1][q & 1][3] + a.w);
        }
      }
#pragma unroll
      for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int h = 0; h < 2; ++h) out[t][h][0] = out[t][h][1] = out[t][h][2] = out[t][h][3] = 0.f;
      named_bar_sync(bar_id, kConsumers);
      // thread (wwarp, lane) finalises quad q = wwarp = (row tile wwarp>>1, token half wwarp&1) of lane `lane`
      float4 v = red[(0 * 8 + wwarp) * 32 + lane];
#pragma unroll
      for (int w2 = 1; w2 < 4; ++w2) {
        const float4 a = red[(w2 * 8 + wwarp) * 32 + lane];
        v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
      }
      // pieces this row tile receives in total, and this worker's piece index inside its slab
      int total = 0, first_here = 0;
      for (int s2 = lane; s2 < plan.S; s2 += 32) {
        const SlabGeom g2 = slab_geom(plan, s2);
        int f;
        total += tile_pieces(g2, nt, &f);
      }
      total = __reduce_add_sync(0xffffffffu, total);
      tile_pieces(sg, nt, &first_here);

      if (total > 1) {
        pieces[((size_t)(s * plan.maxp + (bl - first_here)) * NT + nt) * kConsumers + ctid] = v;
      } else {
        store_tile<T>(v, y, bias, nt, wwarp, rp, c, M, N);
      }
      if (total > 1) {
        if (npend < kMaxPend) {
          if (ctid == 0) { pend[npend] = nt; pend[kMaxPend + npend] = total; }
          ++npend;
        } else if (ctid == 0) {
          atomicExch(err, 4);  // cannot happen for a plan the host accepted
        }
      }
      named_bar_sync(bar_id, kConsumers);  // `red` is free again
    }
    if (++kc == sg.cs) { kc = 0; ++nt; }
  }
  if (npend > 0) flush_tickets();
}

// ------------------------------------------------------------------------------------------
// General kernel: any K % 32 == 0, K % G == 0, any N, any alignment of the row starts.  One warp per
// output column; exact fp32 dequantisation.  Used for shapes the streaming kernel does not take.
template <typename T>
__global__ void __launch_bounds__(256) qmm_general_kernel(const T* __restrict__ x, const uint32_t* __restrict__ wq,
                                                          const T* __restrict__ scales, const T* __restrict__ biases,
                                                          const T* __restrict__ bias, T* __restrict__ y, int M, int K,
                                                          int N, int G) {
  using TR = MmaTraits<T>;
  pdl_wait();
  pdl_trigger();
  const int n = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (n >= N) return;
  float acc[16];
#pragma unroll
  for (int m = 0; m < 16; ++m) acc[m] = 0.f;
  const int words = K / 8, groups = K / G;
  for (int j = lane; j < words; j += 32) {
    const uint32_t w = wq[(size_t)n * words + j];
    const int grp = (j * 8) / G;
    const float s = TR::to_float(scales[(size_t)n * groups + grp]), b = TR::to_float(biases[(size_t)n * groups + grp]);
    float wv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) wv[i] = fmaf((float)((w >> (4 * i)) & 0xF), s, b);
#pragma unroll
    for (int m = 0; m < 16; ++m) {
      if (m < M) {
        const T* xr = x + (size_t)m * K + j * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[m] = fmaf(TR::to_float(xr[i]), wv[i], acc[m]);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < 16; ++m) {
    float v = acc[m];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0 && m < M) y[(size_t)m * N + n] = TR::from_float(v + (bias ? TR::to_float(bias[n]) : 0.f));
  }
}

// ------------------------------------------------------------------------------------------
int g_max_blocks = 0;
int g_k_parts = 0;  // > 0: K is cut into at least this many slabs (dflash_verify_qmm_set_k_parts)
int g_impl = 0;  // 0 = by shape and dtype (tcgen05 kernel wherever it applies: bf16, group 64, K % 512 == 0), 1 = mma.sync
                 // streaming kernel always, 2 = tcgen05 kernel wherever it applies
long long g_tc_min_weights = 0;  // N*K from which impl 0 picks the tcgen05 kernel (measured faster at every size)
thread_local int g_last_impl = 0;  // 1 = mma.sync streaming kernel, 2 = tcgen05 kernel, 3 = general kernel

bool make_plan(int M, int K, int N, int G, int device, QmmPlan* p, bool gathered = false) {
  const int BK = 8 * G;
  const int C = K / BK;
  const int csmax = (G == 128 ? 1024 : 2048) / BK;
  p->M = M; p->K = K; p->N = N;
  p->NT = (N + kBN - 1) / kBN;
  p->S = (C + csmax - 1) / csmax;
  if (!gathered && g_k_parts > p->S) p->S = g_k_parts < C ? g_k_parts : C;  // (the device-side re-plan has no such knob)
  if (p->S > kMaxSlabs || p->NT > kMaxRowTiles) return false;
  for (int i = 0; i <= p->S; ++i) p->slab_chunk0[i] = (int)((long long)i * C / p->S);
  const long long U = (long long)p->NT * C;
  // Work is dealt to "workers": two per thread block.  A block's two workers share one activation slab,
  // so every slab starts at an even worker index and gets at least one block.
  long long blocks = g_max_blocks > 0 ? g_max_blocks : sm_count(device);
  if (2 * blocks > U + 1) blocks = (U + 1) / 2;
  if (blocks < p->S) blocks = p->S;
  for (int i = 0; i <= p->S; ++i) p->slab_cta0[i] = 2 * (int)(blocks * p->slab_chunk0[i] / C);
  for (int i = 1; i <= p->S; ++i)
    if (p->slab_cta0[i] < p->slab_cta0[i - 1] + 2) p->slab_cta0[i] = p->slab_cta0[i - 1] + 2;
  p->slab_cta0[p->S] = 2 * (int)blocks;
  for (int i = p->S - 1; i >= 1; --i)
    if (p->slab_cta0[i] > p->slab_cta0[i + 1] - 2) p->slab_cta0[i] = p->slab_cta0[i + 1] - 2;
  int maxp = 1, cap = 4;
  for (int i = 0; i < p->S; ++i) {
    const int cs = p->slab_chunk0[i + 1] - p->slab_chunk0[i];
    const long long Us = (long long)p->NT * cs;
    long long ctas = p->slab_cta0[i + 1] - p->slab_cta0[i];
    if (ctas > Us) ctas = Us;
    const long long L = Us / ctas;
    const long long touched = (L + 1 + cs - 1) / cs + 2;  // row tiles one worker's span can touch
    if (touched > cap) cap = (int)touched;
    const int mp = (int)((cs - 1 + L - 1) / L) + 1;
    if (cs > 1 && mp > maxp) maxp = mp;
    if ((Us + 1) * (p->slab_cta0[i + 1] - p->slab_cta0[i]) >= (1ll << 31)) return false;
  }
  p->maxp = maxp;
  p->pend_cap = cap;
  return true;
}

// The ticket counters sit in a fixed-size prefix of the workspace, so that the bytes they occupy never
// hold anything else (the workspace is zero-filled once and shared by calls of every shape).
size_t counters_bytes(int) { return (size_t)kMaxRowTiles * 4; }
// then the workers' lists of written partial tiles (sized for one worker pair per SM), then the partial tiles
size_t pend_bytes(const QmmPlan& p, int device) {
  // workers of this plan (two per block); an expert-gathered launch always uses one block per SM (or the cap) but at
  // least one per K slab of its largest case
  size_t workers = (size_t)p.slab_cta0[p.S];
  const size_t full = 2 * (size_t)(g_max_blocks > 0 ? g_max_blocks : sm_count(device));
  if (workers < full) workers = full;
  return (workers * 3 * p.pend_cap * sizeof(int) + 255) / 256 * 256;
}
size_t plan_workspace(const QmmPlan& p, int device) {
  return counters_bytes(p.NT) + pend_bytes(p, device) + (size_t)p.S * p.maxp * p.NT * kConsumers * sizeof(float4);
}

bool fast_path_ok(const void* x, const void* wq, const void* sc, const void* bi, int K, int G) {
  if (K % (8 * G) != 0) return false;
  auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  return al(x) && al(wq) && al(sc) && al(bi);
}

struct MapKey {
  const void* p; int rows, inner, kind;
  bool operator==(const MapKey& o) const { return p == o.p && rows == o.rows && inner == o.inner && kind == o.kind; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.p) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.inner * 7919u) ^ (size_t)k.kind;
  }
};
std::mutex g_map_mu;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

// kind 0: packed weights, uint8 [rows, inner bytes], box 128 x 64, 128B swizzle.
// kind 1: scales / biases, uint16 [rows, inner elements], box 8 x 64, no swizzle.
bool get_map(const void* ptr, int rows, int inner, int kind, CUtensorMap* out) {
  MapKey key{ptr, rows, inner, kind};
  {
    std::lock_guard<std::mutex> lk(g_map_mu);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return true; }
  }
  tensormap_encode_fn enc = get_tensormap_encoder();
  if (!enc) return false;
  CUtensorMap m;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r;
  if (kind == 0) {
    cuuint64_t strides[1] = {(cuuint64_t)inner};
    cuuint32_t box[2] = {128, (cuuint32_t)kBN};
    r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    cuuint64_t strides[1] = {(cuuint64_t)inner * 2};
    cuuint32_t box[2] = {8, (cuuint32_t)kBN};
    r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed (%d) rows=%d inner=%d kind=%d", (int)r, rows, inner, kind);
    return false;
  }
  std::lock_guard<std::mutex> lk(g_map_mu);
  if (g_maps.size() > 16384) g_maps.clear();
  g_maps.emplace(key, m);
  *out = m;
  return true;
}

template <typename T, int G>
int launch_stream(const void* x, const void* wq, const void* sc, const void* bi, const void* bias, void* y,
                  const QmmPlan& plan, void* ws, cudaStream_t st, int device) {
  using C = Cfg<G>;
  CUtensorMap tw, ts, tb;
  if (!get_map(wq, plan.N, plan.K / 2, 0, &tw) || !get_map(sc, plan.N, plan.K / G, 1, &ts) ||
      !get_map(bi, plan.N, plan.K / G, 1, &tb))
    return DFLASH_ERR_LAUNCH;
  auto kern = qmm_stream_kernel<T, G, 0>;
  static bool attr_done[64] = {};
  if (!attr_done[device & 63]) {
    cudaError_t e0 = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::kSmemBytes);
    if (e0 != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e0));
    attr_done[device & 63] = true;
  }
  cudaError_t e;
  unsigned* counters = (unsigned*)ws;
  int* pend_ws = (int*)((uint8_t*)ws + counters_bytes(plan.NT));
  float4* pieces = (float4*)((uint8_t*)pend_ws + pend_bytes(plan, device));
  const int grid = plan.slab_cta0[plan.S] / 2;
  const bool dependent = pdl_enabled_for_next_launch();
  e = launch_kernel_as(dependent, kern, dim3(grid), dim3(kThreads), C::kSmemBytes, st, tw, ts, tb, (const T*)x,
                       (const T*)bias, (T*)y, pieces, counters, plan, device_error_word(device), dependent ? 1 : 0,
                       GatherArgs{}, pend_ws);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "qmm launch: %s", cudaGetErrorString(e));
  return DFLASH_OK;
}

// Expert-gathered launch (see GatherArgs).  E stacked expert matrices of block_rows x Kb.
template <typename T, int MODE>
int launch_gather(const void* x, const void* wq, const void* sc, const void* bi, void* y, int M, int E, int block_rows,
                  int Kb, const int* slot_expert, const int* n_dev, int n_max, void* ws, size_t ws_bytes,
                  cudaStream_t st) {
  constexpr int G = 64;
  using C = Cfg<G>;
  int device = 0;
  cudaGetDevice(&device);
  QmmPlan plan;
  const int K = MODE == 1 ? Kb : n_max * Kb, N = MODE == 1 ? n_max * block_rows : block_rows;
  if (!make_plan(M, K, N, G, device, &plan, true)) return fail(DFLASH_ERR_BAD_SHAPE, "moe_qmm: shape too large");
  plan.maxp = C::kSlabKMax / C::BK + 1;  // bound for every number of active slots
  const size_t need = plan_workspace(plan, device);
  if (ws == nullptr || ws_bytes < need)
    return fail(DFLASH_ERR_WORKSPACE, "moe_qmm needs %zu workspace bytes, got %zu", need, ws_bytes);
  if (((uintptr_t)ws & 255) != 0) return fail(DFLASH_ERR_MISALIGNED, "workspace must be 256-byte aligned");
  CUtensorMap tw, ts, tb;
  if (!get_map(wq, E * block_rows, Kb / 2, 0, &tw) || !get_map(sc, E * block_rows, Kb / G, 1, &ts) ||
      !get_map(bi, E * block_rows, Kb / G, 1, &tb))
    return DFLASH_ERR_LAUNCH;
  auto kern = qmm_stream_kernel<T, G, MODE>;
  static bool attr_done[64] = {};
  if (!attr_done[device & 63]) {
    cudaError_t e0 = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::kSmemBytes);
    if (e0 != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e0));
    attr_done[device & 63] = true;
  }
  GatherArgs ga;
  ga.slot_expert = slot_expert; ga.n_dev = n_dev; ga.mode = MODE; ga.block_rows = block_rows;
  ga.block_tiles = block_rows / kBN; ga.cpb = Kb / C::BK; ga.csmax = C::kSlabKMax / C::BK;
  ga.blocks = g_max_blocks > 0 ? g_max_blocks : sm_count(device);
  if (ga.blocks < plan.S) ga.blocks = plan.S;  // every K slab of the largest case gets a block
  unsigned* counters = (unsigned*)ws;
  int* pend_ws = (int*)((uint8_t*)ws + counters_bytes(plan.NT));
  float4* pieces = (float4*)((uint8_t*)pend_ws + pend_bytes(plan, device));
  const bool dependent = pdl_enabled_for_next_launch();
  cudaError_t e = launch_kernel_as(dependent, kern, dim3(ga.blocks), dim3(kThreads), C::kSmemBytes, st, tw, ts, tb,
                                   (const T*)x, (const T*)nullptr, (T*)y, pieces, counters, plan,
                                   device_error_word(device), dependent ? 1 : 0, ga, pend_ws);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "moe_qmm launch: %s", cudaGetErrorString(e));
  return DFLASH_OK;
}

template <typename T>
int launch_any(const void* x, const void* wq, const void* sc, const void* bi, const void* bias, void* y, int M, int K,
               int N, int G, void* ws, size_t ws_bytes, cudaStream_t st) {
  int device = 0;
  cudaGetDevice(&device);
  if ((g_impl == 2 || (g_impl == 0 && (long long)N * K >= g_tc_min_weights)) && G == 64 && sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value && fast_path_ok(x, wq, sc, bi, K, G) &&
      ((uintptr_t)ws & 255) == 0) {
    const int rc = tc::launch(x, wq, sc, bi, bias, y, M, K, N, ws, ws_bytes, st, device, g_max_blocks);
    if (rc <= 0) { g_last_impl = 2; return rc; }
  }
  QmmPlan plan;
  if (fast_path_ok(x, wq, sc, bi, K, G) && make_plan(M, K, N, G, device, &plan)) {
    const size_t need = plan_workspace(plan, device);
    if (ws == nullptr || ws_bytes < need)
      return fail(DFLASH_ERR_WORKSPACE, "verify_qmm needs %zu workspace bytes, got %zu", need, ws_bytes);
    if (((uintptr_t)ws & 255) != 0) return fail(DFLASH_ERR_MISALIGNED, "workspace must be 256-byte aligned");
    g_last_impl = 1;
    switch (G) {
      case 32: return launch_stream<T, 32>(x, wq, sc, bi, bias, y, plan, ws, st, device);
      case 64: return launch_stream<T, 64>(x, wq, sc, bi, bias, y, plan, ws, st, device);
      default: return launch_stream<T, 128>(x, wq, sc, bi, bias, y, plan, ws, st, device);
    }
  }
  g_last_impl = 3;
  cudaError_t e = launch_kernel(qmm_general_kernel<T>, dim3((N + 7) / 8), dim3(256), 0, st, (const T*)x,
                                (const uint32_t*)wq, (const T*)sc, (const T*)bi, (const T*)bias, (T*)y, M, K, N, G);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DFLASH_ERR_LAUNCH, "qmm general launch: %s", cudaGetErrorString(e));
  return DFLASH_OK;
}

}  // namespace
}  // namespace dflash

using namespace dflash;

extern "C" void dflash_verify_qmm_set_max_blocks(int max_blocks) { g_max_blocks = max_blocks < 0 ? 0 : max_blocks; }
extern "C" void dflash_verify_qmm_set_k_parts(int k_parts) {
  g_k_parts = k_parts < 0 ? 0 : k_parts;
  tc::set_k_parts(g_k_parts);
}

extern "C" size_t dflash_verify_qmm_workspace_bytes(int M, int K, int N, int group_size) {
  if (M < 1 || K < 1 || N < 1 || (group_size != 32 && group_size != 64 && group_size != 128)) return 0;
  if (K % (8 * group_size) != 0) return 256;  // general kernel: no workspace (a token amount keeps callers uniform)
  int device = 0;
  cudaGetDevice(&device);
  QmmPlan plan;
  if (!make_plan(M, K, N, group_size, device, &plan)) return 256;
  size_t need = plan_workspace(plan, device);
  if (group_size == 64) {
    const size_t t = tc::workspace_bytes(M, K, N, device, g_max_blocks);
    if (t > need) need = t;
  }
  return need;
}

namespace {
// An announcement (dflash_verify_qmm_prefetch_next) is good for exactly one call, whichever kernel that call ends up in:
// a hint left pending could outlive the weights it names.
struct NextHintScope {
  ~NextHintScope() { dflash::tc::set_next(nullptr, nullptr, nullptr, 0, 0); }
};
}  // namespace

extern "C" size_t dflash_moe_qmm_workspace_bytes(int M, int block_rows, int Kb, int n_max, int mode) {
  if (M < 1 || M > 16 || block_rows < kBN || block_rows % kBN != 0 || Kb < 512 || Kb % 512 != 0 || n_max < 1 ||
      (mode != 1 && mode != 2))
    return 0;
  int device = 0;
  cudaGetDevice(&device);
  QmmPlan plan;
  const int K = mode == 1 ? Kb : n_max * Kb, N = mode == 1 ? n_max * block_rows : block_rows;
  if (!make_plan(M, K, N, 64, device, &plan, true)) return 0;
  plan.maxp = Cfg<64>::kSlabKMax / Cfg<64>::BK + 1;
  const size_t a = plan_workspace(plan, device), b = tc::gather_workspace_bytes(M, block_rows, Kb, n_max, mode, device, g_max_blocks);
  return a > b ? a : b;   // either kernel may run (dflash_verify_qmm_set_impl)
}

extern "C" int dflash_moe_qmm(const void* x, const void* w_q, const void* scales, const void* biases, void* y, int M,
                              int experts, int block_rows, int Kb, int mode, const int* slot_expert, const int* n_active,
                              int n_max, int dtype, void* workspace, size_t workspace_bytes, void* stream) {
  NextHintScope hint_scope;
  if (!x || !w_q || !scales || !biases || !y || !slot_expert || !n_active)
    return fail(DFLASH_ERR_BAD_ARG, "moe_qmm: null operand");
  if (M < 1 || M > 16 || experts < 1 || n_max < 1 || n_max > experts || (mode != 1 && mode != 2))
    return fail(DFLASH_ERR_BAD_ARG, "moe_qmm: need 1 <= M <= 16, 1 <= n_max <= experts, mode 1 or 2");
  if (block_rows < kBN || block_rows % kBN != 0 || Kb < 512 || Kb % 512 != 0)
    return fail(DFLASH_ERR_BAD_SHAPE, "moe_qmm: block_rows %% 64 == 0 and Kb %% 512 == 0 (group size 64)");
  auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  if (!al(x) || !al(w_q) || !al(scales) || !al(biases)) return fail(DFLASH_ERR_MISALIGNED, "moe_qmm: operands must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == DFLASH_BF16 && g_impl != 1 && ((uintptr_t)workspace & 255) == 0) {   // the tcgen05 kernel where it applies
    int device = 0;
    cudaGetDevice(&device);
    const int rc = tc::launch_gather(x, w_q, scales, biases, y, M, experts, block_rows, Kb, mode, slot_expert, n_active, n_max,
                                     workspace, workspace_bytes, st, device, g_max_blocks);
    if (rc <= 0) { if (rc == 0) g_last_impl = 2; return rc; }
  }
  g_last_impl = 1;
  if (dtype == DFLASH_BF16)
    return mode == 1 ? launch_gather<__nv_bfloat16, 1>(x, w_q, scales, biases, y, M, experts, block_rows, Kb, slot_expert, n_active, n_max, workspace, workspace_bytes, st)
                     : launch_gather<__nv_bfloat16, 2>(x, w_q, scales, biases, y, M, experts, block_rows, Kb, slot_expert, n_active, n_max, workspace, workspace_bytes, st);
  if (dtype == DFLASH_F16)
    return mode == 1 ? launch_gather<__half, 1>(x, w_q, scales, biases, y, M, experts, block_rows, Kb, slot_expert, n_active, n_max, workspace, workspace_bytes, st)
                     : launch_gather<__half, 2>(x, w_q, scales, biases, y, M, experts, block_rows, Kb, slot_expert, n_active, n_max, workspace, workspace_bytes, st);
  return fail(DFLASH_ERR_BAD_ARG, "moe_qmm: dtype %d (want bf16 or f16)", dtype);
}

extern "C" int dflash_moe_qmm_fused_supported(int M, int block_rows, int Kb, int n_max, int mode, int dtype) {
  return (dtype == DFLASH_BF16 && g_impl != 1 && M >= 1 && M <= 16 && block_rows >= 128 && block_rows % 128 == 0 && Kb >= 512 &&
          Kb % 512 == 0 && n_max >= 1 && n_max <= 272 && (mode == 1 || mode == 2)) ? 1 : 0;
}

extern "C" int dflash_moe_qmm_fused(const void* x, const void* w_q, const void* scales, const void* biases, void* y, int M,
                                    int experts, int block_rows, int Kb, int mode, const int* slot_expert,
                                    const int* n_active, int n_max, int dtype, const dflash_qmm_epilogue* ep,
                                    void* workspace, size_t workspace_bytes, void* stream) {
  NextHintScope hint_scope;
  if (!x || !w_q || !scales || !biases || !y || !slot_expert || !n_active || !ep)
    return fail(DFLASH_ERR_BAD_ARG, "moe_qmm_fused: null operand");
  if (n_max > experts || !dflash_moe_qmm_fused_supported(M, block_rows, Kb, n_max, mode, dtype))
    return fail(DFLASH_ERR_BAD_SHAPE, "moe_qmm_fused: needs bf16, 1 <= M <= 16, block_rows %% 128 == 0, Kb %% 512 == 0, n_max <= 272");
  if (ep->mode != 0 && !(ep->mode == 1 && mode == 2))
    return fail(DFLASH_ERR_BAD_ARG, "moe_qmm_fused: epilogue mode %d with gather mode %d (0 anywhere, 1 on the summed output)", ep->mode, mode);
  if (ep->in_ssq != nullptr && (ep->in_parts < 1 || !(ep->in_dim > 0.f) || ((uintptr_t)ep->in_ssq & 15) != 0))
    return fail(DFLASH_ERR_BAD_ARG, "moe_qmm_fused: in_ssq needs in_parts >= 1, in_dim > 0 and 16-byte alignment");
  if (ep->mode == 1 && (!ep->residual || ((const void*)ep->scaled == (const void*)y && ep->scaled)))
    return fail(DFLASH_ERR_BAD_ARG, "moe_qmm_fused: mode 1 needs a residual, and scaled must not alias y");
  auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  if (!al(x) || !al(w_q) || !al(scales) || !al(biases) || ((uintptr_t)workspace & 255) != 0)
    return fail(DFLASH_ERR_MISALIGNED, "moe_qmm_fused: operands must be 16-byte, the workspace 256-byte aligned");
  int device = 0;
  cudaGetDevice(&device);
  const int rc = tc::launch_gather(x, w_q, scales, biases, y, M, experts, block_rows, Kb, mode, slot_expert, n_active, n_max,
                                   workspace, workspace_bytes, (cudaStream_t)stream, device, g_max_blocks, ep);
  if (rc > 0) return fail(DFLASH_ERR_BAD_SHAPE, "moe_qmm_fused: shape not handled by the tcgen05 kernel");
  if (rc == 0) g_last_impl = 2;
  return rc;
}

extern "C" void dflash_verify_qmm_set_impl(int impl) { g_impl = (impl == 2) ? 2 : (impl == 1 ? 1 : 0); }
extern "C" int dflash_verify_qmm_last_impl(void) { return g_last_impl; }
extern "C" void dflash_verify_qmm_set_stamps(void* dev_buffer) { tc::set_stamps(dev_buffer); }

extern "C" void dflash_verify_qmm_prefetch_next(const void* w_q, const void* scales, const void* biases, int K, int N) {
  tc::set_next(w_q, scales, biases, K, N);
}
extern "C" void dflash_verify_qmm_set_prefetch_next(int on) { tc::set_prefetch_next(on); }
extern "C" void dflash_verify_qmm_set_tc_roles(int dequant_warps, int issuing_threads) {
  tc::set_roles(dequant_warps, issuing_threads);
}

extern "C" int dflash_verify_qmm(const void* x, const void* w_q, const void* scales, const void* biases,
                                 const void* bias, void* y, int M, int K, int N, int group_size, int dtype,
                                 void* workspace, size_t workspace_bytes, void* stream) {
  NextHintScope hint_scope;
  if (!x || !w_q || !scales || !biases || !y) return fail(DFLASH_ERR_BAD_ARG, "verify_qmm: null operand");
  if (M < 1 || M > 16) return fail(DFLASH_ERR_BAD_SHAPE, "verify_qmm: M=%d outside 1..16", M);
  if (group_size != 32 && group_size != 64 && group_size != 128)
    return fail(DFLASH_ERR_BAD_SHAPE, "verify_qmm: group_size=%d not in {32,64,128}", group_size);
  if (K < group_size || K % group_size != 0 || K % 32 != 0 || N < 1)
    return fail(DFLASH_ERR_BAD_SHAPE, "verify_qmm: K=%d N=%d not supported (K %% G == 0, K %% 32 == 0)", K, N);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == DFLASH_BF16)
    return launch_any<__nv_bfloat16>(x, w_q, scales, biases, bias, y, M, K, N, group_size, workspace, workspace_bytes, st);
  if (dtype == DFLASH_F16)
    return launch_any<__half>(x, w_q, scales, biases, bias, y, M, K, N, group_size, workspace, workspace_bytes, st);
  return fail(DFLASH_ERR_BAD_ARG, "verify_qmm: dtype %d (want bf16 or f16)", dtype);
}

extern "C" int dflash_verify_qmm_fused_supported(int M, int K, int N, int group_size, int dtype) {
  return (M >= 1 && M <= 16 && N >= 1 && group_size == 64 && dtype == DFLASH_BF16 && K >= 512 && K % 512 == 0) ? 1 : 0;
}

extern "C" int dflash_verify_qmm_fused(const void* x, const void* w_q, const void* scales, const void* biases,
                                       const void* bias, void* y, int M, int K, int N, int group_size, int dtype,
                                       const dflash_qmm_epilogue* ep, void* workspace, size_t workspace_bytes,
                                       void* stream) {
  NextHintScope hint_scope;
  if (!x || !w_q || !scales || !biases || !y || !ep) return fail(DFLASH_ERR_BAD_ARG, "verify_qmm_fused: null operand");
  if (!dflash_verify_qmm_fused_supported(M, K, N, group_size, dtype))
    return fail(DFLASH_ERR_BAD_SHAPE, "verify_qmm_fused: needs bf16, group size 64, K %% 512 == 0, M in 1..16 (M=%d K=%d N=%d G=%d)",
                M, K, N, group_size);
  if (ep->mode < 0 || ep->mode > 2) return fail(DFLASH_ERR_BAD_ARG, "verify_qmm_fused: mode %d", ep->mode);
  if (ep->in_ssq != nullptr && (ep->in_parts < 1 || !(ep->in_dim > 0.f) || ((uintptr_t)ep->in_ssq & 15) != 0))
    return fail(DFLASH_ERR_BAD_ARG, "verify_qmm_fused: in_ssq needs in_parts >= 1, in_dim > 0 and 16-byte alignment");
  if (ep->mode == 1 && !ep->residual) return fail(DFLASH_ERR_BAD_ARG, "verify_qmm_fused: mode 1 needs a residual");
  if (ep->mode == 1 && (const void*)ep->scaled == (const void*)y && ep->scaled) return fail(DFLASH_ERR_BAD_ARG, "verify_qmm_fused: scaled aliases y");
  if (ep->mode == 2 && (N % 2 != 0 || bias != nullptr))
    return fail(DFLASH_ERR_BAD_SHAPE, "verify_qmm_fused: mode 2 needs an even N and no bias");
  if (ep->mode == 1 && bias != nullptr) return fail(DFLASH_ERR_BAD_ARG, "verify_qmm_fused: mode 1 takes no bias");
  if (!fast_path_ok(x, w_q, scales, biases, K, group_size) || ((uintptr_t)workspace & 255) != 0)
    return fail(DFLASH_ERR_MISALIGNED, "verify_qmm_fused: operands must be 16-byte, the workspace 256-byte aligned");
  int device = 0;
  cudaGetDevice(&device);
  const int rc = tc::launch(x, w_q, scales, biases, bias, y, M, K, N, workspace, workspace_bytes, (cudaStream_t)stream, device,
                            g_max_blocks, ep);
  if (rc > 0) return fail(DFLASH_ERR_BAD_SHAPE, "verify_qmm_fused: shape not handled by the tcgen05 kernel");
  if (rc == 0) g_last_impl = 2;
  return rc;
}

extern "C" int dflash_verify_qmm_plan(int M, int K, int N, int group_size, int* out, int capacity) {
  if (!out || (group_size != 32 && group_size != 64 && group_size != 128) || K % (8 * group_size) != 0)
    return fail(DFLASH_ERR_BAD_ARG, "verify_qmm_plan: bad arguments");
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) { cudaGetLastError(); device = 0; }
  QmmPlan p;
  if (!make_plan(M, K, N, group_size, device, &p)) return fail(DFLASH_ERR_BAD_SHAPE, "verify_qmm_plan: too many K slabs");
  const int need = 4 + 2 * (p.S + 1);
  if (capacity < need) return fail(DFLASH_ERR_BAD_ARG, "verify_qmm_plan: capacity %d < %d", capacity, need);
  out[0] = p.NT; out[1] = p.S; out[2] = p.maxp; out[3] = p.slab_cta0[p.S];
  for (int i = 0; i <= p.S; ++i) { out[4 + i] = p.slab_chunk0[i]; out[4 + p.S + 1 + i] = p.slab_cta0[i]; }
  return need;
}
