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

/* Programmatic dependent launch (no counterpart in the reference; Metal orders its dispatches itself).
 * When on (default; environment DFLASH_PDL=0 turns it off), every kernel of this library is launched so
 * that its blocks may be scheduled while the previous kernel of the same stream is still draining; each
 * kernel waits on the device for that previous kernel to finish before it reads or writes anything a
 * kernel may have produced, so results do not change.  Works in plain streams and under stream capture.
 *   dflash_set_pdl(on)              process-wide switch
 *   dflash_pdl_plain_next(n)        the next n launches made by the calling thread are ordinary,
 *                                   fully serialised launches (use after work of another library that
 *                                   was joined into the stream through an event, e.g. a collective) */
DFLASH_API void dflash_set_pdl(int on);
DFLASH_API int dflash_get_pdl(void);
DFLASH_API void dflash_pdl_plain_next(int launches);

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
/* verify_qmm with the neighbouring element-wise work of a verify step folded into its epilogue, so that a decoder
 * layer is a chain of matmuls with no small kernels between them (the reference leaves these to MLX's lazy graph:
 * `rms_norm`, the residual `+` and `swiglu` around every quantised linear, mlx-lm's decoder layer as hooked by
 * dflash_mlx/runtime.py:351-452 and :515-613).  Only for shapes dflash_verify_qmm_fused_supported() accepts (bf16,
 * group size 64, K % 512 == 0); anything else is refused, nothing falls back.
 *   mode 0  y[M,N] = acc * inv (+ bias)
 *   mode 1  y = residual + acc, stored in bf16 (`residual` may be y itself: the residual stream is updated in
 *           place); scaled[M,N] = y * next_w[N] (NULL: not written); out_ssq[4*ceil(N/128)][16] floats (NULL: not
 *           written) = partial sums of y^2 per token, one per 32-row slice.  `scaled` and `out_ssq` are what the next
 *           matmul takes as x / in_ssq: together they are the RMSNorm that follows, never materialised.
 *   mode 2  the weight rows are interleaved (gate_0, up_0, gate_1, up_1, ...); y[M,N/2] = silu(gate) * up with gate
 *           and up rounded to bf16 first, as the unfused sequence does.
 *   in_ssq  NULL, or float[in_parts][16] partial sums of squares of the un-normalised input tokens (16-byte aligned):
 *           inv[t] = rsqrt(sum_p in_ssq[p][t] / in_dim + eps) multiplies the accumulators (x then is `scaled` of a
 *           mode-1 call: a per-token factor commutes with the matmul).  Partial sums are added in a fixed order. */
typedef struct dflash_qmm_epilogue {
  int mode;
  int in_parts;
  float in_dim;
  float eps;
  const float* in_ssq;
  const void* residual;
  const void* next_w;
  void* scaled;
  float* out_ssq;
} dflash_qmm_epilogue;
DFLASH_API int dflash_verify_qmm_fused_supported(int M, int K, int N, int group_size, int dtype);
DFLASH_API int dflash_verify_qmm_fused(const void* x, const void* w_q, const void* scales, const void* biases,
                                       const void* bias, void* y, int M, int K, int N, int group_size, int dtype,
                                       const dflash_qmm_epilogue* epilogue, void* workspace, size_t workspace_bytes,
                                       void* stream);
/* Tuning/testing knob: caps the number of thread blocks the fast kernel uses (0 = one per SM). */
DFLASH_API void dflash_verify_qmm_set_max_blocks(int max_blocks);
/* Tuning knob with the meaning of the reference's DFLASH_VERIFY_QMM_KPARTS (dflash_mlx/verify_qmm.py:297): K is cut
 * into at least `k_parts` slabs whose partial sums are combined in a fixed order (0 = as few as the kernel's
 * activation buffer allows, the default). */
DFLASH_API void dflash_verify_qmm_set_k_parts(int k_parts);
/* Kernel choice: 0 (default) = the tcgen05 kernel (weights dequantised to bf16 in tensor memory, accumulator in TMEM)
 * wherever it applies - bf16, group size 64, K % 512 == 0, 16-byte aligned operands - else the mma.sync streaming
 * kernel; 1 = mma.sync kernel always (exact integer nibbles, scale applied to the accumulator: the variant for error
 * attribution); 2 = as 0. */
DFLASH_API void dflash_verify_qmm_set_impl(int impl);
/* Tuning knob of the tcgen05 kernel: how many warps dequantise (8 or 12); the number of threads that
 * issue MMAs is fixed (6) and the second argument is ignored.  Other values leave the setting alone.  Results do not depend on it beyond fp32 summation order. */
DFLASH_API void dflash_verify_qmm_set_tc_roles(int dequant_warps, int issuing_threads);
/* Measurement aid: with a device buffer of 16 * 8 bytes per thread block (one block per SM) the tcgen05 kernel
 * records, per block, %globaltimer at entry [0] and exit [1] and the SM clock at entry [2], set-up done [3], first
 * activation tile landed [4], first pipeline stage complete [5], first operand ready for the tensor core [6], last MMA
 * issued [7], last accumulators ready [8], last output written [9], exit [10].  NULL (default) turns it off. */
DFLASH_API void dflash_verify_qmm_set_stamps(void* dev_buffer);
/* Announces the verify matmul that follows the NEXT dflash_verify_qmm / dflash_verify_qmm_fused call of this thread in
 * the stream (its packed weights, scales, biases, K, N; group size 64).  That next call's kernel then pulls the first units
 * of the announced weights into L2 once its own requests are all issued, so the announced matmul starts from L2 instead
 * of a cold HBM ramp (~2 us per launch in a verify step, where one matmul follows another).  A hint: consumed by one
 * call, ignored when either matmul does not run the tensor-memory kernel; results never depend on it.
 * dflash_verify_qmm_set_prefetch_next(0) turns the hints off (measurements). */
DFLASH_API void dflash_verify_qmm_prefetch_next(const void* w_q, const void* scales, const void* biases, int K, int N);
DFLASH_API void dflash_verify_qmm_set_prefetch_next(int on);
/* Which kernel the calling thread's last dflash_verify_qmm ran: 1 = mma.sync streaming, 2 = tcgen05, 3 = general. */
DFLASH_API int dflash_verify_qmm_last_impl(void);
/* Introspection for host-side tests (needs no GPU): writes the streaming kernel's work partition for a
 * shape as ints {row_tiles, slabs, max_pieces, blocks, slab_chunk0[slabs+1], slab_block0[slabs+1]} and
 * returns how many ints were written (<0 on error). */
DFLASH_API int dflash_verify_qmm_plan(int M, int K, int N, int group_size, int* out, int capacity);

/* ---------------------------------------------------------------------------------------------
 * GatedDeltaNet forward with innovation tape (tape record).
 * Replaces `gated_delta_kernel_with_tape` and the Metal kernels `gated_delta_tape[_vec][_mask]`
 * (dflash_mlx/kernels.py:176-224, 29-105).  Per step t < T, on state S[Dv,Dk] of head hv:
 *   S *= g_t ; kv = S k_t ; delta_t = (v_t - kv) * beta_t ; S += delta_t (x) k_t ; y_t = S q_t
 * and, when the state dtype is not f32, S is rounded to it after every step (kernels.py:89-91).
 *   q,k   in_dtype [B,T,Hk,Dk];  v in_dtype [B,T,Hv,Dv];  beta f32 [B,T,Hv]
 *   g     f32 [B,T,Hv] (g_is_vector=0) or [B,T,Hv,Dk] (g_is_vector=1): the decay FACTOR in (0,1]
 *   mask  uint8 [B,T] or NULL; a masked-out step leaves S unchanged and writes delta = 0, y = 0
 *   state_in/state_out  state_dtype [B,Hv,Dv,Dk], 16-byte aligned (may be the same buffer)
 *   y     in_dtype [B,T,Hv,Dv];  tape f32 [B,T,Hv,Dv]
 * Dk in {32,64,128,256}; Hv % Hk == 0 (head hv reads k-head hv / (Hv/Hk), kernels.py:33).
 */
DFLASH_API int dflash_gdn_forward_tape(const void* q, const void* k, const void* v, const float* g, const float* beta,
                                       const uint8_t* mask, const void* state_in, void* state_out, void* y, float* tape,
                                       int B, int T, int Hk, int Hv, int Dk, int Dv, int g_is_vector, int in_dtype,
                                       int state_dtype, void* stream);

/* Tape replay (rollback): applies the first `steps` tape entries to state_in.
 * Replaces `tape_replay_kernel` and the Metal kernels `tape_replay[_vec][_mask]`
 * (dflash_mlx/kernels.py:361-407, 244-294):  S *= g_t ; S += delta_t (x) k_t  for t < steps.
 *   tape f32 [B,T,Hv,Dv];  k k_dtype [B,T,Hk,Dk];  g f32 as above;  mask uint8 [B,T] or NULL
 *   T is the length the arrays were recorded with (their stride); 0 <= steps <= T; steps == 0 copies.
 *   steps_dev, when not NULL, is a device int that overrides `steps` at run time (clamped to 0..T), so
 *   that a captured CUDA graph can replay a different accepted length every time.
 * To roll back every layer of a model in one launch, stack the layers' arrays along B.
 */
DFLASH_API int dflash_tape_replay(const float* tape, const void* k, const float* g, const uint8_t* mask,
                                  const void* state_in, void* state_out, int B, int T, int steps, const int* steps_dev,
                                  int Hk, int Hv, int Dk, int Dv, int g_is_vector, int k_dtype, int state_dtype,
                                  void* stream);
/* Testing knob: for scalar gates, no mask, fp32 state, Dk = 128 and bf16 k the replay runs a pure-stream kernel (packed
 * fp32 pair arithmetic, bit-identical results): 1 (default) = persistent blocks fed by bulk copies through a shared-
 * memory pipeline (T <= 16, Dv % 4 == 0, 16-byte aligned tape and k), 2 = one block per 64 rows, 0 = the general kernel
 * everywhere. */
DFLASH_API void dflash_tape_replay_set_stream_kernel(int mode);
/* Testing knob for dflash_gdn_forward_tape: 1 (default) = the low-latency record kernel where it applies (scalar gate, no
 * mask, Dk = 128, bf16 inputs, fp32 state, T <= 16, 16-byte aligned q and k: a state row over 8 lanes, both row
 * reductions of a step in one shuffle chain, y_t = S' q_t + delta_t (k_t . q_t)); 0 = the general kernel everywhere.
 * The two agree to fp32 rounding (another summation order), not bit for bit; either one's tape replays to its own
 * state bit for bit. */
DFLASH_API void dflash_gdn_forward_set_kernel(int mode);
/* One-shot promise for this thread's next dflash_gdn_forward_tape call: the kernel launched before it in the stream does
 * not write state_in (true in a verify step, false when one call's state_out feeds the next call).  The low-latency record
 * kernel then requests the state rows before its wait on that kernel.  Results do not change. */
DFLASH_API void dflash_gdn_forward_state_is_settled(void);
/* dflash_gdn_forward_tape (low-latency record kernel: bf16 inputs, fp32 state, Dk = 128, Dv % 16 == 0 and <= 128, scalar
 * gate, no mask, T <= 16) followed by the gated RMSNorm that consumes its output (runtime.py:445), in ONE launch: the
 * Dv / 16 blocks of a head form a thread-block cluster and add up the norm's partial sums through distributed shared
 * memory.  out[b*T + t, hv*Dv + d] = bf16(bf16(y) * rsqrt(mean y^2 + eps) * norm_w[d]) * silu(z[b*T + t, z_off + hv*Dv + d])
 * (z: bf16 rows of z_ld elements, out: bf16 rows of out_ld elements); y itself is not stored.  State and tape are bit
 * for bit those of dflash_gdn_forward_tape. */
DFLASH_API int dflash_gdn_forward_tape_norm_supported(int T, int Hk, int Hv, int Dk, int Dv, int in_dtype, int state_dtype);
DFLASH_API int dflash_gdn_forward_tape_norm(const void* q, const void* k, const void* v, const float* g, const float* beta,
                                            const void* state_in, void* state_out, float* tape, const void* z, long long z_ld,
                                            int z_off, const void* norm_w, void* out, long long out_ld, int B, int T, int Hk,
                                            int Hv, int Dk, int Dv, float eps, int in_dtype, int state_dtype, void* stream);

/* ---------------------------------------------------------------------------------------------
 * verify_sdpa: exact softmax attention of 16 query rows per head over N keys (split-KV + combine).
 * Replaces `batched_sdpa_2pass_exact` and the Metal kernels `batched_sdpa_2pass_partials[_mask]` /
 * `batched_sdpa_2pass_reduce` (dflash_mlx/kernels.py:658-761, 479-565, 579-638).
 *   q    dtype [B,Hq,16,D] contiguous;  out likewise
 *   k,v  dtype [B,Hk,N,D]: element (b,h,n,d) at ((b*Hk+h)*head_stride + n*seq_stride + d); strides in
 *        elements, multiples of 8 (rows 16-byte aligned).  N counts the 16 new positions (runtime.py:550-555)
 *   key n is visible to row i iff n <= N-16+i (kernels.py:530); head hq reads KV head hq/(Hq/Hk)
 *   mask dtype [B,Hq,16,N] additive, or NULL; entries below the dtype's finite minimum hide the key
 *   D in {128,256};  dtype bf16 or f16;  scale multiplies q.k
 *   num_splits: 0 = chosen from the SM count; workspace: dflash_verify_sdpa_workspace_bytes() bytes of
 *   device memory (contents irrelevant), 16-byte aligned; unused when the split count comes out as 1.
 */
DFLASH_API size_t dflash_verify_sdpa_workspace_bytes(int B, int Hq, int Hk, int N, int D, int num_splits);
DFLASH_API int dflash_verify_sdpa(const void* q, const void* k, const void* v, const void* mask, void* out, int B,
                                  int Hq, int Hk, int N, int D, long long k_head_stride, long long k_seq_stride,
                                  long long v_head_stride, long long v_seq_stride, float scale, int dtype,
                                  int num_splits, void* workspace, size_t workspace_bytes, void* stream);
/* Kernel choice for verify_sdpa: 0 (default) = the tcgen05 kernel (K/V by TMA, S = Q K^T and O = P V on the tensor
 * cores with S / P / O in tensor memory, 256 keys per block, bf16 partials) where it applies - bf16, no mask array,
 * num_splits = 0, at most 8 query heads per KV head - else the mma.sync kernel; 1 = the mma.sync kernel always; 2 = as 0
 * but with the combine pass inside the same launch (the blocks of a KV head meet on a counter and share it) whenever the
 * whole grid is resident, i.e. has at most one block per SM - measured slower than the second launch, so not the
 * default; 3 = as 0 with 128 keys per block while that keeps the grid within one block per SM (no faster either).  With
 * the device-side KV length (dflash_verify_sdpa_dev_len) the tcgen05 kernel reads cache rows up to the next multiple of
 * 64 beyond the length: they must hold finite values (they get weight zero). */
DFLASH_API void dflash_verify_sdpa_set_impl(int impl);

/* verify_sdpa for callers that cannot allocate device memory.  (No counterpart in the reference.)
 * Some hosts of this library - a serving loop that has handed all device memory to its own pool, code
 * running inside a CUDA-graph capture, a plugin slot that forbids allocator calls - cannot obtain the
 * split-KV workspace dflash_verify_sdpa asks for.  This entry point computes exactly the same result with the
 * partial-softmax scratch kept in an array built into the library (dflash_verify_sdpa_static_capacity()
 * bytes, 32 MiB, held on every GPU that loads the library until the process exits).  It calls no
 * cudaMalloc / cudaFree and no allocating library routine; inputs and the output are still the caller's.
 *   - Same arguments as dflash_verify_sdpa, minus the workspace.  Shapes whose scratch need
 *     (dflash_verify_sdpa_workspace_bytes) exceeds the capacity are refused with DFLASH_ERR_WORKSPACE.
 *   - The first call on each device resolves the array's device address (that device must be current); make
 *     that first call before any stream capture.
 *   - The array is shared by every call and keeps the previous call's contents.  Nothing in it has to start
 *     at zero (pass 1 writes every slot pass 2 reads), but two calls that overlap on the GPU (different
 *     streams, or graphs replayed concurrently) race on it: serialise them.
 */
DFLASH_API size_t dflash_verify_sdpa_static_capacity(void);
DFLASH_API int dflash_verify_sdpa_static(const void* q, const void* k, const void* v, const void* mask, void* out, int B,
                                         int Hq, int Hk, int N, int D, long long k_head_stride, long long k_seq_stride,
                                         long long v_head_stride, long long v_seq_stride, float scale, int dtype,
                                         int num_splits, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Fused element-wise / normalisation kernels between the matmuls of a verify step.  They restate the
 * layer dataflow of the reference's model hooks; dtype is bf16 or f16, arithmetic fp32, T_rows token rows.
 */
/* h_out = h_in + delta (delta may be NULL; h_out may be NULL or alias h_in); x = rms_norm(h_out) * w.
 * The residual add and the layer norms around every mixer / MLP (mlx-lm decoder layer called at runtime.py:802-809). */
DFLASH_API int dflash_add_rmsnorm(const void* h_in, const void* delta, const void* w, void* h_out, void* x, int T_rows,
                                  int H, float eps, int dtype, void* stream);
/* y[t,i] = silu(gate_up[t,i]) * gate_up[t,I+i]: SwiGLU on a fused [gate | up] projection (mlx-lm MLP). */
DFLASH_API int dflash_swiglu(const void* gate_up, void* y, int T_rows, int I, int dtype, void* stream);
/* h[t,:] = table[ids[t],:]  (embed_tokens, runtime.py:788). */
DFLASH_API int dflash_embed(const int* ids, const void* table, void* h, int T_rows, int H, int V, int dtype, void* stream);
/* dflash_embed plus the inputs of a dflash_verify_qmm_fused call that applies the first layer's RMSNorm:
 * scaled[t,:] = h[t,:] * next_w[:], ssq[t] = sum of h[t,:]^2 (float[16], entries T_rows..15 are left alone:
 * zero them once; in_parts = 1). */
DFLASH_API int dflash_embed_scaled(const int* ids, const void* table, const void* next_w, void* h, void* scaled, float* ssq,
                                   int T_rows, int H, int V, int dtype, void* stream);
/* out[t] = first index of the maximum of logits[t,:]  (greedy_tokens_with_mask, runtime.py:90-98). */
DFLASH_API int dflash_argmax(const void* logits, int* out, int T_rows, int V, int dtype, void* stream);
/* The same with the reference's suppress_token_mask: suppress[v] != 0 (uint8[V], device; NULL = none) makes token v's
 * logit count as -1e9 rounded to the logits' type, as `mx.where(mask, floor, logits)` does (runtime.py:90-98). */
DFLASH_API int dflash_argmax_masked(const void* logits, const uint8_t* suppress, int* out, int T_rows, int V, int dtype,
                                    void* stream);
/* Acceptance and commit of one speculative cycle on the device, one launch (runtime.py:101-108, 878-907;
 * recurrent_rollback_cache.py:148-171).  block_ids[n_tokens] = [staged token, drafted tokens]; posterior[n_tokens] =
 * the target's greedy tokens.  *n_accepted = number of leading drafted tokens that match, *steps = *n_accepted + 1;
 * if offset != NULL: *offset += *steps and (kv_len != NULL) *kv_len = *offset + kv_len_extra.  For each of `layers`
 * GatedDeltaNet layers conv_new[l] ([keep, conv_dim]) = rows steps..steps+keep-1 of [conv_old[l] ; qkv_tape[l]]
 * (qkv_tape is [layers, tape_rows, conv_dim]).  layers = 0 skips the conv part.  All pointers are device memory. */
DFLASH_API int dflash_accept_commit(const int* block_ids, const int* posterior, int n_tokens, int* n_accepted, int* steps,
                                    int* offset, int* kv_len, int kv_len_extra, const void* conv_old, const void* qkv_tape,
                                    void* conv_new, int layers, int tape_rows, int keep, int conv_dim, int dtype,
                                    void* stream);
/* GatedDeltaNet layer between its input projections and the recurrence (runtime.py:368-403).
 * proj[t, 0:conv_dim] = qkv (q heads | k heads | v heads), z at z_off, b and a (Hv columns each) at b_off, a_off;
 * ld = row stride of proj in elements.  conv_state [Kc-1, conv_dim], conv_w [conv_dim, Kc] (tap j multiplies row t+j
 * of [conv_state ; qkv]), conv_b [conv_dim] or NULL.  Outputs: q,k [T,Hk,Dk] (q = Dk^-1 rms_norm, k = Dk^-1/2 rms_norm),
 * v [T,Hv,Dv], g f32 [T,Hv] = exp(-exp(A_log) softplus(a + dt_bias)), beta f32 [T,Hv] = sigmoid(b),
 * new_conv_state [Kc-1, conv_dim] (must not alias conv_state), qkv_tape [T, conv_dim] (copy kept for the rollback). */
DFLASH_API int dflash_gdn_prep(const void* proj, long long ld, int z_off, int b_off, int a_off, const void* conv_state,
                               const void* conv_w, const void* conv_b, const float* A_log, const float* dt_bias, void* q,
                               void* k, void* v, float* g, float* beta, void* new_conv_state, void* qkv_tape, int T_rows,
                               int Hk, int Hv, int Dk, int Dv, int conv_kernel, float eps, int dtype, void* stream);
/* out[t, hv*Dv+d] = rms_norm(y[t,hv,:])[d] * w[d] * silu(z[t,hv,d]), z read from proj at z_off (runtime.py:445). */
DFLASH_API int dflash_gated_rmsnorm(const void* y, const void* proj, long long ld, int z_off, const void* w, void* out,
                                    int T_rows, int Hv, int Dv, float eps, int dtype, void* stream);
/* dflash_gdn_prep + dflash_gdn_forward_tape + dflash_gated_rmsnorm of one GatedDeltaNet layer in ONE launch (same
 * arithmetic in the same order; the last norm's sum of squares is added per 16 rows, so `out` may differ from the
 * three-call sequence in the last bf16 bit; state, tapes and conv window are bit-identical).  Arguments as in those
 * calls: proj/ld/offsets, conv window in / out, conv weights, A_log, dt_bias, g_norm_w [Dv]; state_in/out fp32
 * [Hv,Dv,Dk]; tape fp32 [T,Hv,Dv], tape_k bf16 [T,Hk,Dk], tape_g fp32 [T,Hv], qkv_tape [T,conv_dim]; out [T,out_ld]
 * receives norm(y) * g_norm_w * silu(z), the input of the output projection (runtime.py:368-445).
 * Only where dflash_gdn_layer_supported() says 1 (bf16, fp32 state, Dk = 128, Dv % 16 == 0 and <= 128, T_rows <= 16,
 * conv kernel <= 8); anything else is refused. */
DFLASH_API int dflash_gdn_layer_supported(int T_rows, int Hk, int Hv, int Dk, int Dv, int conv_kernel, int dtype,
                                          int state_dtype);
DFLASH_API int dflash_gdn_layer(const void* proj, long long ld, int z_off, int b_off, int a_off, const void* conv_state,
                                const void* conv_w, const void* conv_b, const float* A_log, const float* dt_bias,
                                const void* g_norm_w, const void* state_in, void* state_out, float* tape, void* tape_k,
                                float* tape_g, void* new_conv_state, void* qkv_tape, void* out, long long out_ld,
                                int T_rows, int Hk, int Hv, int Dk, int Dv, int conv_kernel, float eps, int dtype,
                                int state_dtype, void* stream);
/* Gated attention layer between its projections and the attention kernel (runtime.py:527-555).
 * proj row = [(query D | gate D) x Hq | k Hk*D at k_off | v Hk*D at v_off].  q,k get a per-head RMSNorm with weights
 * and a rotary embedding of the first rope_dims channels (half-split pairing) at position offset + t; q is written as
 * [Hq,T,D]; k and v are appended to the caches [Hk, cache_capacity, D] (cache_head_stride >= cache_capacity * D
 * elements per head) at row offset+t.  offset + T_rows > cache_capacity is refused. */
DFLASH_API int dflash_attn_prep(const void* proj, long long ld, int k_off, int v_off, const void* q_norm_w,
                                const void* k_norm_w, void* q, void* kcache, void* vcache, long long cache_head_stride,
                                int cache_capacity, int T_rows, int Hq, int Hk, int D, int rope_dims, int offset, float eps,
                                float rope_base, int dtype, void* stream);
/* out[t*out_ld + hq*D+d] = o[hq,t,d] * sigmoid(gate[t,hq,d])  (runtime.py:611-612); out_ld >= Hq*D. */
DFLASH_API int dflash_attn_post(const void* o, const void* proj, long long ld, void* out, long long out_ld, int T_rows,
                                int Hq, int D, int dtype, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Variants whose cache position lives on the DEVICE, so that one captured CUDA graph serves every speculative cycle
 * (the reference re-reads its Python-side cache offset each cycle, dflash_mlx/runtime.py:546-550, 878-907; a graph
 * cannot).  dflash_attn_prep_dev_offset = dflash_attn_prep with the offset read from *offset_dev; a row whose
 * position falls outside [0, cache_capacity) is NOT stored and the device error word is set to 31 | row << 8
 * (dflash_device_error): a stale device scalar cannot write into a neighbouring allocation.  dflash_verify_sdpa_dev_len = dflash_verify_sdpa (no mask array) whose KV
 * length is min(*n_dev, N_max): the split-KV geometry and the workspace are those of N_max, splits beyond the actual
 * length contribute nothing. */
DFLASH_API int dflash_attn_prep_dev_offset(const void* proj, long long ld, int k_off, int v_off, const void* q_norm_w,
                                           const void* k_norm_w, void* q, void* kcache, void* vcache,
                                           long long cache_head_stride, int cache_capacity, int T_rows, int Hq, int Hk,
                                           int D, int rope_dims, const int* offset_dev, float eps, float rope_base,
                                           int dtype, void* stream);
DFLASH_API int dflash_verify_sdpa_dev_len(const void* q, const void* k, const void* v, void* out, int B, int Hq, int Hk,
                                          int N_max, const int* n_dev, int D, long long k_head_stride,
                                          long long k_seq_stride, long long v_head_stride, long long v_seq_stride,
                                          float scale, int dtype, int num_splits, void* workspace, size_t workspace_bytes,
                                          void* stream);

/* ---------------------------------------------------------------------------------------------
 * Mixture-of-experts block of a verify step (16 tokens, top_k of E routed experts + one shared expert).
 * The reference has no expert code of its own: routed experts run through mlx-lm's SwitchGLU / `mx.gather_qmm`
 * (dependency), only the shared expert reaches its verify matmul (dflash_mlx/verify_linear.py:160).  These entry
 * points put the whole block on the same weight-streaming kernel: because every rank holds all 16 tokens, each
 * ACTIVE expert's matrices are streamed once and applied to all 16 rows, with the routing weight (0 for tokens that
 * did not choose the expert) folded into the activations of the down projection.
 *
 * dflash_moe_route: logits dtype[T, E+1] (column E = shared-expert gate).  Per token the top_k experts by logit (ties
 *   to the lower index) with softmax weights over the chosen ones.  Experts in [e_lo, e_hi) chosen by any token are
 *   numbered in ascending order: slot_expert[slot] = expert id - e_lo, i.e. the index inside the calling rank's stack
 *   of expert matrices; with_shared != 0 appends the shared expert (stack index e_hi - e_lo, weight
 *   sigmoid(logit[t,E])).  *n_active = number of slots (<= n_max); wdense f32[T, n_max] = weight of token t for
 *   a slot.  topk_ids int[T,top_k] / topk_w f32[T,top_k] are optional outputs (both or neither).  One thread block.
 * dflash_moe_qmm, experts stacked as w_q uint32[experts * block_rows, Kb/8] (+ scales, biases), group size 64:
 *   mode 1 (rows gathered):   y[M, slot*block_rows + r] = x[M,Kb] . W[slot_expert[slot]][r,:]      y: dtype[M, n_max*block_rows]
 *   mode 2 (chunks gathered): y[M, r] = sum_slot x[M, slot*Kb .. +Kb) . W[slot_expert[slot]][r,:]  x: dtype[M, n_max*Kb]
 *   Only slots < *n_active are read / written; the work partition is made on the device from *n_active, so nothing
 *   synchronises the host.  block_rows % 64 == 0, Kb % 512 == 0.  Workspace as for dflash_verify_qmm
 *   (dflash_moe_qmm_workspace_bytes, zero-filled once, may be the same buffer).
 * dflash_moe_swiglu: act[t, slot*I + i] = w[t,slot] * silu(gu[t, slot*2I + i]) * gu[t, slot*2I + I + i], slot < *n_active. */
DFLASH_API int dflash_moe_route(const void* logits, int T_rows, int experts, int top_k, int e_lo, int e_hi, int with_shared,
                                int n_max, int* slot_expert, int* n_active, float* wdense, int* topk_ids, float* topk_w,
                                int dtype, void* stream);
DFLASH_API size_t dflash_moe_qmm_workspace_bytes(int M, int block_rows, int Kb, int n_max, int mode);
DFLASH_API int dflash_moe_qmm(const void* x, const void* w_q, const void* scales, const void* biases, void* y, int M,
                              int experts, int block_rows, int Kb, int mode, const int* slot_expert, const int* n_active,
                              int n_max, int dtype, void* workspace, size_t workspace_bytes, void* stream);
DFLASH_API int dflash_moe_swiglu(const void* gate_up, const float* wdense, const int* n_active, void* act, int T_rows, int I,
                                 int n_max, int dtype, void* stream);
/* dflash_moe_qmm on the tcgen05 kernel with an epilogue of dflash_verify_qmm_fused (bf16, block_rows % 128 == 0):
 * mode 0 (+ in_ssq: x holds h * norm_weight and the per-token RMS factor multiplies the accumulators) on either gather
 * mode; mode 1 (residual add into y, scaled = y * next_w, out_ssq) on the summed output of gather mode 2, which then
 * needs at least one active slot (device error 19 otherwise: keep the shared expert on the rank). */
DFLASH_API int dflash_moe_qmm_fused_supported(int M, int block_rows, int Kb, int n_max, int mode, int dtype);
DFLASH_API int dflash_moe_qmm_fused(const void* x, const void* w_q, const void* scales, const void* biases, void* y, int M,
                                    int experts, int block_rows, int Kb, int mode, const int* slot_expert,
                                    const int* n_active, int n_max, int dtype, const dflash_qmm_epilogue* epilogue,
                                    void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Tensor-parallel reduction over peer-mapped memory, fused with the residual add and RMSNorm that consume it.
 * Generalises the reference's single collective, `mx.distributed.all_sum` after the GatedDeltaNet out_proj
 * (dflash_mlx/runtime.py:449-450), to every row-parallel projection of the step:
 *     h_out = h_in + sum over ranks of delta_rank ;  x = rmsnorm(h_out) * w        (one kernel, one CTA per row)
 * Each rank owns an inbox (dflash_peer_inbox_bytes) and a flag array (dflash_peer_flags_bytes), both allocated
 * zero-filled by dflash_peer_alloc (these two calls DO allocate device memory: cudaMalloc), exported with
 * dflash_peer_export (a 64-byte CUDA IPC handle to hand to the other processes) and mapped there with
 * dflash_peer_open.  inbox_ptrs[r] / flag_ptrs[r] are HOST arrays of `world` device pointers: rank r's inbox / flags
 * as visible from this process (its own allocation for r == rank).  The kernel writes this rank's block into every
 * other inbox as 8-byte entries {two elements, sequence number} (data and "ready" in one indivisible store), waits -
 * at most dflash_peer_set_wait_polls() polls per entry, then it records device error 21 and leaves the row
 * unwritten - for the other ranks' entries and finishes add + norm.  The flags buffer only holds the per-row sequence
 * numbers of its owner.
 * Every rank must issue the same sequence of calls.  h_out may alias h_in.  world <= 8, H % 8 == 0, H <= 16384.
 * Plain peer loads / stores only (no multicast). */
DFLASH_API size_t dflash_peer_inbox_bytes(int world, int T_rows, int H);
DFLASH_API size_t dflash_peer_flags_bytes(int world, int T_rows);
DFLASH_API int dflash_peer_alloc(size_t bytes, void** dev_ptr);
DFLASH_API int dflash_peer_free(void* dev_ptr);
DFLASH_API int dflash_peer_export(void* dev_ptr, unsigned char* handle64);
DFLASH_API int dflash_peer_open(const unsigned char* handle64, void** dev_ptr);
DFLASH_API int dflash_peer_close(void* dev_ptr);
DFLASH_API void dflash_peer_set_wait_polls(unsigned polls);
/* Hand-over protocol: 0 (default) = by rank count - 8-byte {data, sequence} entries for world <= 4 (one NVLink latency),
 * 16-byte pushes + fence + per-row flags above (fewer packets and polls); 1 / 2 force one.  Same value on every rank. */
DFLASH_API void dflash_peer_set_protocol(int protocol);
DFLASH_API int dflash_peer_reduce_add_rmsnorm(const void* delta, void* const* inbox_ptrs, void* const* flag_ptrs, int rank,
                                              int world, const void* h_in, const void* w, void* h_out, void* x,
                                              int T_rows, int H, float eps, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DFLASH_B200_H_ */
