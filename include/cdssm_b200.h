/*
 * C ABI of the B200 (sm_100a) implementation of the CD-SSM scan path.
 *
 * Plain pointers and sizes only: every pointer is a CUDA device pointer unless its comment
 * says "host"; `stream` is a cudaStream_t passed as void*.  Calls enqueue work on `stream`
 * and return without synchronising.  Return value: CDSSM_OK or a negative CDSSM_ERR_* code;
 * nothing throws.  The library allocates no device memory: outputs and workspaces are the
 * caller's.  `dtype` selects the storage type of every activation tensor of the call:
 * CDSSM_BF16 (the only type the reference supports) or CDSSM_F32 (same arithmetic with no
 * intermediate rounding).
 *
 * Layouts are the reference operator layouts (cdssm/ops.py docstrings): sequence-major,
 * head-minor.  "Replaces" lines cite the reference entry point each function stands in for.
 */
#ifndef CDSSM_B200_H
#define CDSSM_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define CDSSM_API __attribute__((visibility("default")))
#else
#define CDSSM_API
#endif

#define CDSSM_OK 0
#define CDSSM_ERR_BAD_ARG (-1)      /* null pointer, non-positive size, odd N, misalignment */
#define CDSSM_ERR_UNSUPPORTED (-2)  /* size outside the supported range (N > 32, D > 128, ...) */
#define CDSSM_ERR_WORKSPACE (-3)    /* workspace missing or too small */
#define CDSSM_ERR_CUDA (-4)         /* a CUDA runtime call failed; see cdssm_b200_last_cuda_error */
#define CDSSM_ERR_TIMEOUT (-5)      /* a bounded device-side wait ran out (status word set) */

#define CDSSM_BF16 0
#define CDSSM_F32 1

/* Library version (major*10000 + minor*100 + patch) and the CUDA error of the last failed call
 * on this host thread (0 if none). */
CDSSM_API int cdssm_b200_version(void);
CDSSM_API int cdssm_b200_last_cuda_error(void);

/* Fused dynamics: gate_raw (B,L,(N+5)*H) -> A_bar (B,L,H,N), vp_scale (B,L,H,N/2),
 * beta (B,L,H), sel_C (B,L,H).  log_dt_scale, rope_freqs: (H) float32.  pos0 is added to the
 * token index (the reference always uses 0).
 * Replaces dynamics_fused_fwd_cuda, cdssm/csrc/kernels/dynamics_fused.cu:392-440
 * (bound at cdssm/csrc/binding.cpp:130-202, called from cdssm/ops.py:53). */
CDSSM_API int cdssm_b200_dynamics_fwd(const void* gate_raw, const float* log_dt_scale,
                            const float* rope_freqs, void* A_bar, void* vp_scale, void* beta,
                            void* sel_C, float gating_c, float omega_thresh, float adt_delta,
                            float adt_smoothness, float adt_eps, int B, int L, int H, int N,
                            int pos0, int dtype, void* stream);

/* L2 normalisation of K and Q rows, x * rsqrt(sum x^2 + 1e-6); rows = B*L*H, any D >= 1.
 * Replaces normalize_kq_fwd_cuda, cdssm/csrc/kernels/normalize_kq.cu:168-204 (cdssm/ops.py:89). */
CDSSM_API int cdssm_b200_normalize_kq_fwd(const void* K, const void* Q, void* K_out, void* Q_out,
                                int64_t rows, int D, int dtype, void* stream);

/* Backward of cdssm_b200_dynamics_fwd: upstream gradients of A_bar (B,L,H,N), vp_scale (B,L,H,N/2), beta, sel_C
 * (B,L,H) -> grad_gate_raw (B,L,(N+5)*H) in the storage type and grad_log_dt_scale (H) float32 (zeroed and
 * accumulated by the call; the accumulation order over tokens is not fixed).
 * Replaces dynamics_fused_bwd_cuda, cdssm/csrc/kernels/dynamics_fused.cu:145-387 (cdssm/ops.py:68-81). */
CDSSM_API int cdssm_b200_dynamics_bwd(const void* grad_A_bar, const void* grad_vp_scale, const void* grad_beta,
                            const void* grad_sel_C, const void* gate_raw, const float* log_dt_scale,
                            const float* rope_freqs, void* grad_gate_raw, float* grad_log_dt_scale,
                            float gating_c, float omega_thresh, float adt_delta, float adt_smoothness,
                            float adt_eps, int B, int L, int H, int N, int pos0, int dtype, void* stream);

/* Backward of cdssm_b200_normalize_kq_fwd: grad_x = n (g - x_hat (g . x_hat)), n = rsqrt(|x|^2 + 1e-6).
 * Replaces normalize_kq_bwd_cuda, cdssm/csrc/kernels/normalize_kq.cu:89-163 (cdssm/ops.py:93-97). */
CDSSM_API int cdssm_b200_normalize_kq_bwd(const void* grad_K_out, const void* grad_Q_out, const void* K, const void* Q,
                                void* grad_K, void* grad_Q, int64_t rows, int D, int dtype, void* stream);

/* Backward of the intra-chunk scan.  Upstream gradients of local_h (BNC,C,H,N,D) and cum_A (BNC,C,H,N); the forward's
 * inputs and its saved outputs (the state before step t is local_h[t-1], as in the reference) -> grad_A, grad_V in the
 * storage type, grad_K (BNC,C,H,D) and grad_beta (BNC,C,H) in float32 (summed over the pairs of a head; zeroed and
 * accumulated by the call).
 * Replaces intra_chunk_scan_bwd_cuda, cdssm/csrc/kernels/intra_chunk_scan.cu:215-553 (cdssm/ops.py:123-135). */
CDSSM_API int cdssm_b200_intra_chunk_scan_bwd(const void* grad_local_h, const void* grad_cum_A, const void* A,
                                    const void* K, const void* V, const void* beta, const void* local_h,
                                    const void* cum_A, void* grad_A, float* grad_K, void* grad_V, float* grad_beta,
                                    int BNC, int C, int H, int D, int N, int dtype, void* stream);

/* Backward of the correction pass: upstream gradient of corrections (B,NC,C,H,N,D), the forward's inputs and saved
 * output -> grad_A (B,NC,C,H,N), grad_K (B,NC,C,H,D) float32, grad_beta (B,NC,C,H) float32, grad_chunk_states
 * (B,NC,H,N,D).  reference_order = 1 reproduces the reference's backward kernel, which adds the upstream gradient of
 * corrections[t] before walking step t back (exact_correction.cu:219-223) although its forward stores corrections[t]
 * before step t (exact_correction.cu:90-94), and whose grad_beta is D times too large (a reduced value is reduced
 * over the D threads again, :347-359): not the derivative of the forward, but what the reference trains with.
 * reference_order = 0 is the true derivative.
 * Replaces exact_correction_bwd_cuda, cdssm/csrc/kernels/exact_correction.cu:169-383 (cdssm/ops.py:188-195). */
CDSSM_API int cdssm_b200_exact_correction_bwd(const void* grad_corrections, const void* A, const void* K,
                                    const void* beta, const void* corrections, void* grad_A, float* grad_K,
                                    float* grad_beta, void* grad_chunk_states, int B, int NC, int C, int H, int D,
                                    int N, int reference_order, int dtype, void* stream);

/* Backward of the inter-chunk carry: upstream gradient of chunk_states, total_A and the saved chunk_states ->
 * grad_total_A (B,NC,H,N), grad_final_local_h (B,NC,H,N,D).
 * Replaces inter_chunk_scan_bwd_cuda, cdssm/csrc/kernels/inter_chunk_scan.cu:89-196 (cdssm/ops.py:157-163). */
CDSSM_API int cdssm_b200_inter_chunk_scan_bwd(const void* grad_chunk_states, const void* total_A,
                                    const void* chunk_states, void* grad_total_A, void* grad_final_local_h,
                                    int B, int NC, int H, int D, int N, int dtype, void* stream);

/* Backward of conv1d + SiLU: grad_x (B,L,Dm) in the storage type, grad_weight (Dm,4) and grad_bias (Dm) float32
 * (zeroed and accumulated by the call).
 * Replaces conv1d_silu_bwd_cuda, cdssm/csrc/kernels/conv1d_silu.cu:94-219 (cdssm/ops.py:22-28). */
CDSSM_API int cdssm_b200_conv1d_silu_bwd(const void* grad_out, const void* x, const void* weight, const void* bias,
                               void* grad_x, float* grad_weight, float* grad_bias, int B, int L, int Dm, int dtype,
                               void* stream);

/* Intra-chunk delta-rule scan from a zero state.  A (BNC,C,H,N), K (BNC,C,H,D), V (BNC,C,H,N),
 * beta (BNC,C,H) -> local_h (BNC,C,H,N,D), cum_A (BNC,C,H,N).
 * Replaces intra_chunk_scan_fwd_cuda, cdssm/csrc/kernels/intra_chunk_scan.cu:560-609
 * (cdssm/ops.py:116). */
CDSSM_API int cdssm_b200_intra_chunk_scan_fwd(const void* A, const void* K, const void* V, const void* beta,
                                    void* local_h, void* cum_A, int BNC, int C, int H, int D,
                                    int N, int dtype, void* stream);

/* Inter-chunk carry.  total_A (B,NC,H,N), final_local_h (B,NC,H,N,D) -> chunk_states
 * (B,NC,H,N,D): the carry BEFORE each chunk, s <- total_A (*) s + final_local_h, from s = 0.
 * Replaces inter_chunk_scan_fwd_cuda, cdssm/csrc/kernels/inter_chunk_scan.cu:201-234
 * (cdssm/ops.py:152). */
CDSSM_API int cdssm_b200_inter_chunk_scan_fwd(const void* total_A, const void* final_local_h,
                                    void* chunk_states, int B, int NC, int H, int D, int N,
                                    int dtype, void* stream);

/* Correction pass: propagate each chunk's carry through erase+rotate, storing the state BEFORE
 * each step.  A (B,NC,C,H,N), K (B,NC,C,H,D), beta (B,NC,C,H), chunk_states (B,NC,H,N,D)
 * -> corrections (B,NC,C,H,N,D).
 * Replaces exact_correction_fwd_cuda, cdssm/csrc/kernels/exact_correction.cu:390-438
 * (cdssm/ops.py:181). */
CDSSM_API int cdssm_b200_exact_correction_fwd(const void* A, const void* K, const void* beta,
                                    const void* chunk_states, void* corrections, int B, int NC,
                                    int C, int H, int D, int N, int dtype, void* stream);

/* Causal depthwise 4-tap convolution + bias + SiLU.  x,out (B,L,Dm); weight (Dm,4); bias (Dm).
 * Replaces conv1d_silu_fwd_cuda, cdssm/csrc/kernels/conv1d_silu.cu:223-274 (cdssm/ops.py:18). */
CDSSM_API int cdssm_b200_conv1d_silu_fwd(const void* x, const void* weight, const void* bias, void* out,
                               int B, int L, int Dm, int dtype, void* stream);

/* ---- block glue: the memory-bound steps either side of the scan, one kernel each -------------------- */

/* RMSNorm over the last dimension: out = (x * rsqrt(mean(x^2) + eps)) * weight, rows x d, d a multiple of 8,
 * 16-byte aligned buffers (CDSSM_ERR_UNSUPPORTED otherwise).
 * Replaces RMSNorm.forward, cdssm/models/modules.py:50-53 (four eager kernels). */
CDSSM_API int cdssm_b200_rmsnorm_fwd(const void* x, const void* weight, void* out, int64_t rows, int d, float eps,
                                     int dtype, void* stream);

/* GroupNorm statistics of y (B,L,di) taken over each group's channels and ALL L positions, as the reference's
 * group_norm on (B, d_inner, L) does (cdssm/models/block.py:216-222): the first B*groups*2 floats of stats are
 * (mean, rstd) per (batch row, group); the buffer must hold cdssm_b200_groupnorm_stats_floats(B, L, groups) floats
 * (the rest is scratch for the per-tile sums of the two-stage, deterministic reduction). */
CDSSM_API size_t cdssm_b200_groupnorm_stats_floats(int B, int L, int groups);
CDSSM_API int cdssm_b200_groupnorm_stats(const void* y, float* stats, int B, int L, int di, int groups, float eps,
                                         int dtype, void* stream);

/* out = GroupNorm(y) * silu(z) + skip * x_conv for y, x_conv, out (B,L,di) contiguous and z (B,L,di) with
 * z_row_stride elements between rows (z is a column slice of the input projection).  stats from
 * cdssm_b200_groupnorm_stats, or NULL: statistics per token and group (the causal form a decode cache needs).
 * di / groups a multiple of 8, di <= 8192.  Replaces cdssm/models/block.py:213-224 (about ten eager kernels). */
CDSSM_API int cdssm_b200_groupnorm_gate_fwd(const void* y, const float* stats, const void* gn_weight,
                                            const void* gn_bias, const void* z, int64_t z_row_stride,
                                            const void* skip, const void* x_conv, void* out, int B, int L, int di,
                                            int groups, float eps, int dtype, void* stream);

/* One position of the causal depthwise 4-tap conv + SiLU from a cached history: hist (B,3,Dm) holds the last three
 * inputs and is shifted in place; x (B,Dm) with x_row_stride elements between rows; out (B,Dm).
 * The decode-time form of conv1d_silu_fwd_cuda (cdssm/csrc/kernels/conv1d_silu.cu:25-90); the reference has no
 * cached decode (cdssm/inference/predict.py:53-67 re-runs the window). */
CDSSM_API int cdssm_b200_conv1d_silu_step(const void* x, int64_t x_row_stride, void* hist, const void* weight,
                                          const void* bias, void* out, int B, int Dm, int dtype, void* stream);

/* ---- the fused path -------------------------------------------------------------------- */

/* Flags of cdssm_b200_scan_fused_fwd. */
#define CDSSM_SCAN_DEFAULT 0
#define CDSSM_SCAN_FORCE_SIMT 1    /* use the CUDA-core kernels even where the tensor-core passes apply */
#define CDSSM_SCAN_REUSE_LOCAL 8    /* the workspace still holds the local pass of exactly these inputs, left
                                      by cdssm_b200_scan_summary_fwd on the same workspace: skip that pass */
#define CDSSM_SCAN_EXACT 32         /* NOT the reference's chunk semantics: the plain token-by-token recurrence
                                      over the whole sequence (what the reference equals inside its first
                                      chunk and what decode continues); h0/final_state/tail_state are then
                                      the recurrent state.  One sequential walk per (batch, head, pair). */
#define CDSSM_SCAN_TENSOR_CORE_WA 128 /* insist on the warp-autonomous tcgen05/TMA passes (Gram blocks on tcgen05,
                                      state products as warp-level mma; the default whenever bf16, N = 2,
                                      D = C in {64, 128}, H a multiple of 4 and no tail_state):
                                      CDSSM_ERR_UNSUPPORTED instead of the CUDA-core kernels otherwise */

#define CDSSM_SCAN_KEEP_SIMT_LOCAL 256  /* tests: with the tensor-core passes, keep the CUDA-core LOCAL pass ... */
#define CDSSM_SCAN_KEEP_SIMT_OUTPUT 512 /* ... or the CUDA-core OUTPUT pass, so that each tensor-core pass is also
                                      checked on its own against the other implementation */
#define CDSSM_SCAN_FP32_DECAY 4096  /* NOT the reference's arithmetic: the transition A_bar keeps float32 precision
                                      between the dynamics and the scan.  The reference stores it as bfloat16
                                      (dynamics_fused.cu:117-125), which puts |a_t| above 1 by rounding for slowly
                                      rotating heads; its carry (inter_chunk_scan.cu:73-83, decay only) then grows
                                      exponentially and overflows float32 after a few 1e5 tokens.  Same speed. */
#define CDSSM_SCAN_TEST_WITHHOLD 2048 /* self-test of the bounded device-side waits (tensor-core passes only): the
                                      producer warp issues no load and no UMMA, so the first wait of every
                                      compute warp runs out after the wait limit, the kernels unwind and set
                                      the status word; outputs are undefined.  Never faults or hangs. */

/* Bytes of workspace cdssm_b200_scan_fused_fwd needs for these sizes (0 on bad sizes). */
CDSSM_API size_t cdssm_b200_scan_fused_workspace_bytes(int B, int L, int H, int D, int N, int C);

/* The whole scan path in one call, nothing of size (B,L,H,N,D) ever stored:
 * dynamics -> L2-normalised q/k -> vp-scaled v -> chunked delta-rule scan in the reference's
 * chunk semantics (local scan from zero per chunk of C tokens, decay-only carry between chunks,
 * correction taken before each step) -> shortcut -> read-out with q -> sel_C gate.
 * Supported: even N <= 32, D <= 128, C <= 256, bf16 or fp32 (CUDA-core kernels, three launches);
 * bf16 with N = 2, D = C in {64, 128}, H a multiple of 4 and no tail_state runs on the tensor cores (tcgen05/TMA
 * local and output pass, four launches).
 *   q,k (B,L,H,D) un-normalised; v (B,L,H,N) before the vp scale; gate_raw (B,L,(N+5)*H);
 *   h0 (B,H,N,D) float32 or NULL: carry into the first chunk;
 *   y (B,L,H,N); final_state (B,H,N,D) float32 or NULL: carry after the last chunk;
 *   tail_state (B,H,N,D) float32 or NULL: the recurrent state after token L-1 (what the
 *   one-token decode step continues from);
 *   workspace: at least cdssm_b200_scan_fused_workspace_bytes bytes, 256-byte aligned.
 * With h0 = NULL and shortcut handled as in cdssm/models/block.py:202-211 this equals
 * DynamicsFusedFn + NormalizeKQFn + SSDChunkwiseScan + the read-out of the reference block.
 * Replaces the call chain cdssm/models/block.py:181-211 -> cdssm/models/ssd.py:39-111 ->
 * cdssm/ops.py:53,89,116,152,181. */
CDSSM_API int cdssm_b200_scan_fused_fwd(const void* q, const void* k, const void* v, const void* gate_raw,
                              const float* log_dt_scale, const float* rope_freqs, const float* h0,
                              void* y, float* final_state, float* tail_state, void* workspace,
                              size_t workspace_bytes, float gating_c, float omega_thresh,
                              float adt_delta, float adt_smoothness, float adt_eps,
                              float shortcut_scale, int B, int L, int H, int D, int N, int C,
                              int pos0, int dtype, int flags, void* stream);

/* Sequence segments.  In the reference's semantics the carry between chunks is the diagonal-linear
 * recurrence s <- gamma_c (*) s + l_c (cdssm/csrc/kernels/inter_chunk_scan.cu:73-83) and neither
 * gamma_c nor l_c depends on s, so a chunk-aligned segment is summarised by (total_decay, carry_out):
 * the product of its gamma_c and its carry-out for the given carry-in h0 (NULL = zero).  Segments of
 * one sequence - on one GPU or one per GPU - are chained by
 *   carry_in[g+1] = total_decay[g] (*) carry_in[g] + carry_out[g]   (carry_out taken with h0 = 0)
 * and then scanned independently with their carry_in as h0.
 *
 * cdssm_b200_scan_summary_fwd: k (B,L,H,D), v (B,L,H,N), gate_raw (B,L,(N+5)H) -> carry_out
 * (B,H,N,D) float32 and total_decay (B,H,N) float32 (re/im interleaved); reads no q, writes no y.
 * cdssm_b200_scan_fused_segmented_fwd: cdssm_b200_scan_fused_fwd whose batch rows are `segs`
 * consecutive segments of B/segs longer sequences: row b starts at position pos0 + (b % segs) * L.
 * Both take the workspace of cdssm_b200_scan_fused_workspace_bytes(B, L, H, D, N, C); the summary
 * leaves its per-chunk results there, and a following fused call on the same inputs and workspace may
 * pass CDSSM_SCAN_REUSE_LOCAL to skip recomputing them.  flags of the summary: 0 or CDSSM_SCAN_FP32_DECAY
 * (which the fused call that follows must then carry as well).
 * No reference counterpart (the reference is single-GPU and scans a sequence in one piece). */
CDSSM_API int cdssm_b200_scan_summary_fwd(const void* k, const void* v, const void* gate_raw,
                                          const float* log_dt_scale, const float* rope_freqs,
                                          const float* h0, float* carry_out, float* total_decay,
                                          void* workspace, size_t workspace_bytes, float gating_c,
                                          float omega_thresh, float adt_delta, float adt_smoothness,
                                          float adt_eps, int B, int L, int H, int D, int N, int C, int pos0,
                                          int segs, int dtype, int flags, void* stream);
CDSSM_API int cdssm_b200_scan_fused_segmented_fwd(const void* q, const void* k, const void* v,
                                                  const void* gate_raw, const float* log_dt_scale,
                                                  const float* rope_freqs, const float* h0, void* y,
                                                  float* final_state, void* workspace,
                                                  size_t workspace_bytes, float gating_c,
                                                  float omega_thresh, float adt_delta, float adt_smoothness,
                                                  float adt_eps, float shortcut_scale, int B, int L, int H,
                                                  int D, int N, int C, int pos0, int segs, int dtype,
                                                  int flags, void* stream);

/* Chains segment summaries: carry_in[g] = s, then s <- decay[g] (*) s + carry_out[g] for g = 0..S-1,
 * starting from s = h0 (NULL = zero).  decay (.,H,N), carry_out / carry_in (.,H,N,D) float32 are indexed
 * by segment; segment g of batch element b sits at index b*batch_stride + g*seg_stride, e.g.
 * (S, 1) for the rows of a segmented batch and (1, B) for summaries gathered rank by rank.
 * carry_in, final_state (B,H,N,D) and total_decay (B,H,N) (the product of all decays) may be NULL.
 * No reference counterpart. */
CDSSM_API int cdssm_b200_compose_carries(const float* decay, const float* carry_out, const float* h0,
                                         float* carry_in, float* final_state, float* total_decay, int B,
                                         int S, int H, int D, int N, int64_t batch_stride,
                                         int64_t seg_stride, void* stream);

/* The fused scan for callers that cannot allocate device memory (a server whose pool already owns
 * the whole GPU, a plugin barred from the CUDA allocator, code that must not trigger the
 * device-wide synchronisation of cudaMalloc).  Same arguments and results as
 * cdssm_b200_scan_fused_fwd without the workspace: the scratch is a 16 MiB array built into the
 * library (cdssm_b200_scan_fused_noalloc_max_bytes()), resident on every GPU that loads it.
 *  - Sizes whose cdssm_b200_scan_fused_workspace_bytes exceeds that limit are refused with
 *    CDSSM_ERR_WORKSPACE; nothing is launched.
 *  - The first call on each device looks up the array's device address (with that device
 *    current); make that first call outside any stream capture.
 *  - No cudaMalloc, cudaFree or other allocating routine is called.
 *  - All calls on a device share the one array and it keeps what the last call left in it; the
 *    scan clears the only word that must start at zero.  Two calls that overlap on the GPU (different
 *    streams, no ordering between them) race on the scratch: serialise them.
 * No counterpart in the reference (its launchers allocate their outputs themselves, e.g.
 * intra_chunk_scan.cu:588-590). */
CDSSM_API int cdssm_b200_scan_fused_fwd_noalloc(const void* q, const void* k, const void* v,
                                                const void* gate_raw, const float* log_dt_scale,
                                                const float* rope_freqs, const float* h0, void* y,
                                                float* final_state, float* tail_state, float gating_c,
                                                float omega_thresh, float adt_delta, float adt_smoothness,
                                                float adt_eps, float shortcut_scale, int B, int L, int H,
                                                int D, int N, int C, int pos0, int dtype, int flags,
                                                void* stream);
CDSSM_API size_t cdssm_b200_scan_fused_noalloc_max_bytes(void);

/* Reads back the status word a cdssm_b200_scan_fused_fwd call left at the start of its workspace
 * (synchronises `stream`).  *status_host = 0 and CDSSM_OK if every bounded device-side wait of the
 * tensor-core kernel completed; otherwise the code of the wait that ran out and
 * CDSSM_ERR_TIMEOUT (the outputs of that call are then undefined; the context stays usable).
 * No reference counterpart: the reference has no device-side waits. */
CDSSM_API int cdssm_b200_scan_fused_status(const void* workspace, int* status_host, void* stream);

/* cdssm_b200_scan_fused_status for the allocation-free entry point: reads the status word that the last
 * cdssm_b200_scan_fused_fwd_noalloc call on the current device left in the built-in scratch
 * (synchronises `stream`).  CDSSM_ERR_BAD_ARG if no such call has been made on this device.
 * No reference counterpart. */
CDSSM_API int cdssm_b200_scan_fused_noalloc_status(int* status_host, void* stream);

/* Limit of every bounded device-side wait of the tensor-core kernels, in nanoseconds of the GPU's global
 * timer (process-wide; default and 0 = 400 ms).  A wait that runs out makes its kernel unwind and set the
 * status word instead of hanging.  Returns the previous limit.  No reference counterpart. */
CDSSM_API uint64_t cdssm_b200_set_wait_limit_ns(uint64_t limit_ns);

/* Self-test of the bounded wait primitive: one thread block waits on a barrier that nothing signals, for at
 * most limit_ns, then writes 1 (the wait gave up, as it must) or 2 (it returned as if signalled) to
 * *status_dev and returns.  No reference counterpart. */
CDSSM_API int cdssm_b200_selftest_bounded_wait(int* status_dev, uint64_t limit_ns, void* stream);

/* One-token recurrent decode step for a batch of sequences: dynamics for position `pos`,
 * normalise q/k, state <- a (*) (state - beta (state k) k^T) + beta v k^T, y = sel_C * (state q
 * + shortcut).  state (B,H,N,D) float32 is updated in place; q,k (B,H,D); v (B,H,N);
 * gate_raw (B,(N+5)*H); y (B,H,N).
 * The reference has no decode step (cdssm/inference/predict.py:53-67 re-runs the whole
 * forward per token); the formula is one iteration of
 * cdssm/csrc/kernels/intra_chunk_scan.cu:117-167 with the gates of dynamics_fused.cu:64-139. */
CDSSM_API int cdssm_b200_decode_step(float* state, const void* q, const void* k, const void* v,
                           const void* gate_raw, const float* log_dt_scale,
                           const float* rope_freqs, void* y, float gating_c, float omega_thresh,
                           float adt_delta, float adt_smoothness, float adt_eps,
                           float shortcut_scale, int B, int H, int D, int N, int pos, int dtype,
                           void* stream);

/* cdssm_b200_decode_step with the position read from device memory at run time (*pos_dev), so that
 * one captured CUDA graph of a decode step can be replayed for every position.
 * No reference counterpart (see cdssm_b200_decode_step). */
CDSSM_API int cdssm_b200_decode_step_at(float* state, const void* q, const void* k, const void* v,
                                        const void* gate_raw, const float* log_dt_scale,
                                        const float* rope_freqs, void* y, float gating_c,
                                        float omega_thresh, float adt_delta, float adt_smoothness,
                                        float adt_eps, float shortcut_scale, int B, int H, int D, int N,
                                        const int* pos_dev, int dtype, void* stream);

/* cdssm_b200_decode_step for q, k, v and gate_raw that are column slices of wider per-token projections (*_row_stride
 * elements between batch rows; q and k rows 16-byte aligned) and, if v_first and mix are not NULL, with the
 * value residual of cdssm/models/block.py:167-171 applied on the fly: v <- lerp(v_first, v, mix[head]) rounded to
 * the storage type (v_first (B,H,N) contiguous, mix (H) in the storage type = sigmoid(v_residual_gate)).  Saves
 * the copy of k and the lerp kernel of a decode step.  pos_dev as in cdssm_b200_decode_step_at (or NULL). */
CDSSM_API int cdssm_b200_decode_step_strided(float* state, const void* q, int64_t q_row_stride, const void* k,
                                             int64_t k_row_stride, const void* v, int64_t v_row_stride,
                                             const void* v_first, const void* mix, const void* gate_raw,
                                             int64_t gate_row_stride, const float* log_dt_scale,
                                             const float* rope_freqs, void* y, float gating_c, float omega_thresh,
                                             float adt_delta, float adt_smoothness, float adt_eps,
                                             float shortcut_scale, int B, int H, int D, int N, int pos,
                                             const int* pos_dev, int dtype, void* stream);

/* One-token decode step that reproduces the reference's CHUNKED scan (whose outputs beyond the first chunk are
 * not those of the plain recurrence): the state per (batch, head) is the local state (zero at every chunk
 * start), the correction (starts from the bf16-rounded carry; erased and rotated, never injected; read BEFORE
 * its step, cdssm/csrc/kernels/exact_correction.cu:89-150), the carry (decay-only recurrence over chunks,
 * inter_chunk_scan.cu:52-84) and the chunk's cumulative decay.  local_state, correction, carry: (B,H,N,D)
 * float32; chunk_decay: (B,H,N) float32 (re/im interleaved), all updated in place.  pos (or *pos_dev if not NULL)
 * is the token's position counted from the start of the sequence; chunks are C tokens.  Starting from
 * local_state = 0, correction = carry rounded to the storage type, chunk_decay = (1, 0) at a chunk boundary, T
 * steps give the y of cdssm_b200_scan_fused_fwd over the same T tokens with that carry as h0.
 * The reference has no decode step; this is what its full re-forward per token
 * (cdssm/inference/predict.py:53-67) computes for the newest position of the scan. */
CDSSM_API int cdssm_b200_decode_step_reference(float* local_state, float* correction, float* carry,
                                               float* chunk_decay, const void* q, const void* k, const void* v,
                                               const void* gate_raw, const float* log_dt_scale,
                                               const float* rope_freqs, void* y, float gating_c, float omega_thresh,
                                               float adt_delta, float adt_smoothness, float adt_eps,
                                               float shortcut_scale, int B, int H, int D, int N, int C, int pos,
                                               const int* pos_dev, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CDSSM_B200_H */
