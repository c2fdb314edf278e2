/*
 * slinoss_b200 -- C ABI of the B200 (sm_100a) v2x2ssd scan backend.
 *
 * Every entry point
 *   - takes raw DEVICE pointers, plain sizes and a CUDA stream (as void*),
 *   - returns an int status: 0 = ok, negative = argument error (SLX_E_*),
 *     positive = the cudaError_t raised by a launch,
 *   - never allocates and never synchronises; scratch memory is passed in by the
 *     caller (sizes from the *_workspace_bytes functions),
 *   - launches on the given stream only.
 * slx_last_error_string() returns a thread-local description of the last
 * non-zero status.
 *
 * Layouts are the reference's canonical ones (slinoss/ops/v2x2ssd/reference.py:
 * 1-41), with (batch, heads) flattened to BH:
 *   U,Y      (BH, T, P)        activation dtype (see slx_dtype)
 *   B,C      (BH, T, 2N)       activation dtype, interleaved [re0,im0,re1,...]
 *   M        (BH, T, 2)        fp32 packed complex
 *   K        (BH, T, 2, 2)     fp32, tap 0 = prev, tap 1 = curr, each (re,im)
 *   states   (BH, P, 2N)       fp32 interleaved complex
 *   chunk tensors (BH, NC, P, 2N) / (BH, NC, 2), NC = ceil(T / chunk), fp32;
 *            chunk_starts and d_inc (its gradient-side counterpart) are stored
 *            in slx_scan_starts_dtype(shape): the activation dtype where the
 *            tensor-core kernels run (they round both to that dtype for their
 *            products anyway), fp32 otherwise
 * Tokens past T in the last chunk behave as M=1, K=U=B=C=0
 * (reference.py:541-667).  Nullable pointers are marked [opt].
 * The scan entry points read and write with 16-byte accesses: every tensor
 * pointer handed to them must be 16-byte aligned (SLX_E_UNSUPPORTED otherwise).
 * Scan prep and conv take any alignment and pick their vector width from it.
 */
#ifndef SLINOSS_B200_H_
#define SLINOSS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SLX_ABI_VERSION 5

typedef enum { SLX_F32 = 0, SLX_BF16 = 1, SLX_F16 = 2 } slx_dtype;

enum {
  SLX_OK = 0,
  SLX_E_NULL = -1,        /* required pointer is NULL */
  SLX_E_SHAPE = -2,       /* non-positive or inconsistent size */
  SLX_E_UNSUPPORTED = -3, /* size/dtype outside what the kernels cover */
  SLX_E_WORKSPACE = -4,   /* workspace too small or misaligned */
  SLX_E_DTYPE = -5
};

typedef struct {
  int32_t batch_heads; /* BH = batch * heads                               */
  int32_t T;           /* tokens                                           */
  int32_t P;           /* head dim (1..64)                                 */
  int32_t N;           /* complex state pairs; D = 2N                      */
  int32_t chunk;       /* chunk length L: multiple of 16, 16..128          */
  int32_t dtype;       /* slx_dtype of U, B, C, Y and their gradients      */
  int32_t starts_dtype; /* slx_dtype of chunk_starts and d_inc.  It also names the
                         * kernel family: the activation dtype = tcgen05 kernels
                         * (half inputs, chunk 128, P 64, 2N in {64,..,256} only),
                         * SLX_F32 = fp32-exact CUDA-core kernels.  Every call of
                         * one forward/backward pair must pass the same value;
                         * slx_scan_starts_dtype() gives the recommended one.   */
} slx_scan_shape;

int slx_abi_version(void);

/* Recommended starts_dtype for this shape (the field itself is not read): the
 * activation dtype where the tensor-core kernels cover the shape, SLX_F32
 * otherwise or after slx_set_tensor_path(0). */
int slx_scan_starts_dtype(const slx_scan_shape *s);
const char *slx_last_error_string(void);

/* ---- forward stages --------------------------------------------------- */

/* Replaces reference.py:937 chunk_increment (CuTe: kernels/fwd/__init__.py:740
 * chunk_increment_cute).  inc (BH,NC,P,2N) stored as inc_dtype: SLX_F32 (what the
 * reference returns), or the activation dtype where the tensor-core kernels run
 * (the whole-op entry points below use that: the increments only feed the fp32
 * state pass, whose output is rounded to that dtype for the chunk kernels, and
 * half storage halves the traffic of two HBM-bound kernels).
 * m_chunk (BH,NC,2) fp32. */
int slx_chunk_increment_fwd(const slx_scan_shape *s, const void *U,
                            const float *M, const float *K, const void *B,
                            const float *B_prev /*[opt] (BH,2N)*/,
                            const float *U_prev /*[opt] (BH,P)*/, void *inc,
                            int32_t inc_dtype, float *m_chunk, void *stream);

/* Replaces reference.py:1015 state_passing (CuTe: kernels/fwd/__init__.py:897).
 * chunk_starts holds starts_dtype values (slx_dtype); with SLX_F32 it may alias
 * inc (the pass is then in place).  chunk_starts == NULL
 * asks for final_state only (nothing else is written): the affine offset of a
 * segment when segments are chained across devices.
 * inc is read as inc_dtype (SLX_F32 or starts_dtype); the recurrence is fp32. */
int slx_state_passing_fwd(int32_t batch_heads, int32_t n_chunks, int32_t P,
                          int32_t N, const void *inc, int32_t inc_dtype,
                          const float *m_chunk,
                          const float *initial_states /*[opt]*/,
                          void *chunk_starts /*[opt]*/, int32_t starts_dtype,
                          float *final_state, void *stream);

/* Replaces reference.py:1059 chunk_scan (CuTe: kernels/fwd/__init__.py:1125). */
int slx_chunk_scan_fwd(const slx_scan_shape *s, const void *U, const float *M,
                       const float *K, const void *B, const void *C,
                       const void *chunk_starts /* slx_scan_starts_dtype(s) */,
                       const float *B_prev /*[opt]*/, const float *U_prev /*[opt]*/,
                       void *Y, void *stream);

/* Replaces reference.py:1195 v2x2ssd / cute/kernels/fwd/__init__.py:1691
 * v2x2ssd_fwd_cute: the three stages back to back on one stream.
 * increments: scratch of (BH, NC, P, 2N) values of starts_dtype for the chunk
 * increments.  NULL makes chunk_starts double as the increment buffer (only where
 * slx_scan_starts_dtype(s) is fp32): no extra memory, but the state pass then
 * overwrites each line it has just read, which runs at well under half the
 * speed of the two-buffer pass on B200. */
int slx_v2x2ssd_fwd(const slx_scan_shape *s, const void *U, const float *M,
                    const float *K, const void *B, const void *C,
                    const float *initial_states /*[opt]*/,
                    const float *B_prev /*[opt]*/, const float *U_prev /*[opt]*/,
                    void *Y, float *final_state,
                    void *chunk_starts /* slx_scan_starts_dtype(s) */,
                    float *m_chunk, void *increments /*[opt]*/, void *stream);

/* ---- backward ----------------------------------------------------------- */

/* Scratch for slx_v2x2ssd_bwd (and the three backward stages). */
size_t slx_v2x2ssd_bwd_workspace_bytes(const slx_scan_shape *s);

/* dZ0[c] = sum_t conj(prefix_t) dY_t (x) c_t : gradient of the loss with respect
 * to each chunk's start state through that chunk's outputs only.  Replaces
 * cute/kernels/bwd/chunk_scan/dz0.py:521.  dZ0 (BH,NC,P,2N) stored as dz0_dtype:
 * SLX_F32, or the activation dtype on the tensor-core path (as for the increments). */
int slx_chunk_scan_bwd_dz0(const slx_scan_shape *s, const float *M, const void *C,
                           const void *dY, void *dZ0, int32_t dz0_dtype,
                           void *stream);

/* Reverse recurrence over chunks (cute/kernels/bwd/state_passing/state.py:119
 * and m.py:83 fused): on return d_inc[c] = dL/d(end state of chunk c), stored as
 * starts_dtype (with SLX_F32 it may alias dZ0), d_initial = dL/d(initial state),
 * and zdot (BH,NC,2) holds sum_{p,n} conj(end_state_c) * d_inc[c] (from the fp32
 * values), the chunk-level term of dM.  final_state is the forward's fp32 final
 * state; chunk_starts is read as starts_dtype, dZ0 as dz0_dtype (SLX_F32 or
 * starts_dtype).
 * zdot_partials is scratch of slx_state_passing_bwd_partials_bytes() bytes.
 * zdot and zdot_partials NULL: no dot products (chunk_starts and final_state are
 * then not read).  d_inc NULL as well: only d_initial is written. */
size_t slx_state_passing_bwd_partials_bytes(int32_t batch_heads, int32_t n_chunks,
                                            int32_t P, int32_t N);
int slx_state_passing_bwd(int32_t batch_heads, int32_t n_chunks, int32_t P,
                          int32_t N, const void *dZ0, int32_t dz0_dtype,
                          const float *m_chunk,
                          const void *chunk_starts /*[opt]*/, int32_t starts_dtype,
                          const float *final_state /*[opt]*/,
                          const float *d_final /*[opt]*/, void *d_inc /*[opt]*/,
                          float *d_initial /*[opt]*/, float *zdot /*[opt]*/,
                          float *zdot_partials /* workspace, [opt] */, void *stream);

/* Per-chunk backward given d_inc (from slx_state_passing_bwd) and zdot: writes
 * dU, dB, dC (activation dtype; the last row of every chunk still lacks the
 * carry of the following chunk), dM, dK (fp32) and the carries
 * carryB (BH,NC,2N), carryU (BH,NC,P) fp32: the gradient each chunk sends to the
 * token before it.  Replaces the chunk_scan and chunk_increment backward
 * kernels of cute/kernels/bwd/__init__.py:930-1042 (scan_db, scan_dcdr,
 * scan_param, scan_du, inc_db, inc_boundary, inc_param, inc_du). */
int slx_chunk_scan_bwd(const slx_scan_shape *s, const void *U, const float *M,
                       const float *K, const void *B, const void *C,
                       const float *B_prev /*[opt]*/, const float *U_prev /*[opt]*/,
                       const void *chunk_starts, const void *d_inc,
                       const float *zdot, const void *dY, void *dU, float *dM,
                       float *dK, void *dB, void *dC, float *carryB,
                       float *carryU, void *stream);

/* Full backward of the scan: what torch.autograd computes through
 * reference.py:1195; replaces cute/kernels/bwd/__init__.py:1310
 * v2x2ssd_bwd_stateful_cute.  Gradients dU,dB,dC in the activation dtype;
 * dM,dK,d_initial,dB_prev,dU_prev fp32. */
int slx_v2x2ssd_bwd(const slx_scan_shape *s, const void *U, const float *M,
                    const float *K, const void *B, const void *C,
                    const float *B_prev /*[opt]*/, const float *U_prev /*[opt]*/,
                    const void *chunk_starts, const float *m_chunk,
                    const float *final_state, const void *dY,
                    const float *d_final /*[opt]*/, void *dU, float *dM,
                    float *dK, void *dB, void *dC, float *d_initial /*[opt]*/,
                    float *dB_prev /*[opt]*/, float *dU_prev /*[opt]*/,
                    void *workspace, size_t workspace_bytes, void *stream);

/* The backward in two calls, for a sequence whose segments live on different
 * devices (no counterpart in the reference, which has no distributed code).
 * _begin computes dZ0 into the workspace and the segment's d_initial for a zero
 * d_final (fp32, like d_initial); the caller chains the true d_final across
 * segments (d_initial = d_initial_zero_final + conj(prod m_chunk) d_final) and
 * then calls _finish with the same workspace, which runs the rest of
 * slx_v2x2ssd_bwd without recomputing dZ0.  Same workspace size. */
int slx_v2x2ssd_bwd_begin(const slx_scan_shape *s, const float *M, const void *C,
                          const float *m_chunk, const void *dY,
                          float *d_initial_zero_final, void *workspace,
                          size_t workspace_bytes, void *stream);
int slx_v2x2ssd_bwd_finish(const slx_scan_shape *s, const void *U, const float *M,
                           const float *K, const void *B, const void *C,
                           const float *B_prev /*[opt]*/, const float *U_prev /*[opt]*/,
                           const void *chunk_starts, const float *m_chunk,
                           const float *final_state, const void *dY,
                           const float *d_final /*[opt]*/, void *dU, float *dM,
                           float *dK, void *dB, void *dC, float *d_initial /*[opt]*/,
                           float *dB_prev /*[opt]*/, float *dU_prev /*[opt]*/,
                           void *workspace, size_t workspace_bytes, void *stream);

/* ---- segment chaining across devices (no counterpart in the reference) ------ */

/* A segment of a sequence acts on the incoming scan state as z_out = m_seg * z_in + f
 * (m_seg one complex number per batch*head, f one state).  When the segments live on
 * different devices, every device gathers all (m_seg, f) pairs and folds the ones in
 * front of it (forward) or behind it (backward, conj != 0 conjugates the transitions):
 *   out = offsets[0];  for j = 1 .. count-1:  out = m[j] * out + offsets[j]
 * offsets: `count` states (BH,P,2N) fp32, slice j at offsets + j*slice_stride elements;
 * m: transitions (BH,2) fp32, slice j at m + j*m_stride elements (m[0] is not read).
 * Strides may be negative (the backward chain walks the gathered buffer downwards). */
int slx_segment_fold(int32_t batch_heads, int32_t P, int32_t N, int32_t count,
                     const float *offsets, int64_t slice_stride, const float *m,
                     int64_t m_stride, int32_t conj, float *out, void *stream);

/* out = m * z + f (conj != 0: conj(m) * z + f) for one segment. */
int slx_segment_axpy(int32_t batch_heads, int32_t P, int32_t N, const float *m,
                     const float *z, const float *f, int32_t conj, float *out,
                     void *stream);

/* m_seg (BH,2) = product over the chunks of m_chunk (BH,NC,2). */
int slx_segment_transition(int32_t batch_heads, int32_t n_chunks, const float *m_chunk,
                           float *m_seg, void *stream);

/* ---- scan preparation ---------------------------------------------------- */

typedef struct {
  int32_t batch, T, heads, P, N;
  int32_t dtype;        /* slx_dtype of value / params / bc and of U, B, C  */
  int32_t normalize_bc; /* RMS-norm (eps 1e-5) + per-head scale when != 0   */
  float dt_min, dt_max, r_min, r_max, theta_bound, k_max, eps;
  /* row strides in elements of the (batch*T, width) inputs: they may be column
   * slices of one wider projection output */
  int64_t value_stride, params_stride, bc_stride;
} slx_prep_shape;

/* Replaces slinoss/layers/scanprep.py:351 _prepare_inputs_reference (CuTe:
 * ops/scanprep/cute/kernels/fwd.py:83).  value (b,T,H*P), params (b,T,H*13),
 * bc (b,T,H*4*N) -> U (b,H,T,P), B,C (b,H,T,2N) activation dtype; M (b,H,T,2),
 * K (b,H,T,2,2) fp32.  bias (H,13) fp32 (zeros in the unbiased slots),
 * scale (H,4,N) fp32 [opt when normalize_bc == 0]. */
int slx_scanprep_fwd(const slx_prep_shape *s, const void *value,
                     const void *params, const void *bc, const float *bias,
                     const float *scale, void *U, float *M, float *K, void *B,
                     void *C, void *stream);

size_t slx_scanprep_bwd_workspace_bytes(const slx_prep_shape *s);

/* VJP of slx_scanprep_fwd (CuTe: ops/scanprep/cute/kernels/bwd.py:113,271).
 * d_value/d_params/d_bc are contiguous (b,T,width) in the activation dtype;
 * d_bias (H,13) and d_scale (H,4,N) fp32 are overwritten (deterministic
 * two-level reduction through the workspace, no atomics). */
int slx_scanprep_bwd(const slx_prep_shape *s, const void *params, const void *bc,
                     const float *bias, const float *scale, const void *dU,
                     const float *dM, const float *dK, const void *dB,
                     const void *dC, void *d_value, void *d_params, void *d_bc,
                     float *d_bias, float *d_scale, void *workspace,
                     size_t workspace_bytes, void *stream);

/* ---- one-token decode step ------------------------------------------------- */

typedef struct {
  int32_t batch, heads, P, N; /* N even */
  int32_t dtype;              /* slx_dtype of value, params, bc, gate, skip, b_prev, u_prev, out */
  int32_t normalize_bc;
  float dt_min, dt_max, r_min, r_max, theta_bound, k_max, eps;
} slx_decode_shape;

/* Replaces SLinOSSMixer._decode_step_reference (layers/mixer.py:714-748) and the contract
 * of mixer_decode_step_cute (ops/v2x2ssd/cute/decode.py:117-149; that kernel is limited to
 * P = 64, N = 64, batch in {1,2,4,8,16}): scan prep of one token, one recurrence step on
 * the carried state, skip and gate.
 *   value, gate (batch, heads, P); params (batch, heads, 13); bc (batch, heads, 4, N);
 *   skip (heads, P); bias (heads, 13) fp32; scale (heads, 4, N) fp32 [needed iff normalize_bc];
 *   state_in (batch, heads, P, 2N) fp32 [NULL = zero state]; b_prev (batch, heads, 2N) and
 *   u_prev (batch, heads, P) in dtype [both NULL = no previous token];
 *   out (batch, heads*P); state_out like state_in; b_last, u_last like b_prev, u_prev [opt].
 * state_out may be state_in, b_last may be b_prev, u_last may be u_prev (in-place update of
 * a ScanState, as the reference's final_state_out / b_last_out / u_last_out do). */
int slx_decode_step(const slx_decode_shape *s, const void *value, const void *params,
                    const void *bc, const void *gate, const void *skip, const float *bias,
                    const float *scale /*[opt]*/, const float *state_in /*[opt]*/,
                    const void *b_prev /*[opt]*/, const void *u_prev /*[opt]*/, void *out,
                    float *state_out, void *b_last /*[opt]*/, void *u_last /*[opt]*/,
                    void *stream);

/* ---- depthwise causal conv1d --------------------------------------------- */

typedef struct {
  int32_t batch, T, channels, width; /* width 2..4 */
  int32_t dtype;                     /* slx_dtype of x, y, weight, bias, state */
  int32_t silu;                      /* fuse y = silu(conv) when != 0          */
  int64_t x_stride;                  /* row stride of x (batch*T, channels)    */
  int64_t x_batch_stride;            /* elements between batches of x          */
} slx_conv_shape;

/* Replaces csrc/causal_conv1d/causal_conv1d.cpp:150 causal_conv1d_fwd as the
 * mixer uses it (slinoss/layers/mixer.py:456 _apply_cconv_cuda): x (b,T,C)
 * channel-last, weight (C,W), bias (C) [opt], state (b,C,W-1) [opt] ->
 * y (b,T,C) contiguous, next_state (b,C,W-1) [opt]. */
int slx_cconv1d_fwd(const slx_conv_shape *s, const void *x, const void *weight,
                    const void *bias, const void *state, void *y,
                    void *next_state, void *stream);

/* One decode token of the same convolution: replaces
 * csrc/causal_conv1d/causal_conv1d_update.cu:25 causal_conv1d_update_kernel as the mixer
 * uses it (slinoss/layers/mixer.py:614 _apply_causal_depthwise_conv_step).  s->T must be 1;
 * x (b,C) with batch stride s->x_batch_stride, state (b,C,W-1) [opt = zeros] ->
 * y (b,C) = act(bias + w . [state, x]), next_state (b,C,W-1) [opt] = [state[1:], x].
 * next_state may be state (in-place rolling update). */
int slx_cconv1d_update(const slx_conv_shape *s, const void *x, const void *weight,
                       const void *bias, const void *state, void *y,
                       void *next_state, void *stream);

size_t slx_cconv1d_bwd_workspace_bytes(const slx_conv_shape *s);

/* Replaces causal_conv1d.cpp:261 causal_conv1d_bwd.  dy (b,T,C) contiguous,
 * d_next_state (b,C,W-1) [opt]; dx (b,T,C) contiguous activation dtype;
 * dweight (C,W), dbias (C) fp32, overwritten, deterministic; dstate (b,C,W-1)
 * fp32 [opt]. */
int slx_cconv1d_bwd(const slx_conv_shape *s, const void *x, const void *weight,
                    const void *bias, const void *state, const void *dy,
                    const void *d_next_state, void *dx, float *dweight,
                    float *dbias, float *dstate, void *workspace,
                    size_t workspace_bytes, void *stream);

/* Same computation and results as slx_cconv1d_bwd, for callers that cannot hand
 * over a workspace because they cannot allocate device memory at call time: a
 * serving process whose own allocator was given all device memory at start-up, a
 * plugin host that forbids driver allocations once it is running, or any place
 * where a cudaMalloc would stall the device.  (No counterpart in the reference.)
 * The partial sums go to a buffer that is part of the library image: 4 MiB per GPU
 * that loads the library, kept until the process exits.  Limit:
 * batch * ceil(T/128) * channels * 5 floats <= 1,048,576, otherwise SLX_E_UNSUPPORTED
 * with a message naming the sizes.  The entry point allocates nothing and frees
 * nothing.  Its first call on each device looks up the buffer's device address (with
 * that device current); make that first call outside any stream capture.  All calls
 * on one GPU share the buffer: two calls whose kernels can overlap on the GPU
 * (different streams, no ordering) race on it and must be serialised by the caller.
 * Nothing in the buffer needs clearing between calls: every slot that is read was
 * written earlier in the same call. */
int slx_cconv1d_bwd_noalloc(const slx_conv_shape *s, const void *x,
                            const void *weight, const void *bias, const void *state,
                            const void *dy, const void *d_next_state, void *dx,
                            float *dweight, float *dbias, float *dstate,
                            void *stream);

/* ---- mixer glue: skip, re-layout and gate in one pass ---------------------------- */

typedef struct {
  int32_t batch, T, heads, P; /* P a multiple of 8 */
  int32_t dtype;              /* slx_dtype of y, u, gate, out and their gradients */
  int64_t gate_stride;        /* elements between tokens of gate (a column slice of a wider row is fine) */
  int64_t gate_batch_stride;  /* elements between batches of gate */
} slx_glue_shape;

/* Replaces SLinOSSMixer._apply_gate_skip (slinoss/layers/mixer.py:585-599) without its
 * output norm: out (b,T,H*P) = (y + skip * u) re-laid from (b,H,T,P), times silu(gate).
 * y, u (b,H,T,P); gate (b,T,H*P) with the given strides; skip (H*P) fp32; out contiguous.
 * All pointers 16-byte aligned. */
int slx_gate_skip_fwd(const slx_glue_shape *s, const void *y, const void *u,
                      const void *gate, const float *skip, void *out, void *stream);

size_t slx_gate_skip_bwd_workspace_bytes(const slx_glue_shape *s);

/* VJP of slx_gate_skip_fwd: d_out (b,T,H*P) contiguous -> dy, du (b,H,T,P), d_gate
 * (b,T,H*P) contiguous, d_skip (H*P) fp32 (overwritten; two-level fixed-order sum
 * through the workspace, no atomics). */
int slx_gate_skip_bwd(const slx_glue_shape *s, const void *y, const void *u,
                      const void *gate, const float *skip, const void *d_out, void *dy,
                      void *du, void *d_gate, float *d_skip, void *workspace,
                      size_t workspace_bytes, void *stream);

/* ---- diagnostics ----------------------------------------------------------- */

/* Half inputs with chunk 128, P 64 and 2N in {64,128,192,256} run on the
 * tcgen05 tensor-core kernels: enable = 2 the persistent warp-specialised ones,
 * enable = 1 the one-chunk-per-CTA ones; everything else, and everything after
 * slx_set_tensor_path(0), runs on the fp32-exact CUDA-core kernels.  Returns the
 * previous setting.  (Process-wide switch for tests; no reference counterpart.) */
int slx_set_tensor_path(int enable);

/* The persistent tensor-core kernels launch one CTA per SM, each walking several
 * chunks.  max_ctas > 0 caps the number of CTAs (a tuning and test knob: a small cap
 * makes small inputs walk the multi-chunk loop); 0 restores one per SM.  Returns the
 * previous cap.  Process-wide; no reference counterpart. */
int slx_set_persistent_ctas(int max_ctas);

/* Synchronising read-and-clear (one atomic exchange on the device) of the status
 * word of the tensor-core kernels on the CURRENT device: *host_out != 0 means a
 * bounded wait on a completion barrier ran out in some launch since the last read;
 * the outputs of the affected chunks were filled with NaN.  One word per device,
 * shared by all streams and threads. */
int slx_read_tc_status(int *host_out);

/* Synchronising read-and-clear (one atomic exchange, current device, one word per
 * device) of the scan's input status word: *host_out != 0
 * means some launch since the last read met a transition M of magnitude exactly 0.
 * The reference raises for such input (reference.py:480-485: the log-magnitude /
 * phase split does not exist); these kernels cannot raise from the device, so they
 * set this word and fill the affected chunk and everything downstream with NaN. */
int slx_read_scan_status(int *host_out);

#ifdef __cplusplus
}
#endif
#endif /* SLINOSS_B200_H_ */
