/* ossm_b200 -- C ABI of the B200 (sm_100a) recurrent-scan library.
 *
 * Drop-in boundary for the scan hot path of ossm (b-vitamins/ossm): these are
 * the entry points a binding for `ossm._kernels` calls instead of the
 * reference's pybind11 functions (src/ossm/csrc/bindings.cpp:159-223).  Plain
 * pointers and extents only; no allocation, no synchronisation, no exceptions.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer on the current CUDA device;
 *   - complex64 buffers are passed as `void*` to interleaved (re, im) float pairs;
 *   - all tensors are dense and contiguous in the stated layout;
 *   - kernels are enqueued on `stream` and the call returns immediately;
 *   - return value 0 = success, negative = error (see OSSM_B200_ERR_*), with a
 *     per-thread message available from ossm_b200_last_error().
 */
#ifndef OSSM_B200_H_
#define OSSM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* ossm_b200_stream_t; /* == cudaStream_t */

#define OSSM_B200_ERR_INVALID_ARGUMENT (-1)
#define OSSM_B200_ERR_CUDA (-2)
#define OSSM_B200_ERR_UNSUPPORTED (-3)
#define OSSM_B200_ERR_WORKSPACE (-4)

/* Recurrence variants of the time-invariant 2x2 oscillator scan. */
#define OSSM_B200_VARIANT_IMEX1 0       /* D-LinOSS imex1  (_dlinoss_scan.py:54-68)  */
#define OSSM_B200_VARIANT_IMEX2 1       /* D-LinOSS imex2  (_dlinoss_scan.py:69-75)  */
#define OSSM_B200_VARIANT_IM 2          /* D-LinOSS im     (_dlinoss_scan.py:76-84)  */
#define OSSM_B200_VARIANT_EX 3          /* D-LinOSS ex     (_dlinoss_scan.py:85-91)  */
#define OSSM_B200_VARIANT_LINOSS_IM 4   /* LinOSS IM       (linoss.py:244-251)       */
#define OSSM_B200_VARIANT_LINOSS_IMEX 5 /* LinOSS IMEX     (linoss.py:253-258)       */
/* Complex diagonal scan x_t = lambda x_{t-1} + b_t of the LRU / S5 layers (lru_scan.cpp:68-110,
 * s5_scan.cpp): a = Re lambda, g = Im lambda, step unused (may be NULL); grad_a / grad_g receive
 * Re / Im of sum_t G_t conj(x_{t-1}) (lru.py:69-78); only component 1 of states/carries is used. */
#define OSSM_B200_VARIANT_DIAG 6

/* ---- library ------------------------------------------------------------ */
int ossm_b200_version(void);
const char* ossm_b200_last_error(void);
/* Reads (and optionally clears) the device status word that a kernel sets when
 * one of its bounded waits gives up (0 = fine).  Synchronises the device. */
int ossm_b200_device_status(int* status, int clear);
/* Self-test of the bounded waits (no counterpart in the reference, whose kernels never wait):
 * launches one thread that waits on a barrier nothing ever completes, for at most `limit_ns`
 * (1 ns .. 100 ms) of GPU time.  The wait gives up, the kernel returns normally, *gave_up_dev
 * (a device int) becomes 1 and the device status word becomes 1 until it is read with clear. */
int ossm_b200_selftest_wait_timeout(uint64_t limit_ns, int* gave_up_dev, ossm_b200_stream_t stream);

/* ---- D-LinOSS / LinOSS oscillator scan ------------------------------------
 * Replaces ossm::dlinoss_{imex1,imex2,im,ex}_forward / _backward
 * (src/ossm/csrc/dlinoss_imex1.cpp:317-390, dlinoss_imex2.cpp:329-402,
 * dlinoss_im.cpp:347-420, dlinoss_ex.cpp:264-337; bindings.cpp:161-169) and,
 * for the two LinOSS variants, LinOSSLayer._run_recurrence with
 * _LinossScanFn.backward (src/ossm/models/linoss.py:83-151, 260-315).
 *
 *   a, g, step : float32 [P] (g may be NULL for the LinOSS variants)
 *   bu         : complex64 [L, B, P], time-major, P contiguous
 */

/* Steps between saved states ("carries") = rows per shared-memory stage. */
int ossm_b200_lti_chunk(void);
/* Bytes of the carry buffer written by forward and read by backward:
 * (ceil(L/chunk) - 1) * B * P * 16. */
size_t ossm_b200_lti_carry_bytes(int64_t L, int64_t B, int64_t P);
/* Bytes of scratch the backward needs: per-series partial sums (6*B*P floats) and, when a
 * long sequence of few series is split into time segments, the segment summaries. */
size_t ossm_b200_lti_backward_workspace_bytes(int64_t L, int64_t B, int64_t P);
/* Bytes of scratch for ossm_b200_lti_scan_forward_ws (0 unless the sequence is split). */
size_t ossm_b200_lti_forward_workspace_bytes(int64_t L, int64_t B, int64_t P);

/* Forward.  Any of the three outputs may be NULL, but not both x and states:
 *   x       : complex64 [L, B, P]      position state x_t (the op's result)
 *   states  : complex64 [L, B, P, 2]   full trajectory, the layout
 *             `ossm._kernels.dlinoss_*_forward` returns (bindings.cpp:12-15)
 *   carries : complex64 [ceil(L/chunk)-1, B, P, 2]  state after every chunk-th step
 */
int ossm_b200_lti_scan_forward(int variant, const float* a, const float* g, const float* step, const void* bu,
                               void* x, void* states, void* carries, int64_t L, int64_t B, int64_t P,
                               ossm_b200_stream_t stream);

/* Forward with scratch (16-byte aligned).  With fewer than ~12k series the time axis is
 * split into segments that run on different SMs: a summary pass finds every segment's
 * end state, a stitching kernel turns them into entry states (segment transition by
 * matrix power in double precision), and the scan proper starts each segment from its
 * entry state.  Results are those of ossm_b200_lti_scan_forward up to rounding of the
 * entry states.  The reference has one thread per series for any shape
 * (dlinoss_imex1_cuda.cu:189-197). */
int ossm_b200_lti_scan_forward_ws(int variant, const float* a, const float* g, const float* step, const void* bu,
                                  void* x, void* states, void* carries, void* workspace, size_t workspace_bytes,
                                  int64_t L, int64_t B, int64_t P, ossm_b200_stream_t stream);

/* Backward from the saved carries (recomputes the states chunk by chunk).
 *   grad_x : complex64 [L, B, P]  upstream gradient on x (contiguous)
 *   grad_bu: complex64 [L, B, P];  grad_a / grad_g / grad_step: float32 [P]
 *   (grad_g may be NULL for the LinOSS variants). */
int ossm_b200_lti_scan_backward(int variant, const float* a, const float* g, const float* step, const void* bu,
                                const void* carries, const void* grad_x, void* grad_bu, float* grad_a,
                                float* grad_g, float* grad_step, void* workspace, size_t workspace_bytes, int64_t L,
                                int64_t B, int64_t P, ossm_b200_stream_t stream);

/* The scan over one TIME SLICE of a longer sequence (no counterpart in the reference, which always holds the
 * whole sequence on the device): a caller that streams a long sequence through the GPU piece by piece hands
 * the recurrence state from slice to slice.
 *   state_in  : complex64 [B, P, 2] state (s0, s1) entering the slice, NULL = zero (the first slice)
 *   state_out : complex64 [B, P, 2] state leaving the slice, NULL = not wanted
 *   carries   : as in ossm_b200_lti_scan_forward, for this slice alone (ossm_b200_lti_carry_bytes(L, B, P))
 * Backward slices run in reverse time order:
 *   adjoint_in  : complex64 [B, P, 2] adjoint entering the slice from the later slice, NULL = zero (the last slice)
 *   adjoint_out : complex64 [B, P, 2] adjoint leaving towards the earlier slice, NULL = not wanted
 *   state_in    : the state_in the forward call of the same slice was given
 * grad_a / grad_g / grad_step receive this slice's share of the coefficient gradients (the caller adds the
 * slices).  The states and grad_bu of a sliced run are those of the unsliced call bit for bit when the slices
 * are multiples of ossm_b200_lti_chunk() steps (same arithmetic, step for step); the coefficient gradients
 * agree up to the rounding of their partial sums. */
int ossm_b200_lti_scan_forward_slice(int variant, const float* a, const float* g, const float* step, const void* bu,
                                     void* x, void* carries, const void* state_in, void* state_out, int64_t L,
                                     int64_t B, int64_t P, ossm_b200_stream_t stream);
int ossm_b200_lti_scan_backward_slice(int variant, const float* a, const float* g, const float* step, const void* bu,
                                      const void* carries, const void* state_in, const void* grad_x,
                                      const void* adjoint_in, void* adjoint_out, void* grad_bu, float* grad_a,
                                      float* grad_g, float* grad_step, void* workspace, size_t workspace_bytes,
                                      int64_t L, int64_t B, int64_t P, ossm_b200_stream_t stream);

/* Backward with the reference's argument list: the full trajectory `states`
 * ([L,B,P,2], as returned by forward) stands in for the carries
 * (dlinoss_imex1.cpp:354-390 takes a_diag, g_diag, step, bu, states, grad_output). */
int ossm_b200_lti_scan_backward_states(int variant, const float* a, const float* g, const float* step,
                                       const void* bu, const void* states, const void* grad_x, void* grad_bu,
                                       float* grad_a, float* grad_g, float* grad_step, void* workspace,
                                       size_t workspace_bytes, int64_t L, int64_t B, int64_t P,
                                       ossm_b200_stream_t stream);

/* Backward for callers that cannot provide scratch memory (no counterpart in the
 * reference).  Same arguments and results as ossm_b200_lti_scan_backward minus the
 * workspace: the per-series partial sums -- and, when a long sequence of few series is
 * split into time segments, the segment summaries (at most 1.1 MB for any shape the
 * split applies to, so the split is the one ossm_b200_lti_scan_backward makes with the
 * workspace it asks for) -- go to a fixed 1.5 MiB array that is part of the library image
 * on every GPU that loads it.  Meant for hosts that may not
 * allocate device memory when the call is made -- a serving or control process that
 * freezes its allocations after start-up, or a foreign-language stub (cgo, JNI) that
 * owns no CUDA allocator.  Limits and rules:
 *   - B*P must not exceed ossm_b200_lti_scan_backward_static_max_series() (65536);
 *     larger problems are refused with OSSM_B200_ERR_WORKSPACE;
 *   - all calls on a device share the one array: calls that may overlap on the GPU
 *     (different streams) race -- keep them on one stream or serialise them;
 *   - the first call on each device looks up the array's device address; make that
 *     call, with the device current, before starting any stream capture;
 *   - nothing in the array has to be cleared between calls (every element that is
 *     read has been written by the same call). */
size_t ossm_b200_lti_scan_backward_static_max_series(void);
int ossm_b200_lti_scan_backward_static(int variant, const float* a, const float* g, const float* step,
                                       const void* bu, const void* carries, const void* grad_x, void* grad_bu,
                                       float* grad_a, float* grad_g, float* grad_step, int64_t L, int64_t B,
                                       int64_t P, ossm_b200_stream_t stream);

/* Launch-shape knobs ("fwd_ring", "fwd_warps", "bwd_ring", "bwd_warps", "force_plain",
 * "segments" = forced number of time segments, 0 = automatic); process-wide, meant for
 * benchmarking and tests. */
int ossm_b200_lti_set_tuning(const char* key, int value);

/* ---- projections of the D-LinOSS layer on the tensor cores ---------------------------
 * The layer body around the scan (src/ossm/models/dlinoss.py:217-247):
 *     bu = u B_re^T + i u B_im^T  ->  permute to [L,B,P]  ->  scan  ->  permute back  ->
 *     y  = x.real C_re^T - x.imag C_im^T + u * D
 * is two instances of   out[dest(m), n] = sum_k A[m,k] W[n,k]  (+ diag[n] * aux[dest(m), n])
 * where dest() is the row permutation between batch-major (b*L + l) and time-major (l*B + b)
 * row order, so the permute copies and the real / imaginary splits disappear:
 *     prologue  A = u [B*L, H],   W = rows (B_re[p], B_im[p]) interleaved [2P, H],
 *               out = bu viewed as float [L*B, 2P], row_map 1
 *     epilogue  A = x viewed as float [L*B, 2P], W = columns (C_re[:,p], -C_im[:,p]) interleaved [H, 2P],
 *               out = y [B*L, H], aux = u, diag = D, row_map 2
 * and likewise in the backward pass.  The product is evaluated on the tcgen05 tensor cores as
 * three TF32 products of hi / lo operand halves (float32-level accuracy, float32 accumulation).
 *
 *   A          float32 [M, K] dense row-major, 16-byte aligned, K a multiple of 4
 *   W_hi, W_lo float32 [N, K]: the two halves of the weight matrix made by ossm_b200_split_tf32
 *   out, aux   float32, row pitch ldo floats (aux is read at the same position out is written)
 *   diag       float32 [N]; aux and diag are both NULL or both given
 *   row_map    0: dest(m) = m;  1: m = b*length + l -> l*batch + b;  2: m = l*batch + b -> b*length + l
 *   col_block, plane_stride
 *              the output may be split into planes of col_block columns each, plane_stride floats apart
 *              (column n -> plane n / col_block, column n % col_block; ldo is then the row pitch inside a
 *              plane): the layout a reduce-scatter over the output columns consumes.  col_block <= 0 or
 *              >= N means one plain [M, N] matrix.
 */
#define OSSM_B200_ROWS_IDENTITY 0
#define OSSM_B200_ROWS_BATCH_TO_TIME 1
#define OSSM_B200_ROWS_TIME_TO_BATCH 2
int ossm_b200_split_tf32(const float* w, float* w_hi, float* w_lo, int64_t count, ossm_b200_stream_t stream);
int ossm_b200_gemm_tf32x3(const float* A, const float* W_hi, const float* W_lo, float* out, const float* aux,
                          const float* diag, int64_t M, int64_t N, int64_t K, int64_t ldo, int64_t col_block,
                          int64_t plane_stride, int row_map, int64_t batch, int64_t length,
                          ossm_b200_stream_t stream);

/* Weight gradients of the two projections: out[m, n] = sum over all (b, l) of X[row(b,l), m] * Y[row(b,l), n]
 * (grad_B from grad_bu and u, grad_C from grad_y and x), same three-product TF32 scheme.  X [batch*length, M] and
 * Y [batch*length, N] are dense float32 matrices whose rows are ordered batch-major (b*length + l,
 * *_time_major = 0) or time-major (l*batch + b, 1), independently of each other; M and N must be multiples of 32.
 * The contraction is divided over *splits_out CTAs per output tile, each of which writes one partial
 * [M, N] matrix into `partial` (ossm_b200_wgrad_tf32x3_workspace_bytes() bytes); the caller adds the
 * partials (fixed order: deterministic). */
size_t ossm_b200_wgrad_tf32x3_workspace_bytes(int64_t M, int64_t N, int64_t batch, int64_t length);
int ossm_b200_wgrad_tf32x3(const float* X, int x_time_major, const float* Y, int y_time_major, float* partial,
                           size_t partial_bytes, int* splits_out, int64_t M, int64_t N, int64_t batch,
                           int64_t length, ossm_b200_stream_t stream);

/* grad_D of the layer (y = ... + D * u, dlinoss.py:247): partial[c, n] = sum over the rows of CTA c of
 * X[m, n] * Y[m, n] for dense float32 [rows, cols] matrices (cols a multiple of 4, 16-byte aligned).  `partial` has
 * ossm_b200_colwise_dot_partials(rows) rows of `cols` floats; the caller adds them (fixed order: deterministic). */
/* Key "reserve_sms" (0 .. 64, default 0): SMs the persistent projection and weight-gradient kernels leave free, for a
 * caller that runs a collective beside them (their CTAs fill an SM's shared memory).  Read at launch time; the workspace
 * query and the launch of one weight gradient must see the same value. */
int ossm_b200_layer_set_tuning(const char* key, int value);
int ossm_b200_colwise_dot_partials(int64_t rows);
int ossm_b200_colwise_dot(const float* X, const float* Y, float* partial, int64_t rows, int64_t cols,
                          ossm_b200_stream_t stream);

/* ---- generic LinOSS scan (complex 2x2 per channel, forcing per step) --------
 * Replaces ossm::linoss_scan (src/ossm/csrc/linoss_scan.cpp:115-146; bindings.cpp:160)
 * and the Python-loop backward of _LinossScanFn (src/ossm/models/linoss.py:83-151).
 *
 *   m11, m12, m21, m22 : complex64 [P]
 *   b_seq, out/states, grad_out, grad_b : complex64 [L, B, P, 2] (16-byte aligned)
 *   grad_m : complex64 [P, 2, 2]  =  sum_{t,b} G_t conj(s_{t-1})^T   (the caller keeps
 *            the real part when the transition matrix is real, linoss.py:133-138)
 */
int ossm_b200_linoss_scan_forward(const void* m11, const void* m12, const void* m21, const void* m22,
                                  const void* b_seq, void* out, int64_t L, int64_t B, int64_t P,
                                  ossm_b200_stream_t stream);
size_t ossm_b200_linoss_scan_backward_workspace_bytes(int64_t L, int64_t B, int64_t P);
int ossm_b200_linoss_scan_backward(const void* m11, const void* m12, const void* m21, const void* m22,
                                   const void* states, const void* grad_out, void* grad_b, void* grad_m,
                                   void* workspace, size_t workspace_bytes, int64_t L, int64_t B, int64_t P,
                                   ossm_b200_stream_t stream);

/* ---- selective D-LinOSS (per-step coefficients) ---------------------------------
 * Replaces ossm::sdlinoss_<v>_forward / sdlinoss_<v>_backward for v = imex1, imex2, im, ex
 * (src/ossm/csrc/sdlinoss_imex1.cpp:331-427 and the same entries of sdlinoss_imex2.cpp,
 * sdlinoss_im.cpp, sdlinoss_ex.cpp; CUDA bodies sdlinoss_<v>_cuda.cu; bindings.cpp).
 * `variant` is OSSM_B200_VARIANT_IMEX1 .. OSSM_B200_VARIANT_EX.
 *
 *   A, G, step : float32 fields over (L, B, M).  `*_strides` points at three element
 *                strides {L, B, M} in host memory; a stride of 0 marks a broadcast axis
 *                (the forms (M,), (L,M), (B,M), (L,B,M) of the reference's Strided3,
 *                dlinoss_common.h:25-41).  The raw step is clamped to [1e-6, 1] inside.
 *   bu, x, grad_x, grad_bu : complex64 [L, B, M], contiguous
 *   states     : complex64 [L, B, M, 2] = (w, x) per step, the reference's forward output
 *   carries    : the state after every ossm_b200_sdlinoss_carry_interval() steps,
 *                ossm_b200_sdlinoss_carry_bytes() bytes; what the backward needs instead of
 *                `states`
 *
 * Forward writes `x` and / or `states` (either may be NULL, not both) and `carries` when
 * given.  Backward takes `states` or `carries` (states wins; neither is needed for
 * L <= ossm_b200_lti_chunk()) and writes grad_bu and grad_A / grad_G / grad_step, each laid
 * out with the strides of its parameter.  A gradient whose parameter is broadcast along
 * the batch or state axis is accumulated with atomic adds and must be zero on entry (the
 * reference allocates it with at::zeros_like); every other gradient is overwritten.
 * The TMA-staged kernels run when A, G, step are all dense [L, B, M] with 16-byte aligned
 * bases and B*M a multiple of 4; other views take plain-load kernels.
 */
int ossm_b200_sdlinoss_carry_interval(void);
size_t ossm_b200_sdlinoss_carry_bytes(int64_t L, int64_t B, int64_t M);
int ossm_b200_sdlinoss_forward(int variant, const float* A, const int64_t* A_strides, const float* G,
                               const int64_t* G_strides, const float* step, const int64_t* step_strides,
                               const void* bu, void* x, void* states, void* carries, int64_t L, int64_t B,
                               int64_t M, ossm_b200_stream_t stream);
int ossm_b200_sdlinoss_backward(int variant, const float* A, const int64_t* A_strides, const float* G,
                                const int64_t* G_strides, const float* step, const int64_t* step_strides,
                                const void* bu, const void* carries, const void* states, const void* grad_x,
                                float* grad_A, float* grad_G, float* grad_step, void* grad_bu, int64_t L,
                                int64_t B, int64_t M, ossm_b200_stream_t stream);
/* Launch-shape knobs of the two kernels above (keys fwd_ring, fwd_warps, bwd_ring, bwd_warps,
 * force_plain); for experiments, the defaults are the measured best. */
int ossm_b200_sdlinoss_set_tuning(const char* key, int value);

/* ---- Mamba selective scan ------------------------------------------------------
 * Replaces ossm::selective_scan_cuda_forward / selective_scan_cuda_backward
 * (src/ossm/csrc/selective_scan_cuda.cu:253-393; bindings.cpp:199-222) and the CPU
 * pair selective_scan / selective_scan_backward (selective_scan_cpu.cpp:78-360).
 *
 *   u, z, out, dout, du, dz : [B, D, L]  element type `io_dtype` (time contiguous)
 *   dt, ddt                 : [B, D, L]  float32
 *   A, dA                   : [D, N]     float32
 *   Bm, Cm                  : [B, N, L]  element type `io_dtype` (time contiguous; the
 *                             transpose of ossm's [B, L, N] argument)
 *   dB, dC                  : [B, N, L]  float32 (zeroed by the call)
 *   z / dz, Dskip / dD      : optional (NULL): SiLU gate and skip term Dskip[d]*u
 *   chunk_states            : float32, B * D * ceil(L/chunk) * N values: the state entering
 *                             each chunk, in a layout private to the kernel pair; written by
 *                             forward (may be NULL when no backward will follow), read by
 *                             backward.
 */
#define OSSM_B200_DTYPE_F32 0
#define OSSM_B200_DTYPE_BF16 1

/* Time steps between the states the forward saves for the backward, for a state size N. */
int ossm_b200_selective_scan_chunk(int64_t N);
/* Kernel choice for experiments: key "serial" = 1 (default) runs the serial-in-time kernels for the
 * state sizes they cover (d_state 16), 0 the time-parallel kernels for every size; it changes the
 * value of ossm_b200_selective_scan_chunk(), so forward and backward of one scan must run under the
 * same setting.  Key "bwd_split" = 2 (default) or 4: lanes per channel in the serial backward of d_state 16.
 * Key "split_bwd_wide_from": state size from which the backward of d_state 32 .. 256 uses 8-warp CTAs.
 * Key "split_flush_parts": threads sharing one item of that backward's dB / dC sums (0 = measured default by state size). */
int ossm_b200_selective_scan_set_tuning(const char* key, int value);
size_t ossm_b200_selective_scan_state_bytes(int64_t B, int64_t D, int64_t L, int64_t N);
size_t ossm_b200_selective_scan_backward_workspace_bytes(int64_t B, int64_t D, int64_t L, int64_t N);

/* delta_bias (float32 [D], may be NULL) and delta_softplus (0 / 1) fold the step-size transform of the
 * Mamba mixer into the scan: the kernels use dt = raw + delta_bias[d], passed through softplus when
 * delta_softplus is set (identity above 20) -- the switches of the vendored kernel
 * (csrc/mamba/selective_scan_fwd_kernel.cuh:123-161) that ossm's wrapper leaves off
 * (selective_scan_cuda.cu:133-140) while the mixer applies F.softplus(dt_proj(.)) as a separate pass
 * (mambarec.py:155).  With either of them `ddt` is the gradient of the raw step, and ddelta_bias
 * (float32 [D], required when delta_bias is given) receives the gradient of the bias. */
int ossm_b200_selective_scan_forward(const void* u, const float* dt, const float* A, const void* Bm, const void* Cm,
                                     const void* z, const float* Dskip, const float* delta_bias, int delta_softplus,
                                     void* out, float* chunk_states, int64_t B, int64_t D, int64_t L, int64_t N,
                                     int io_dtype, ossm_b200_stream_t stream);

int ossm_b200_selective_scan_backward(const void* u, const float* dt, const float* A, const void* Bm,
                                      const void* Cm, const void* z, const float* Dskip, const float* delta_bias,
                                      int delta_softplus, const void* dout, const float* chunk_states, void* du,
                                      float* ddt, float* dA, float* dB, float* dC, void* dz, float* dD,
                                      float* ddelta_bias, void* workspace, size_t workspace_bytes, int64_t B,
                                      int64_t D, int64_t L, int64_t N, int io_dtype, ossm_b200_stream_t stream);

/* The same pair with Bm, Cm given [B, L, N] -- the order of ossm's own arguments (a step's N values contiguous,
 * bindings.cpp:199-222) -- with bc_pitch elements between the rows of consecutive steps (N for dense tensors; the
 * mixer's B and C are column slices of one projection, mambarec.py:153-154, whose row pitch is dt_rank + 2 N), so
 * that the caller's transposing copies disappear; dB, dC stay dense [B, N, L].  Taken for the
 * state sizes whose kernels keep a [step][state] tile in shared memory: ossm_b200_selective_scan_step_major_bc(N)
 * returns 1 for them (d_state 16, 32, 64, 128, 256 under the default kernel choice), 0 otherwise, and the calls
 * return an error for any other N. */
int ossm_b200_selective_scan_step_major_bc(int64_t N);
int ossm_b200_selective_scan_forward_step_major_bc(const void* u, const float* dt, const float* A, const void* Bm,
                                                   const void* Cm, const void* z, const float* Dskip,
                                                   const float* delta_bias, int delta_softplus, void* out,
                                                   float* chunk_states, int64_t B, int64_t D, int64_t L, int64_t N,
                                                   int64_t bc_pitch, int io_dtype, ossm_b200_stream_t stream);
int ossm_b200_selective_scan_backward_step_major_bc(const void* u, const float* dt, const float* A, const void* Bm,
                                                    const void* Cm, const void* z, const float* Dskip,
                                                    const float* delta_bias, int delta_softplus, const void* dout,
                                                    const float* chunk_states, void* du, float* ddt, float* dA,
                                                    float* dB, float* dC, void* dz, float* dD, float* ddelta_bias,
                                                    void* workspace, size_t workspace_bytes, int64_t B, int64_t D,
                                                    int64_t L, int64_t N, int64_t bc_pitch, int io_dtype,
                                                    ossm_b200_stream_t stream);

/* ---- causal depthwise conv1d + bias + SiLU of the Mamba mixer ----------------------------------
 * Replaces the chain transpose -> F.pad -> nn.Conv1d(groups = D) -> nn.SiLU -> transpose of
 * _MambaMixer.forward (src/ossm/models/mambarec.py:143-151) by one pass that reads x once and writes
 * the result in both layouts its consumers need:
 *   x        float32 [B, L, D] with row pitch ldx floats (the x half of in_proj's output has ldx = 2 D)
 *   weight   float32 [D, taps] (nn.Conv1d's [D, 1, taps]), taps = 1..4;  bias float32 [D] or NULL
 *   out_bdl  float32 [B, D, L]  (time contiguous: the selective scan's operand), may be NULL
 *   out_bld  float32 [B, L, D]  (channel contiguous: the x_proj GEMM's operand), may be NULL
 * Backward takes the upstream gradient of either or both outputs and writes grad_x [B, L, D],
 * grad_weight [D, taps] and grad_bias [D] (sums over batch and time, accumulated with float atomics:
 * not bitwise reproducible from run to run). */
int ossm_b200_conv1d_silu_forward(const float* x, int64_t ldx, const float* weight, const float* bias, float* out_bdl,
                                  float* out_bld, int64_t B, int64_t L, int64_t D, int taps,
                                  ossm_b200_stream_t stream);
int ossm_b200_conv1d_silu_backward(const float* x, int64_t ldx, const float* weight, const float* bias,
                                   const float* grad_bdl, const float* grad_bld, float* grad_x, float* grad_weight,
                                   float* grad_bias, int64_t B, int64_t L, int64_t D, int taps,
                                   ossm_b200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* OSSM_B200_H_ */
