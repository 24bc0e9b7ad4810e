/*
 * lrnnx_b200.h — C ABI of liblrnnx_b200.so, the sm_100a scan back end for lrnnx.
 *
 * Every entry point takes a pointer to a plain-old-data argument block (raw
 * device pointers, sizes, element strides, flags) plus the CUDA stream to
 * launch on (a cudaStream_t passed as void*), and returns an int status:
 *   0            success (kernels enqueued on `stream`; nothing is synchronised)
 *   negative     argument rejected (B200_ERR_*); b200_last_error() has the text
 *   positive     CUDA runtime error code from the launch
 * No entry point allocates device memory unless its comment says so; outputs
 * and accumulators are caller-allocated.  All strides count ELEMENTS of the
 * tensor's own dtype (a complex64 element is one element).  The innermost
 * (sequence) stride of every activation tensor must be 1.
 *
 * The "replaces" notes cite the lrnnx source file and lines whose behaviour the
 * entry point reproduces (paths are relative to the lrnnx repository root).
 */
#ifndef LRNNX_B200_H_
#define LRNNX_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* activation dtypes */
enum { B200_F32 = 0, B200_F16 = 1, B200_BF16 = 2 };

/* discretization methods; same set and meaning as
 * csrc/selective_scan/selective_scan.h:14-21 (enum DiscretizationMethod) */
enum {
  B200_DISC_ZOH = 0,
  B200_DISC_BILINEAR = 1,
  B200_DISC_DIRAC = 2,
  B200_DISC_MAMBA = 3,
  B200_DISC_RGLRU = 4,
  B200_DISC_S7 = 5
};

/* status codes */
enum {
  B200_OK = 0,
  B200_ERR_NULL = -1,      /* required pointer is null */
  B200_ERR_SHAPE = -2,     /* size out of range (e.g. dstate > 256) */
  B200_ERR_DTYPE = -3,     /* unknown dtype / discretization / combination */
  B200_ERR_ALIGN = -4,     /* pointer alignment */
  B200_ERR_UNSUPPORTED = -5,
  B200_ERR_TOO_LARGE = -6  /* exceeds a fixed capacity of a no-allocation entry point */
};

const char *b200_last_error(void);   /* thread-local text of the last negative status */
int b200_abi_version(void);          /* bumped when any struct below changes */
int b200_sizeof(const char *struct_name);   /* sizeof() of a named argument block, -1 if unknown */

/* ------------------------------------------------------------------------
 * Selective scan forward.
 * Replaces selective_scan_fwd (csrc/selective_scan/selective_scan_cpu.cpp:263-421)
 * and the kernel it launches (csrc/selective_scan/selective_scan.cuh:73-382).
 *   u, delta, z, deltaA, out, out_z : (batch, dim, seqlen) activations dtype
 *   A : (dim, dstate) float32 or complex64
 *   B, C : constant (dim, dstate) in A's dtype, or variable
 *          (batch, n_groups, dstate, seqlen) activations dtype
 *          (last dim 2*seqlen interleaved re/im when A is complex)
 *   D, delta_bias : (dim) float32, nullable
 *   x : (batch, dim, n_chunks, 2*dstate) in A's dtype, n_chunks = ceil(seqlen/2048);
 *       x[b,d,c,2n] = running product of the discrete A from t=0 to the end of
 *       chunk c, x[b,d,c,2n+1] = state at the end of chunk c.
 * ------------------------------------------------------------------------ */
typedef struct b200_selscan_fwd_args {
  int32_t batch, dim, seqlen, dstate, n_groups;
  int32_t dtype;            /* B200_F32 / F16 / BF16: u, delta, z, deltaA, variable B/C, out */
  int32_t is_complex;       /* A (and constant B/C, x) are complex64 */
  int32_t var_B, var_C;
  int32_t delta_softplus;
  int32_t method;           /* B200_DISC_* */
  int32_t l_segments;       /* forward only; 0 or 1: plain scan.  S > 1: the sequence is cut into S
                               segments of ceil(seqlen/S) steps rounded up to a multiple of 2048, each
                               scanned from a zero state by its own thread blocks (more parallelism for
                               long rows); out, out_z and x of segments >= 1 are then zero-start results
                               that the caller must stitch with b200_selscan_fixup (n_segments = S).
                               Honoured only on the shape class served by the throughput kernels,
                               rejected with B200_ERR_UNSUPPORTED elsewhere. */
  int32_t stage_len;        /* spacing in steps of the states in stage_h: the value returned by
                               b200_selscan_stage_states() for this problem (0 when stage_h is NULL) */
  int32_t reserved0;
  const void *u, *delta, *A, *B, *C;
  const void *D, *z, *delta_bias, *deltaA;      /* nullable */
  void *out;                                    /* (batch, dim, seqlen) */
  void *out_z;                                  /* required iff z != NULL */
  void *x;                                      /* required */
  void *stage_h;                                /* nullable; no counterpart in the reference.  (batch, dim,
                                                   ceil(seqlen/stage_len), dstate) float32, 16-byte aligned: the
                                                   state at the end of every stage of stage_len steps.  Written
                                                   by the forward call and read by the backward call (which then
                                                   skips its recomputation of these states) only where
                                                   b200_selscan_stage_states() says so; ignored otherwise. */
  int64_t u_bs, u_ds;
  int64_t delta_bs, delta_ds;
  int64_t z_bs, z_ds;
  int64_t deltaA_bs, deltaA_ds;
  int64_t out_bs, out_ds;
  int64_t out_z_bs, out_z_ds;
  int64_t A_ds, A_ns;
  int64_t B_bs, B_gs, B_ns;   /* variable: batch/group/state strides; constant: B_gs = dim stride */
  int64_t C_bs, C_gs, C_ns;
} b200_selscan_fwd_args;

int b200_selscan_fwd(const b200_selscan_fwd_args *args, void *stream);

/* Stage spacing (in steps) with which b200_selscan_fwd with these arguments (stage_h and
 * stage_len aside) would write stage_h and b200_selscan_bwd on the same problem would read it;
 * 0 if stage states are not used for this problem.  Non-zero on the shape class of the throughput
 * kernels with l_segments <= 1: 32 for the streaming kernels (enough rows to fill the GPU with
 * one warp per 16 channels), 256 for the lane-scan kernels. */
int b200_selscan_stage_states(const b200_selscan_fwd_args *args);

/* ------------------------------------------------------------------------
 * Selective scan backward (reverse scan with recomputation of the states).
 * Replaces selective_scan_bwd (csrc/selective_scan/selective_scan_cpu.cpp:423-632)
 * and its kernel (csrc/selective_scan/selective_scan_backward.cuh:86-845).
 * The caller zero-fills dA, dB, dC, dD, ddelta_bias before the call; the kernel
 * accumulates into them with atomics.  dB/dC are float32 accumulators when the
 * matching input is variable ((batch, n_groups, dstate, seqlen[*2]) float32),
 * otherwise (dim, dstate) in A's dtype.
 *   x   : forward checkpoints; may be NULL only when seqlen <= 2048
 *   out : forward output before gating; required iff z != NULL
 *   dz  : required iff z != NULL;  out_z : optional recomputed gated output
 * ------------------------------------------------------------------------ */
typedef struct b200_selscan_bwd_args {
  b200_selscan_fwd_args f;   /* f.out = saved forward `out` (or NULL), f.out_z = optional recompute target */
  const void *dout;          /* (batch, dim, seqlen) activations dtype */
  void *du, *ddelta;         /* (batch, dim, seqlen) activations dtype */
  void *ddeltaA;             /* required iff f.deltaA != NULL */
  void *dz;                  /* required iff f.z != NULL */
  void *dA;                  /* (dim, dstate) A dtype, zero-filled */
  void *dB, *dC;             /* see above, zero-filled */
  void *dD, *ddelta_bias;    /* (dim) float32 zero-filled; required iff D / delta_bias given */
  int64_t dout_bs, dout_ds;
  int64_t du_bs, du_ds;
  int64_t ddelta_bs, ddelta_ds;
  int64_t ddeltaA_bs, ddeltaA_ds;
  int64_t dz_bs, dz_ds;
  int64_t dA_ds, dA_ns;
  int64_t dB_bs, dB_gs, dB_ns;
  int64_t dC_bs, dC_gs, dC_ns;
  /* Sequence-parallel backward (both optional, float32 (batch, dim, dstate), real A only; no
   * counterpart in lrnnx).  h_in: the state entering the first step (instead of zero), with f.x
   * holding the checkpoints corrected for it (b200_selscan_fixup does that).  q_in: the gradient
   * of the loss with respect to the state after the last step, i.e. what later slices of the
   * sequence send back (b200_selscan_adjoint_summary, folded from the right). */
  const void *h_in, *q_in;
} b200_selscan_bwd_args;

int b200_selscan_bwd(const b200_selscan_bwd_args *args, void *stream);

/* ------------------------------------------------------------------------
 * Sequence-parallel helpers for the selective scan (no counterpart in lrnnx,
 * which is single-GPU; they implement the chunk-summary exchange that
 * the long-sequence benchmark configuration asks for).
 * b200_selscan_fixup adds the contribution of an incoming state h_in
 * (batch, dim, dstate) float32 to an already computed zero-state output:
 *   out[b,d,t] += sum_n C[t,n] * (prod_{k<=t} a_k[n]) * h_in[b,d,n]
 * and rewrites out_z, the checkpoints x (product entries are multiplied by
 * p_in, state entries corrected) accordingly.  Real A, variable B/C only.
 * ------------------------------------------------------------------------ */
typedef struct b200_selscan_fixup_args {
  b200_selscan_fwd_args f;      /* same tensors as the forward call on this rank's slice */
  const void *h_in;             /* (n_segments, batch, dim, dstate) float32: state entering each segment */
  const void *p_in;             /* same shape: product of a over everything before the segment */
  int32_t n_segments;           /* 0 or 1: the whole slice is one segment */
  int32_t seg_len;              /* segment length in steps (multiple of 2048) when n_segments > 1;
                                   segment s covers [s*seg_len, min(seqlen, (s+1)*seg_len)); entries of
                                   h_in / p_in for a segment that needs no correction may be 0 / 1 */
} b200_selscan_fixup_args;

int b200_selscan_fixup(const b200_selscan_fixup_args *args, void *stream);

/* Folds the zero-start summaries of the n_segments > 1 segments of one forward call (the last
 * checkpoint entry of each segment in f.x) into the state and product entering every segment:
 *   h_in[0] = 0, p_in[0] = 1,  h_in[s] = P[s-1] h_in[s-1] + h[s-1],  p_in[s] = p_in[s-1] P[s-1].
 * Writes h_in and p_in (same layout as above; the pointers are outputs here); uses f.x, f.batch,
 * f.dim, f.dstate, f.seqlen, n_segments and seg_len only. */
int b200_selscan_fold(const b200_selscan_fixup_args *args, void *stream);

/* Adjoint summary of a slice for the sequence-parallel backward: what the slice hands to the
 * slice before it when nothing arrives from the slices after it,
 *   G[b,d,n] = sum_t (prod_{k<=t} a_k[n]) * C[t,n] * dy[b,d,t],   dy = dout (* silu(z) when z is given),
 * a_k = exp(delta'_k A_n) with delta' = delta after bias and softplus (the transposed map of
 * b200_selscan_fixup; same restrictions: real A, variable C, "mamba" / "zoh" / "dirac" without
 * deltaA).  With P = the product of a over the whole slice (the forward's last checkpoint entry
 * before the fix-up) the gradient arriving at the end of slice r-1 is q[r-1] = G[r] + P[r] q[r].
 * Uses f.delta, f.delta_bias, f.delta_softplus, f.A, f.C, f.z and their strides; dout
 * (batch, dim, seqlen) activations dtype with the strides given; G float32 (batch, dim, dstate). */
typedef struct b200_selscan_adjsum_args {
  b200_selscan_fwd_args f;
  const void *dout;
  void *G;
  int64_t dout_bs, dout_ds;
} b200_selscan_adjsum_args;

int b200_selscan_adjoint_summary(const b200_selscan_adjsum_args *args, void *stream);

/* ------------------------------------------------------------------------
 * Simplified (diagonal, complex-input) scan used by LTV-S5.
 * Replaces simplified_scan_fwd/bwd (csrc/simplified_scan/simplified_scan_cpu.cpp:160-331)
 * and kernels (csrc/simplified_scan/simplified_scan.cuh:85-262,
 * csrc/simplified_scan/simplified_scan_backward.cuh:91-420).
 *   u, out, dout, du : (batch, dim, seqlen) complex64
 *   delta, deltaA, ddelta, ddeltaA : (batch, dim, seqlen) float32
 *   A, B, C, dA, dB, dC : (dim, dstate) complex64  (dA/dB/dC zero-filled by caller;
 *                         dB and dC may both be null when dstate == 1: the sums are then skipped)
 *   x : (batch, dim, n_chunks, 2*dstate) complex64
 *   method : ZOH, BILINEAR or DIRAC
 * ------------------------------------------------------------------------ */
typedef struct b200_simpscan_args {
  int32_t batch, dim, seqlen, dstate;
  int32_t method;
  int32_t reserved0;
  const void *u, *delta, *A, *B, *C;
  const void *deltaA;              /* nullable */
  void *out;                       /* fwd: output.  bwd: optional (nullable), the forward output for the
                                      same arguments; with dstate == 1 and B C != 0 it is the state sequence
                                      and the backward then skips the forward recomputation */
  void *x;                         /* fwd: written; bwd: read (may be NULL when seqlen <= 2048) */
  int64_t u_bs, u_ds, delta_bs, delta_ds, deltaA_bs, deltaA_ds, out_bs, out_ds;
  int64_t A_ds, A_ns, B_ds, B_ns, C_ds, C_ns;
  /* backward only */
  const void *dout;
  void *du, *ddelta, *ddeltaA;
  void *dA, *dB, *dC;
  int64_t dout_bs, dout_ds, du_bs, du_ds, ddelta_bs, ddelta_ds, ddeltaA_bs, ddeltaA_ds;
} b200_simpscan_args;

int b200_simpscan_fwd(const b200_simpscan_args *args, void *stream);
int b200_simpscan_bwd(const b200_simpscan_args *args, void *stream);

/* Diagnostic: non-zero after a kernel abandoned a bounded wait on a shared-memory
 * barrier (its outputs are then invalid).  Synchronises the device. */
int b200_device_status(void);

/* ------------------------------------------------------------------------
 * One-token state update used in decoding.
 * Replaces selective_state_update and its Triton kernel
 * (lrnnx/ops/triton/selective_state_update.py:300-476, 17-297).
 * All tensors are described in the 4-D "heads" form; strides may be 0 for
 * broadcast dimensions.  `state` is updated in place.
 *   state (batch|*, nheads, dim, dstate) state_dtype
 *   x, dt, z, deltaA, out (batch, nheads, dim) act dtype
 *   A (nheads, dim, dstate) f32 ; B, C (batch, ngroups, dstate) bc dtype
 *   D, dt_bias (nheads, dim) ; state_batch_indices (batch) int32, nullable
 * ------------------------------------------------------------------------ */
typedef struct b200_ssu_args {
  int32_t batch, nheads, dim, dstate, ngroups;
  int32_t state_dtype, x_dtype, dt_dtype, A_dtype, bc_dtype, D_dtype, z_dtype, dt_bias_dtype, deltaA_dtype;
  int32_t dt_softplus;
  int32_t method;
  int32_t reserved0;
  void *state;
  const void *x, *dt, *A, *B, *C;
  const void *D, *z, *dt_bias, *deltaA;         /* nullable */
  const int32_t *state_batch_indices;           /* nullable */
  void *out;                                    /* x dtype */
  int64_t state_bs, state_hs, state_ds, state_ns;
  int64_t x_bs, x_hs, x_ds;
  int64_t dt_bs, dt_hs, dt_ds;
  int64_t A_hs, A_ds, A_ns;
  int64_t B_bs, B_gs, B_ns;
  int64_t C_bs, C_gs, C_ns;
  int64_t D_hs, D_ds;
  int64_t z_bs, z_hs, z_ds;
  int64_t dt_bias_hs, dt_bias_ds;
  int64_t deltaA_bs, deltaA_hs, deltaA_ds;
  int64_t out_bs, out_hs, out_ds;
} b200_ssu_args;

int b200_ssu_step(const b200_ssu_args *args, void *stream);

/* ------------------------------------------------------------------------
 * One-token update of the S5 (simplified) recurrence with its projections fused.
 * Replaces simplified_state_update and its Triton kernel
 * (lrnnx/ops/triton/simplified_state_update.py:254-401, 13-251):
 *   Bu = B x;  state <- a * state + k * Bu  (a, k as in the simplified scan, from dt / deltaA);
 *   out = (conj_sym ? 2 : 1) * Re(C state) + D x.
 *   state (batch, P) complex64, in place; x, out (batch, H) float32;
 *   dt, deltaA (batch, P) float32 (batch stride 0 for a (P,) tensor); A (P) complex64;
 *   B (P, H), C (H, P) complex64 row-major dense; D (H, H) float32 row-major dense, nullable.
 * ------------------------------------------------------------------------ */
typedef struct b200_s5_step_args {
  int32_t batch, P, H;
  int32_t method;          /* ZOH, BILINEAR or DIRAC */
  int32_t conj_sym;
  int32_t reserved0;
  void *state;
  const void *x, *dt, *deltaA /* nullable */, *A, *B, *C, *D /* nullable */;
  void *out;
  int64_t state_bs, x_bs, dt_bs, deltaA_bs, out_bs;
} b200_s5_step_args;

int b200_s5_step(const b200_s5_step_args *args, void *stream);

/* ------------------------------------------------------------------------
 * S4 structured kernels (contiguous tensors).
 * Replace cauchy_mult_sym_fwd/bwd and vand_log_mult_sym_fwd/bwd
 * (csrc/s4/cauchy.cpp:20-102, csrc/s4/cauchy_cuda.cu:34-368).
 *   Cauchy: v, w (batch, n) complex64 (n = half size: one member of each
 *           conjugate pair; any n >= 1), z (seqlen) complex64,
 *           out/dout (batch, seqlen) complex64, dv, dw (batch, n) complex64.
 *   Vandermonde: v, x (batch, n) complex64 (x passed in the `w` field),
 *           out/dout (batch, seqlen) float32, dv, dx (batch, n) complex64
 *           (dx returned in the `dw` field).
 * The backward entry points reduce over the sequence in two passes: per-chunk
 * partial sums go to `scratch` (caller-allocated device memory of at least
 * b200_s4_bwd_scratch_bytes(batch, n, seqlen) bytes, 16-byte aligned; contents
 * on entry are ignored), then a second kernel folds them into dv / dw in a fixed
 * order, so results are deterministic.  dv / dw are overwritten.
 * ------------------------------------------------------------------------ */
typedef struct b200_s4_args {
  int32_t batch, n, seqlen, reserved0;
  const void *v, *z, *w;
  void *out;
  const void *dout;
  void *dv, *dw;
  void *scratch;
  int64_t scratch_bytes;
} b200_s4_args;

int64_t b200_s4_bwd_scratch_bytes(int32_t batch, int32_t n, int32_t seqlen);
int b200_cauchy_fwd(const b200_s4_args *args, void *stream);
int b200_cauchy_bwd(const b200_s4_args *args, void *stream);

/* Cauchy backward for callers that cannot provide scratch memory.  It has no
 * counterpart in lrnnx.  Same inputs, outputs and results as b200_cauchy_bwd, but
 * `scratch` / `scratch_bytes` of the argument block are ignored: the partial sums
 * go to a fixed B200_CAUCHY_STATIC_SCRATCH_BYTES area that is part of the library
 * image on every GPU that loads it.  The call performs no cudaMalloc / cudaFree
 * and uses no allocating library routine.
 *  - Limit: problems whose b200_s4_bwd_scratch_bytes(batch, n, seqlen) exceeds the
 *    area are rejected with B200_ERR_TOO_LARGE (nothing is launched).
 *  - The first call on each device looks up the area's device address (the device
 *    the call should run on must be current); make that first call before any
 *    stream capture begins.
 *  - All calls on a device share the one area, which keeps the previous call's
 *    contents (no part of it needs clearing: each call overwrites every slot it
 *    later reads).  Two calls that overlap in time on the same GPU, e.g. on
 *    different streams, race on it; serialise them. */
#define B200_CAUCHY_STATIC_SCRATCH_BYTES (4 * 1024 * 1024)
int b200_cauchy_bwd_static(const b200_s4_args *args, void *stream);
int b200_vand_fwd(const b200_s4_args *args, void *stream);
int b200_vand_bwd(const b200_s4_args *args, void *stream);

/* ------------------------------------------------------------------------
 * Depthwise causal convolution of a Mamba block (+ optional SiLU), its backward, and the
 * one-token update used in decoding.  Replace the nn.Conv1d(groups=d_inner, padding=width-1)
 * fallback of lrnnx/models/ltv/mamba.py:270-279 (forward), its autograd backward, and the
 * roll + dot of Mamba.step (lrnnx/models/ltv/mamba.py:394-409); lrnnx's own fast path for them
 * is the un-vendored causal_conv1d package (mamba.py:24-27).
 *   x, out, dout, dx : (batch, dim, seqlen) activations dtype, seqlen contiguous (16-byte accesses
 *                      where a row segment is 16-byte aligned, element accesses otherwise)
 *   weight (dim, width) and bias (dim, nullable) : activations dtype, dense; width 2..4
 *   out[b,d,t] = act(bias[d] + sum_k weight[d,k] * x[b,d,t-(width-1)+k]),  x = 0 before t = 0
 *   dweight (dim, width), dbias (dim) : float32 accumulators, zero-filled by the caller
 *   update: x, out (batch, dim) with strides x_bs/x_ds, out_bs/out_ds; state (batch, dim, width)
 *           activations dtype, innermost stride 1, shifted left by one and appended with x in place
 * ------------------------------------------------------------------------ */
typedef struct b200_conv1d_args {
  int32_t batch, dim, seqlen, width;
  int32_t dtype;              /* B200_F32 / F16 / BF16 */
  int32_t silu;               /* apply SiLU to the output */
  const void *x, *weight, *bias;
  void *out;
  void *state;                /* update only */
  const void *dout;           /* backward only */
  void *dx, *dweight, *dbias; /* backward only */
  int64_t x_bs, x_ds, out_bs, out_ds, state_bs, state_ds;
  int64_t dout_bs, dout_ds, dx_bs, dx_ds;
} b200_conv1d_args;

int b200_conv1d_fwd(const b200_conv1d_args *args, void *stream);
int b200_conv1d_bwd(const b200_conv1d_args *args, void *stream);
int b200_conv1d_update(const b200_conv1d_args *args, void *stream);

/* ------------------------------------------------------------------------
 * Fused residual add + RMSNorm, forward and backward.  Replaces rms_norm_fn / layer_norm_fn with
 * is_rms_norm (lrnnx/ops/triton/layer_norm.py:994-1094) as the LM blocks call it
 * (lrnnx/layers/block.py:77-87, lrnnx/architectures/language_model.py:374-384):
 *   z = x + residual (residual nullable);  y = z * rsqrt(mean(z^2) + eps) * weight
 *   x, y, dy, dx (rows, cols) activations dtype; residual, residual_out, dresidual, dresidual_in
 *   (rows, cols) in residual_dtype (the activations dtype, or float32 = residual_in_fp32);
 *   weight (cols) activations dtype; rstd (rows) float32; dweight (cols) float32, zero-filled.
 *   forward writes y, residual_out (= z, optional) and rstd (optional);
 *   backward reads dy, residual_out (z), rstd, weight and dresidual (gradient arriving at
 *   residual_out, nullable), writes dx and (optional) dresidual_in — both equal dz — and adds to dweight.
 * cols must be a multiple of 8 and at most 4096; every row 16-byte aligned.
 * ------------------------------------------------------------------------ */
typedef struct b200_rmsnorm_args {
  int64_t rows;
  int32_t cols;
  int32_t dtype, residual_dtype;
  float eps;
  const void *x, *residual, *weight;
  void *y, *residual_out, *rstd;
  const void *dy, *dresidual;
  void *dx, *dresidual_in, *dweight;
  int64_t x_rs, residual_rs, y_rs, residual_out_rs, dy_rs, dresidual_rs, dx_rs, dresidual_in_rs;
} b200_rmsnorm_args;

int b200_rmsnorm_fwd(const b200_rmsnorm_args *args, void *stream);
int b200_rmsnorm_bwd(const b200_rmsnorm_args *args, void *stream);

/* ------------------------------------------------------------------------
 * Complex projection on the tensor cores (tcgen05, 3xTF32: float32-class accuracy):
 *     out[b] (M x N) = W (M x K) * x[b] (K x N),  complex64.
 * Replaces the torch.einsum calls (cuBLAS cgemm) around the simplified scan in lrnnx's
 * SimplifiedScanFn / S5InnerFn (lrnnx/ops/simplified_scan.py:67,87,136,165,401,419,483-524):
 * Bu = B~ u, y = C~ x and the data gradients du = B~^H dBu, dx = C~^H dy.
 *   w_planes : float32 (4, M, K), K contiguous: Re(W) rounded to TF32 (low 13 mantissa bits
 *              zero), the remainder rounded to TF32, and the same two planes of Im(W)
 *   x        : complex64 (batch, K, N) dense;  out : complex64 (batch, M, N), N contiguous
 * M a multiple of 128, K of 32, N of 64; all pointers 16-byte aligned.
 * ------------------------------------------------------------------------ */
typedef struct b200_cgemm_args {
  int32_t batch, M, K, N;
  const void *w_planes, *x;
  void *out;
  int64_t x_bs, x_ks;        /* complex elements */
  int64_t out_bs, out_ms;    /* complex elements */
} b200_cgemm_args;

int b200_cgemm_wx(const b200_cgemm_args *args, void *stream);

/* Weight gradient of a projection on the tensor cores (same 3xTF32 arithmetic):
 *     out (M x N) += sum over b, l of g[b, m, l] * conj(u[b, n, l])
 * g (batch, M, L), u (batch, N, L), out (M, N): complex64, dense, L contiguous.  out must be
 * zero-filled by the caller (the contraction is cut over several thread blocks which add their
 * partial results with float32 reductions).  M and N multiples of 128, L of 16. */
typedef struct b200_cgemm_grad_args {
  int32_t batch, M, N, L;
  const void *g, *u;
  void *out;
} b200_cgemm_grad_args;

int b200_cgemm_grad(const b200_cgemm_grad_args *args, void *stream);

/* Builds the w_planes operand of b200_cgemm_wx from a complex64 matrix W (M, K) given by element
 * strides (so a transposed view is free), optionally conjugated (conj != 0): planes is float32
 * (4, M, K), written densely. */
typedef struct b200_cgemm_planes_args {
  int32_t M, K, conj, reserved0;
  const void *w;
  void *planes;
  int64_t w_rs, w_cs;        /* complex elements */
} b200_cgemm_planes_args;

int b200_cgemm_planes(const b200_cgemm_planes_args *args, void *stream);

/* ------------------------------------------------------------------------
 * Linear layer for the few tokens of one decoding step: out (M, N) = x (M, K) W^T (+ bias), with
 * W (N, K) the row-major weight of an nn.Linear, 16-bit operands, float32 accumulation.  Takes the
 * place of the library GEMMs behind F.linear in Mamba.step (lrnnx/models/ltv/mamba.py:355-487:
 * in_proj, x_proj, dt_proj, out_proj) and the LM head at decoding time, where each weight is
 * streamed once per generated token.  1 <= M <= 64; K a multiple of 64; rows of x and W start on
 * 16-byte boundaries (strides multiples of 8 elements); out rows may have any stride.
 * Deterministic (no atomics).
 * ------------------------------------------------------------------------ */
typedef struct b200_skinny_linear_args {
  int32_t M, N, K, dtype;          /* dtype: B200_BF16 or B200_F16 (x, weight, bias, out) */
  const void *x, *weight, *bias;   /* bias (N) nullable */
  void *out;
  int64_t x_rs, w_rs, out_rs;      /* row strides in elements */
} b200_skinny_linear_args;

int b200_skinny_linear(const b200_skinny_linear_args *args, void *stream);

/* ------------------------------------------------------------------------
 * Next-token cross-entropy over a wide vocabulary, read straight from the logits in their own
 * dtype (no float32 copy of the (rows, cols) logits).  lrnnx has no counterpart: its LM returns
 * logits (lrnnx/architectures/language_model.py:615-727) and its training benchmark sums them
 * (benchmarks/benchmark_training.py:33-34); this is the loss the LM harness trains with.
 *   forward : lse[r] = log sum_j exp(logits[r, j]);  loss[r] = lse[r] - logits[r, labels[r]],
 *             0 for rows whose label equals ignore_index
 *   backward: dlogits[r, j] = (exp(logits[r, j] - lse[r]) - [j == labels[r]]) * scale[0],
 *             0 for ignored rows;  scale is a float32 scalar in device memory
 *             (upstream gradient / number of counted rows)
 *   logits, dlogits (rows, cols) float32 / float16 / bfloat16, cols contiguous;
 *   labels int64 (rows); lse, loss float32 (rows).
 * ------------------------------------------------------------------------ */
typedef struct b200_xent_args {
  int64_t rows;
  int32_t cols, dtype;
  int64_t ignore_index;
  const void *logits, *labels, *scale;
  void *lse, *loss, *dlogits;
  int64_t logits_rs, dlogits_rs;
} b200_xent_args;

int b200_xent_fwd(const b200_xent_args *args, void *stream);
int b200_xent_bwd(const b200_xent_args *args, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* LRNNX_B200_H_ */
