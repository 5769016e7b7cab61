/*
 * ssm_b200 — C ABI of the B200 (sm_100a) backend for the five state-space operators
 * of the b-vitamins/ssm package.
 *
 * Every entry point takes a plain argument struct (raw device pointers, sizes, element
 * strides, dtype codes) plus a CUDA stream handle, enqueues its kernels on that stream and
 * returns without synchronising.  The library never allocates: outputs and scratch are
 * passed in by the caller.  Return value: 0 on success; a negative SSM_ERR_* code when an
 * argument is rejected (nothing was launched); a positive value is a cudaError_t from the
 * launch.  ssm_b200_last_error() returns a thread-local description of the last failure.
 *
 * The functions replace, one for one, the compiled operators that the upstream package
 * binds in src/ssm/ops/cuda/bindings.cpp:96-152 (the citation beside each declaration
 * names the host function there whose device work it takes over).  Layouts follow the
 * upstream Python specification src/ssm/ops/python/reference.py.
 */
#ifndef SSM_B200_H_
#define SSM_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SSM_B200_ABI_VERSION 3

/* element types of activation tensors.  SSM_F64 selects the double-precision variants of the five operators (forward and
 * backward; written for gradient checking as in upstream's tests/ops/test_backend_gradients.py:1172-1612, not for speed): with
 * io_dtype == SSM_F64 EVERY floating-point tensor of the call -- activations, A, B, C, D, biases, weights, states, gradients --
 * is double, whatever C type the argument struct gives its pointer; bc_dtype, par_dtype, res_dtype, resout_dtype and last_dtype
 * are ignored; d_state <= 256; the scan backward takes batch * dim * len * nstate doubles of scratch through fwd.checkpoints (no
 * forward checkpoints are needed); the chunk-scan history is double; the norm backward ACCUMULATES into dweight / dbias (the
 * caller zero-fills them) and needs no `partial`.  The decode-time conv update, the SSD entry points and the allocation-free norm
 * backward have no fp64 variant. */
enum { SSM_F32 = 0, SSM_BF16 = 1, SSM_F16 = 2, SSM_F64 = 3 };

enum {
  SSM_OK = 0,
  SSM_ERR_NULL = -1,        /* a required pointer is NULL */
  SSM_ERR_SHAPE = -2,       /* a size is negative/zero where it may not be, or sizes disagree */
  SSM_ERR_DTYPE = -3,       /* unknown dtype code */
  SSM_ERR_ALIGN = -4,       /* a pointer misses its natural alignment */
  SSM_ERR_UNSUPPORTED = -5, /* valid in the operator's contract but outside what is built */
  SSM_ERR_TOO_LARGE = -6,   /* exceeds a documented capacity */
  SSM_ERR_DEVICE = -7       /* device-side status word reported a bounded wait that ran out */
};

/* The stream is a cudaStream_t passed as an opaque pointer so that this header needs no CUDA include. */
typedef void* ssm_stream_t;

int ssm_b200_abi_version(void);
const char* ssm_b200_last_error(void);

/* ---------------------------------------------------------------------------------------
 * Selective scan (Mamba-1), forward.   Replaces selective_scan_cuda
 * (src/ssm/ops/cuda/selective_scan.cu:1034-1161; spec reference.py:87-194).
 *
 *   dl_t = softplus?(delta_t + dt_bias);  h_t = exp(dl_t*A) .* h_{t-1} + dl_t*B_t*u_t
 *   y_t  = <C_t, h_t> + D*u_t;            out_t = y_t * silu(z_t)
 *
 * u, delta, z, out: (batch, dim, len) with contiguous time axis and the batch / channel strides
 * row_sb / row_sd, element type io_dtype.  A: (dim, nstate)
 * fp32.  Bm / Cm are addressed as  base[b*sb + g*sg + n*sn + t*st]  (element strides, type
 * bc_dtype) with g = d / (dim / bc_groups); this one form covers the (D,N), (B,D,N) and
 * grouped time-varying (B,G,N,L) layouts of reference.py:22-56.  D, dt_bias: (dim) fp32
 * or NULL.  initial_state: (batch, dim, nstate) fp32 or NULL (zeros).  last_state: optional
 * output (batch, dim, nstate) of type last_dtype.  checkpoints: optional output
 * (batch, dim, ceil(len / ssm_scan_checkpoint_interval()), nstate) fp32 holding the state
 * before every interval; the backward pass needs it.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  int32_t batch, dim, len, nstate;
  int32_t io_dtype, bc_dtype, last_dtype, delta_softplus;
  const void* u;
  const void* delta;
  const void* z; /* nullable */
  const float* A;
  const void* Bm;
  const void* Cm;
  int32_t bc_groups, reserved0;
  int64_t b_sb, b_sg, b_sn, b_st;
  int64_t c_sb, c_sg, c_sn, c_st;
  const float* D;             /* nullable */
  const float* dt_bias;       /* nullable */
  const float* initial_state; /* nullable */
  void* out;
  void* last_state;   /* nullable */
  float* checkpoints; /* nullable */
  /* Element strides of the batch and channel axes of u, delta, z, out (and of dout, du, ddelta,
   * dz in the backward call); the time axis is contiguous.  Dense (B, D, L) is {dim*len, len};
   * a (D, B, L) buffer viewed as (B, D, L) is {len, batch*len}, which lets the projections
   * around the scan be plain 2-D GEMMs with no transposing copies. */
  int64_t row_sb, row_sd;
  /* Optional time-parallel execution for calls whose (batch x dim) rows alone cannot fill the GPU (e.g. batch 1): the sequence
   * is cut into split_segments pieces that are integrated in parallel and stitched by a short serial pass (the block-level
   * prefix over the (A, B u) recurrence).  split_scratch: 2 * batch * dim * split_segments * nstate floats.  NULL or
   * split_segments <= 1: one pass over the whole sequence.  ssm_scan_split_segments() suggests the count. */
  float* split_scratch;
  int32_t split_segments, reserved1;
} ssm_scan_fwd_args;

int ssm_scan_checkpoint_interval(void);
int ssm_scan_split_segments(int32_t batch, int32_t dim, int32_t len, int32_t nstate);
int ssm_selective_scan_fwd(const ssm_scan_fwd_args* args, ssm_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Selective scan, backward.   Replaces selective_scan_backward_cuda
 * (src/ssm/ops/cuda/selective_scan.cu:1696-1875) and, because grad_last_state is
 * handled on the device, the Python fall-back in src/ssm/ops/__init__.py:365-436.
 *
 * fwd holds the forward call's arguments (out/last_state unused; checkpoints required).
 * dout: (batch, dim, len) io_dtype.  dlast_state: (batch, dim, nstate) fp32 or NULL.
 * du, ddelta, dz: io_dtype (dz NULL iff fwd.z is NULL).  dA (dim, nstate), dD, ddt_bias
 * (dim): fp32, ACCUMULATED into (caller zero-fills); dD / ddt_bias may be NULL.
 * dB / dC: fp32 buffers addressed with db_* / dc_* strides exactly like Bm / Cm,
 * accumulated into (caller zero-fills).
 * ------------------------------------------------------------------------------------- */
typedef struct {
  ssm_scan_fwd_args fwd;
  const void* dout;
  const float* dlast_state; /* nullable */
  void* du;
  void* ddelta;
  void* dz; /* nullable */
  float* dA;
  float* dB;
  float* dC;
  int64_t db_sb, db_sg, db_sn, db_st;
  int64_t dc_sb, dc_sg, dc_sn, dc_st;
  float* dD;       /* nullable */
  float* ddt_bias; /* nullable */
  float* dinitial_state; /* nullable: (batch, dim, nstate) fp32, written: gradient of fwd.initial_state (additive extension) */
} ssm_scan_bwd_args;

int ssm_selective_scan_bwd(const ssm_scan_bwd_args* args, ssm_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Single-token state step (decode).   Replaces selective_state_step_cuda
 * (src/ssm/ops/cuda/state_step.cu:310-434; spec reference.py:197-309).
 *
 * state: (batch, dim, nstate) fp32, updated in place.  x, z, out: (batch, dim) io_dtype.
 * Parameters are per channel when param_heads == 0: dt (batch, dim), A (dim, nstate),
 * D / dt_bias (dim).  With param_heads = H > 0 (Mamba-2 layout, channel d belongs to head
 * d / (dim / H)) they are per head: dt (batch, H), A (H), D / dt_bias (H).  Bm / Cm:
 * base[b*sb + g*sg + n*sn], type bc_dtype, g = d / (dim / bc_groups), which covers (D,N),
 * (B,D,N) and grouped (B,G,N).
 * ------------------------------------------------------------------------------------- */
typedef struct {
  int32_t batch, dim, nstate, io_dtype;
  int32_t bc_dtype, bc_groups, dt_softplus, param_heads;
  float* state;
  const void* x;
  const void* dt;
  const void* z; /* nullable */
  const float* A;
  const void* Bm;
  const void* Cm;
  int64_t b_sb, b_sg, b_sn;
  int64_t c_sb, c_sg, c_sn;
  const float* D;       /* nullable */
  const float* dt_bias; /* nullable */
  void* out;
} ssm_step_args;

int ssm_selective_state_step(const ssm_step_args* args, ssm_stream_t stream);

/* Backward of the step (per-channel parameters only).  Replaces
 * selective_state_step_backward_cuda (src/ssm/ops/cuda/state_step.cu:436-693).
 * state is the state BEFORE the step.  dout (batch, dim) io_dtype; dnew_state
 * (batch, dim, nstate) fp32 or NULL.  dstate (batch, dim, nstate) fp32; dx, ddt, dz
 * io_dtype; dA, dD, ddt_bias, dB, dC fp32 accumulated into (caller zero-fills);
 * dB / dC use the Bm / Cm strides of fwd. */
typedef struct {
  ssm_step_args fwd;
  const void* dout;
  const float* dnew_state; /* nullable */
  float* dstate;
  void* dx;
  void* ddt;
  void* dz; /* nullable */
  float* dA;
  float* dB;
  float* dC;
  float* dD;       /* nullable */
  float* ddt_bias; /* nullable */
} ssm_step_bwd_args;

int ssm_selective_state_step_bwd(const ssm_step_bwd_args* args, ssm_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Element-wise chunked recurrence ("ssd_chunk_scan" upstream).   Replaces
 * ssd_chunk_scan_cuda (src/ssm/ops/cuda/ssd_chunk_scan.cu:637-860; spec reference.py:312-463).
 *
 * X, Y: (batch, len, heads, proj) io_dtype.  dt: (batch, len, heads) io_dtype.  Every
 * parameter p in {A, Bm, Cm, D, z, initial} is addressed  base[b*sb + t*st + h*sh + q*sq]
 * with zero strides for broadcast axes (A/D/initial fp32; Bm/Cm/z of type par_dtype).
 * seq_lens: (batch) int64 on the device or NULL; outputs beyond a row's length are zero.
 * final_state: optional output (batch, heads, proj) fp32 (additive; upstream returns none).
 * chunk_size splits the sequence into independently processed chunks (it has no numerical
 * effect beyond rounding).  scratch: fp32 workspace of ssm_chunk_scan_scratch_floats()
 * elements; when NULL the sequence is walked serially by one thread per (batch, head, proj).
 * ------------------------------------------------------------------------------------- */
typedef struct {
  const void* ptr;
  int64_t sb, st, sh, sq;
} ssm_bcast4;

typedef struct {
  int32_t batch, len, heads, proj;
  int32_t io_dtype, par_dtype, reserved0, typed_grads; /* typed_grads: backward only, see ssm_chunk_bwd_args */
  const void* X;
  const void* dt;
  ssm_bcast4 A, Bm, Cm, D, z, initial; /* D, z, initial: ptr may be NULL */
  const int64_t* seq_lens;             /* nullable */
  void* Y;
  float* final_state; /* nullable */
  float* scratch;     /* nullable */
  int32_t chunk_size, reserved2;
} ssm_chunk_args;

int64_t ssm_chunk_scan_scratch_floats(int32_t batch, int32_t len, int32_t heads, int32_t proj, int32_t chunk_size);
int ssm_chunk_scan_fwd(const ssm_chunk_args* args, ssm_stream_t stream);

/* Backward.  Replaces ssd_chunk_scan_backward_cuda (src/ssm/ops/cuda/ssd_chunk_scan.cu:341-635).
 * dY io_dtype.  dX (io_dtype), ddt fp32 (batch, len, heads), and fp32 gradient buffers
 * dA/dB/dC/dD/dz/dinitial addressed with the strides given here (broadcast axes = stride 0),
 * accumulated into (caller zero-fills).  history: scratch (batch, len, heads, proj) fp32.
 * fwd.typed_grads, bits 0 / 1 / 2: dB / dC / dz is instead a buffer of par_dtype elements with no broadcast axis (every
 * (b, t, h, q) a distinct element) that the call WRITES, every element of it, zeros beyond a row's length included: no zero-fill
 * by the caller, no fp32 copy to convert afterwards. */
typedef struct {
  ssm_chunk_args fwd;
  const void* dY;
  void* dX;
  float* ddt;
  ssm_bcast4 dA, dB, dC, dD, dz, dinitial; /* ptr as float*; NULL to skip where fwd's is NULL */
  float* history;
  float* scratch; /* nullable: ssm_chunk_scan_bwd_scratch_floats() floats; with it the chunks run in parallel, without it one thread
                     per (batch, head, proj) walks the whole sequence */
} ssm_chunk_bwd_args;

int64_t ssm_chunk_scan_bwd_scratch_floats(int32_t batch, int32_t len, int32_t heads, int32_t proj, int32_t chunk_size);
int ssm_chunk_scan_bwd(const ssm_chunk_bwd_args* args, ssm_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Depthwise causal conv1d.   Replaces dw_causal_conv_cuda / dw_causal_conv_backward_cuda
 * (src/ssm/ops/cuda/dw_causal_conv.cu:771-857, 859-965; spec reference.py:466-537).
 *
 * x, y: channels_first ? (batch, channels, len) : (batch, len, channels), io_dtype.
 * weight: (channels, width) fp32, tap j multiplies x[t - (width-1) + j].  bias fp32/NULL.
 * 1 <= width <= 8.  Optional halo: (batch, channels, width-1) fp32 inputs that precede
 * t = 0 (sequence-sharded prefill; NULL means zeros, the upstream behaviour).
 * Backward: dx io_dtype; dweight (channels, width), dbias (channels) fp32 accumulated into.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  int32_t batch, channels, len, width;
  int32_t io_dtype, channels_first, silu, reserved0;
  const void* x;
  const float* weight;
  const float* bias; /* nullable */
  const float* halo; /* nullable */
  void* y;
  /* channels_first only: element strides of the batch and channel axes of x, y (and dy, dx);
   * dense is {channels*len, len}.  Ignored for the channels-last layout. */
  int64_t row_sb, row_sc;
} ssm_conv_args;

int ssm_dw_causal_conv_fwd(const ssm_conv_args* args, ssm_stream_t stream);

typedef struct {
  ssm_conv_args fwd;
  const void* dy;
  void* dx;
  float* dweight;
  float* dbias; /* nullable */
} ssm_conv_bwd_args;

int ssm_dw_causal_conv_bwd(const ssm_conv_bwd_args* args, ssm_stream_t stream);

/* Decode-time form of the same convolution: push one token into the rolling window and take
 * the dot product.  Upstream does this with torch.roll in Python
 * (src/ssm/modules/mamba1.py:345-353).  conv_state: (batch, channels, width) fp32, shifted
 * left by one and x appended, in place.  x, out: (batch, channels) io_dtype;
 * out = silu?(bias + <conv_state, weight>). */
typedef struct {
  int32_t batch, channels, width, io_dtype;
  int32_t silu, reserved0;
  float* conv_state;
  const void* x;
  const float* weight;
  const float* bias; /* nullable */
  void* out;
} ssm_conv_update_args;

int ssm_dw_causal_conv_update(const ssm_conv_update_args* args, ssm_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Residual add fused with LayerNorm / RMSNorm.   Replaces fused_layer_norm_cuda /
 * fused_layer_norm_backward_cuda (src/ssm/ops/cuda/layer_norm.cu:372-496, 498-676; spec
 * reference.py:540-609).
 *
 * x, y: (rows, hidden) io_dtype.  residual: res_dtype or NULL.  weight, bias fp32.
 * prenorm: y = norm(x + residual)*w + b, else y = norm(x)*w + b + residual.
 * All arithmetic is fp32 (upstream's residual_in_fp32 only matters for fp64 inputs, which
 * are not built).  hidden <= 16384 (16-bit) / 8192 (fp32).  residual_out: optional
 * (rows, hidden) of resout_dtype receiving x + residual (additive extension).
 * Backward: dx io_dtype, dresidual res_dtype (NULL iff residual NULL); dweight, dbias fp32
 * (hidden) written (not accumulated); partial: scratch fp32 of
 * ssm_norm_bwd_scratch_floats(rows, hidden) floats.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  int64_t rows;
  int32_t hidden, io_dtype, res_dtype, resout_dtype;
  int32_t is_rms, prenorm, reserved0, reserved2;
  float eps, reserved1;
  const void* x;
  const void* residual; /* nullable */
  const float* weight;
  const float* bias; /* nullable */
  void* y;
  void* residual_out; /* nullable */
} ssm_norm_args;

int ssm_fused_add_norm_fwd(const ssm_norm_args* args, ssm_stream_t stream);

typedef struct {
  ssm_norm_args fwd;
  const void* dy;
  void* dx;
  void* dresidual; /* nullable */
  float* dweight;
  float* dbias; /* nullable */
  float* partial;
  const void* dresidual_out; /* nullable: gradient arriving through residual_out, (rows, hidden) of fwd.resout_dtype; added to dx and dresidual */
} ssm_norm_bwd_args;

int64_t ssm_norm_bwd_scratch_floats(int64_t rows, int32_t hidden);
int ssm_fused_add_norm_bwd(const ssm_norm_bwd_args* args, ssm_stream_t stream);

/* Backward of the fused add + norm for callers that are not allowed to allocate device memory
 * (it has no counterpart in the upstream package).  Code that runs inside someone else's memory
 * plan -- an inference server that hands out one fixed arena at start-up, a plugin that must not
 * touch the CUDA allocator of its host process, a real-time loop that cannot risk the implicit
 * synchronisation of cudaMalloc / cudaFree -- cannot provide the `partial` scratch that
 * ssm_fused_add_norm_bwd needs.  This entry point computes the same result but keeps that
 * scratch in a fixed array inside the library's own device image: `args->partial` is ignored
 * and neither this call nor anything it launches allocates or frees memory.
 *
 * Limits and rules:
 *  - hidden <= 8192 (larger rows are rejected with SSM_ERR_TOO_LARGE); the array takes
 *    9.25 MiB on every GPU that loads the library, for the life of the process;
 *  - the first call on each device looks up the array's device address (with that device
 *    current) and remembers it; make that first call outside any stream capture.  The tensors
 *    must live on the current device (checked: SSM_ERR_DEVICE otherwise);
 *  - all calls on a device share the one array.  Nothing in it has to start at zero (every
 *    launch overwrites the part it later reads), but two calls whose kernels overlap on
 *    the GPU (different streams, no ordering) race on it: serialise them on one stream or
 *    with events;
 *  - weight / bias gradients are summed over at most 148 partial rows instead of up to 592, so
 *    they can differ from ssm_fused_add_norm_bwd in the last bits; dx / dresidual are identical. */
int ssm_fused_add_norm_bwd_noalloc(const ssm_norm_bwd_args* args, ssm_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * State-space-dual scan with a d_state axis (Mamba-2), forward, on the tcgen05 tensor cores.
 * Upstream has no operator of this shape (its ssd_chunk_scan has no state axis,
 * src/ssm/ops/python/reference.py:312-463); the semantics are those of its selective_scan
 * (reference.py:87-194) on channel h*P+p with delta[b,h*P+p,t] = dt[b,t,h], A[h*P+p,:] = A[h]
 * and B, C shared per group, the final state being selective_scan's last state kept in fp32.
 *
 * X, z, Y: (batch, len, heads, headdim) io_dtype.  dt: (batch, len, heads) io_dtype.  A: (heads)
 * fp32.  Bm, Cm: (batch, len, groups, nstate) io_dtype.  D: (heads) or, with d_has_p,
 * (heads, headdim) fp32, nullable.  dt_bias: (heads) fp32, nullable.  initial_states /
 * final_states: (batch, heads, headdim, nstate) fp32, nullable.  Built for headdim 64,
 * nstate 128, chunk_size 256, bf16 / fp16 (ssm_ssd_supported()).  Scratch, in this order, is
 * carved by the caller from one buffer of ssm_ssd_scratch_bytes() bytes:
 *   ws_dt, ws_cum : (batch, heads, nchunks * 256) fp32 each; per chunk ws_cum[i] = log2(e) * sum_{k<=i} delta_k A
 *                   (running decay exponent, base 2) and ws_dt[i] = ws_cum[i] - log2(delta_i)
 *   ws_state      : (batch, heads, headdim, nstate) fp32 — the final state reached from the given (or zero)
 *                   initial state, kept for a later phase-2 call on the same scratch — followed by (batch, heads)
 *                   fp32, the total log-decay sum(delta A) of the call; the two together (ssm_ssd_shard_summary_floats()
 *                   floats) are what a sequence shard sends to the other ranks; then, from the next 256-byte boundary,
 *                   (batch, heads, nchunks) fp32 decay exponents from the start of the call to each chunk.  The whole
 *                   region takes ssm_ssd_state_scratch_bytes() bytes
 *   ws_state_in   : (batch, nchunks, heads, headdim * nstate) in io_dtype — the state before every chunk, in
 *                   the operand order of the scan kernel
 * status: optional device int, set non-zero when a bounded device-side wait ran out.
 * phase: 0 runs everything.  1 stops after the chunk states (it fills the scratch and
 * final_states from the given, normally absent, initial_states and writes no Y); 2 adds the
 * given initial_states on top of what phase 1 left in the scratch (by linearity), writes
 * the corrected final_states and produces Y.  A sequence shard uses 1, exchanges final
 * states with its neighbours, then 2.
 * dt_mode: 0 = dt is (batch, len, heads) in io_dtype and goes through dt_bias / dt_softplus.  1 = dt is fp32 and holds
 * the step sizes as they are used (dt_bias and dt_softplus are ignored).  3 = as 1, and the step size enters the
 * decay exp(dt A) only: the inputs are added with unit weight, S_t = exp(dt_t A) S_{t-1} + x_t B_t^T.  Modes 1 and 3
 * are what the backward pass uses to run the adjoint recurrence through the same kernels.  + 4 (to any mode): the caller
 * promises that heads 2 i and 2 i + 1 have equal step sizes and decay; the decay mask is then formed once per pair.
 * row_dots: (batch, len, heads) fp32, zero-filled by the caller.  When given, z is not a gate: Y is written ungated and
 * row_dots[b, t, h] receives sum_p y[p] z[p], with y taken before the D x term and before rounding to io_dtype (the
 * backward pass forms dy . y and d(dt x) . x this way).
 * row_scale: (batch, len, heads) fp32 positive weights: output row t of head h is multiplied by row_scale[b, t, h],
 * applied to the decay mask before it is rounded to the operand dtype (so a pass weighted this way rounds the same
 * masked tile as the forward pass, whose mask carries dt of the source step).
 * ws_state_in_f32: optional (batch, nchunks, heads, headdim * nstate) fp32: ws_state_in before rounding, same element order.
 * bc_width: stored width of the rows of Bm and Cm.  0 or nstate: (batch, len, groups, nstate).  64: (batch, len, groups, 64),
 * read as nstate-wide rows whose upper part is zero (the tensor-map copies fill what lies outside the tensor with
 * zeros) -- how the backward pass feeds x and dy in the places of B and C.
 * x_heads: 0, or the number of distinct input heads: X is then (batch, len, x_heads, headdim) and head h reads input head
 * h % x_heads (heads % x_heads == 0) -- how the backward pass feeds the two halves of a single group's B (or C) row to every
 * head without writing them out per head.  dt, z, Y and the states keep `heads` heads.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  int32_t batch, len, heads, headdim;
  int32_t nstate, groups, chunk_size, io_dtype;
  int32_t dt_softplus, d_has_p, phase, dt_mode;
  const void* X;
  const void* dt;
  const float* A;
  const void* Bm;
  const void* Cm;
  const float* D;              /* nullable */
  const void* z;               /* nullable */
  const float* dt_bias;        /* nullable */
  const float* initial_states; /* nullable */
  void* Y;
  float* final_states; /* nullable */
  float* ws_dt;
  float* ws_cum;
  float* ws_state;
  void* ws_state_in;
  int32_t* status; /* nullable */
  float* row_dots; /* nullable */
  const float* row_scale; /* nullable */
  int32_t bc_width;       /* 0 (= nstate) or 64 */
  int32_t x_heads;        /* 0 (= heads) or a divisor of heads */
  float* ws_state_in_f32; /* nullable */
} ssm_ssd_args;

int ssm_ssd_supported(int32_t headdim, int32_t nstate, int32_t chunk_size, int32_t io_dtype);

/* Self-test of the bounded device-side waits (no counterpart upstream).  Launches one warp that waits on a barrier nothing
 * arms, with a limit of `probes` probes of about a microsecond each (1 .. 100000); when the limit runs out the kernel
 * writes 3 to *status (device int) and returns normally -- the error path of ssm_ssd_fwd's kernels, without a fault. */
int ssm_ssd_wait_selftest(int32_t* status, int32_t probes, ssm_stream_t stream);
int64_t ssm_ssd_scratch_bytes(int32_t batch, int32_t len, int32_t heads);
int64_t ssm_ssd_state_scratch_bytes(int32_t batch, int32_t len, int32_t heads);
int ssm_ssd_fwd(const ssm_ssd_args* args, ssm_stream_t stream);

/* Sequence shards (no reference counterpart: the reference is single-device).  After phase 1 every rank all-gathers its
 * summary (ws_state: final state from a zero start, then total log-decay; ssm_ssd_shard_summary_floats() floats) into
 * `gathered` (world x that many floats).  ssm_ssd_fold_shards writes the incoming state (batch, heads, headdim, nstate)
 * fp32 of shard `rank`:  sum_{q<rank} exp(sum_{q<m<rank} logP_m) S_q  (+ the decayed `initial_states`, nullable),
 * which is the initial_states of the phase-2 call. */
int64_t ssm_ssd_shard_summary_floats(int32_t batch, int32_t heads);
int ssm_ssd_fold_shards(const float* gathered, int32_t world, int32_t rank, int32_t batch, int32_t heads, const float* initial_states,
                        float* incoming, ssm_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Backward of the state-space-dual scan in the dual form (no counterpart upstream, whose Mamba-2 scan has no d_state
 * axis).  Its contractions are four more runs of ssm_ssd_fwd (dt_mode 1 / 3, row_dots, row_scale, bc_width above) on
 * transformed operands; the entry points below are the bandwidth passes around them.  `len` is the sequence length
 * rounded up to whole chunks (the length of the work tensors dy, dy_rev, y_plain, dx_rev), `len_valid` the length
 * of the caller's tensors (gY, z, X, dX, dz); work rows beyond len_valid are written as zeros.
 *   ssm_ssd_bwd_gate    dy = gY * silu(z) (gY when z is NULL), in time order and time-reversed (dy_rev)
 *   ssm_ssd_bwd_finish  dz = gY (y_plain + D x) silu'(z);  dX = reversed(dx_rev) + D dy;  dD (heads) or (heads, headdim)
 *                       += sum dy x (zero-filled by the caller; NULL when D is NULL)
 *   ssm_time_flip       dst[b, len - 1 - t] = src[b, t] for rows of row_bytes bytes (a multiple of 16); src has len_valid rows
 *   ssm_ssd_bwd_group_sum  out[b, t, g, :] = sum over the heads h of group g of weight[b, t, h] * y[b, ts, h, :]
 *                       (ts = len - 1 - t when reversed, else t; weight nullable; y (batch, len, heads, nstate);
 *                       out (batch, len_out, groups, nstate) in out_dtype = io_dtype or SSM_F32)
 *   ssm_ssd_bwd_spread  dst[r, h, :] = src[r, h / (heads / groups), :] for `rows` rows r: (rows, groups, row_bytes) ->
 *                       (rows, heads, row_bytes), the row of a B / C group handed to each of its heads
 *   ssm_ssd_state_dot   out[b, c, h] = <fwd_states[b, c, h, :], adj_states[b, nchunks - c, h, :]> for c >= 1, 0 for c = 0;
 *                       both (batch, nchunks, heads, elems) in io_dtype or SSM_F32 (ws_state_in / ws_state_in_f32 of two
 *                       ssm_ssd_fwd runs)
 * --------------------------------------------------------------------------------------- */
typedef struct {
  int32_t batch, len, len_valid, heads;
  int32_t headdim, io_dtype, d_has_p, reserved0;
  const void* gY;      /* (batch, len_valid, heads, headdim); nullable in finish when z is NULL */
  const void* z;       /* nullable */
  const void* X;       /* finish */
  const void* y_plain; /* finish, with z: output of the forward pass without skip and gate, (batch, len, ...) */
  const void* dx_rev;  /* finish: output of the adjoint pass, time-reversed, (batch, len, ...) */
  const float* D;      /* nullable */
  void* dy;            /* gate: out; finish: in */
  void* dy_rev;        /* gate: out */
  void* dX;            /* finish: out */
  void* dz;            /* finish: out, with z */
  float* dD;           /* finish: accumulated, nullable */
} ssm_ssd_bwd_args;

int ssm_ssd_bwd_gate(const ssm_ssd_bwd_args* args, ssm_stream_t stream);
int ssm_ssd_bwd_finish(const ssm_ssd_bwd_args* args, ssm_stream_t stream);
int ssm_time_flip(const void* src, void* dst, int32_t batch, int32_t len, int32_t len_valid, int64_t row_bytes, ssm_stream_t stream);
int ssm_ssd_bwd_group_sum(const void* y, const float* weight, void* out, int32_t batch, int32_t len, int32_t len_out, int32_t heads, int32_t groups,
                          int32_t nstate, int32_t reversed, int32_t io_dtype, int32_t out_dtype, ssm_stream_t stream);
int ssm_ssd_bwd_spread(const void* src, void* dst, int64_t rows, int32_t heads, int32_t groups, int64_t row_bytes, ssm_stream_t stream);
int ssm_ssd_state_dot(const void* fwd_states, const void* adj_states, float* out, int32_t batch, int32_t nchunks, int32_t heads, int32_t elems,
                      int32_t io_dtype, ssm_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* SSM_B200_H_ */
