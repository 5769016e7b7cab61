// Double-precision variants of the five operators, forward and backward.
//
// They exist for gradient checking (upstream runs torch.autograd.gradcheck on its CUDA operators in float64,
// tests/ops/test_backend_gradients.py:1172-1612), not for speed: one thread per independent row walks its sequence with
// the arithmetic of the reference restated in double, parameter gradients are accumulated with double atomics.  They
// are reached through the ordinary entry points when io_dtype == SSM_F64; then EVERY floating-point tensor of the call
// -- activations, A, B, C, D, biases, weights, states, gradients, scratch -- is double, whatever C type the argument
// struct gives its pointer, and bc_dtype / par_dtype / res_dtype / last_dtype are ignored.
#include "common.cuh"

namespace ssmb {
namespace f64 {

constexpr int kThreads = 128;
constexpr int kMaxState = 256;

__device__ __forceinline__ double softplus_d(double x) { return x > 20.0 ? x : log1p(exp(x)); }
__device__ __forceinline__ double sigmoid_d(double x) { return 1.0 / (1.0 + exp(-x)); }
__device__ __forceinline__ double softplus_grad_d(double x) { return x > 20.0 ? 1.0 : sigmoid_d(x); }
__device__ __forceinline__ double silu_d(double x) { return x * sigmoid_d(x); }
__device__ __forceinline__ double silu_grad_d(double x) {
  const double s = sigmoid_d(x);
  return s * (1.0 + x * (1.0 - s));
}
template <typename P>
__device__ __forceinline__ const double* cd(P p) { return reinterpret_cast<const double*>(p); }
template <typename P>
__device__ __forceinline__ double* md(P p) { return reinterpret_cast<double*>(const_cast<void*>(reinterpret_cast<const void*>(p))); }

// ---------------------------------------------------------------------------------------------
// selective scan: thread = (batch, channel)
// ---------------------------------------------------------------------------------------------
// WITH_STATES: also write the state after every step to `states` (batch, dim, len, nstate), the backward pass's input
template <bool WITH_STATES>
__global__ void __launch_bounds__(kThreads) scan_fwd_kernel(const ssm_scan_fwd_args a, double* states, bool write_out) {
  const int64_t row = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (row >= (int64_t)a.batch * a.dim) return;
  const int b = (int)(row / a.dim), d = (int)(row % a.dim);
  const int N = a.nstate, L = a.len;
  const int g = d / (a.dim / a.bc_groups);
  const double* u = cd(a.u) + (int64_t)b * a.row_sb + (int64_t)d * a.row_sd;
  const double* dl = cd(a.delta) + (int64_t)b * a.row_sb + (int64_t)d * a.row_sd;
  const double* z = a.z ? cd(a.z) + (int64_t)b * a.row_sb + (int64_t)d * a.row_sd : nullptr;
  double* out = md(a.out) + (int64_t)b * a.row_sb + (int64_t)d * a.row_sd;
  const double* A = cd(a.A) + (int64_t)d * N;
  const double* Bm = cd(a.Bm) + (int64_t)b * a.b_sb + (int64_t)g * a.b_sg;
  const double* Cm = cd(a.Cm) + (int64_t)b * a.c_sb + (int64_t)g * a.c_sg;
  const double Dv = a.D ? cd(a.D)[d] : 0.0, bias = a.dt_bias ? cd(a.dt_bias)[d] : 0.0;
  double h[kMaxState];
  for (int n = 0; n < N; ++n) h[n] = a.initial_state ? cd(a.initial_state)[row * N + n] : 0.0;
  for (int t = 0; t < L; ++t) {
    double dt = dl[t] + bias;
    if (a.delta_softplus) dt = softplus_d(dt);
    const double ut = u[t];
    double y = 0.0;
    for (int n = 0; n < N; ++n) {
      h[n] = exp(dt * A[n]) * h[n] + dt * Bm[(int64_t)n * a.b_sn + (int64_t)t * a.b_st] * ut;
      y += Cm[(int64_t)n * a.c_sn + (int64_t)t * a.c_st] * h[n];
      if (WITH_STATES) states[(row * L + t) * N + n] = h[n];
    }
    y += Dv * ut;
    if (z) y *= silu_d(z[t]);
    if (write_out) out[t] = y;
  }
  if (write_out && a.last_state)
    for (int n = 0; n < N; ++n) md(a.last_state)[row * N + n] = h[n];
}

__global__ void __launch_bounds__(kThreads) scan_bwd_kernel(const ssm_scan_bwd_args g, const double* states) {
  const ssm_scan_fwd_args& a = g.fwd;
  const int64_t row = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (row >= (int64_t)a.batch * a.dim) return;
  const int b = (int)(row / a.dim), d = (int)(row % a.dim);
  const int N = a.nstate, L = a.len;
  const int grp = d / (a.dim / a.bc_groups);
  const int64_t ro = (int64_t)b * a.row_sb + (int64_t)d * a.row_sd;
  const double *u = cd(a.u) + ro, *dl = cd(a.delta) + ro, *z = a.z ? cd(a.z) + ro : nullptr, *dout = cd(g.dout) + ro;
  double *du = md(g.du) + ro, *ddl = md(g.ddelta) + ro, *dz = g.dz ? md(g.dz) + ro : nullptr;
  const double* A = cd(a.A) + (int64_t)d * N;
  const double* Bm = cd(a.Bm) + (int64_t)b * a.b_sb + (int64_t)grp * a.b_sg;
  const double* Cm = cd(a.Cm) + (int64_t)b * a.c_sb + (int64_t)grp * a.c_sg;
  double* dB = md(g.dB) + (int64_t)b * g.db_sb + (int64_t)grp * g.db_sg;
  double* dC = md(g.dC) + (int64_t)b * g.dc_sb + (int64_t)grp * g.dc_sg;
  const double Dv = a.D ? cd(a.D)[d] : 0.0, bias = a.dt_bias ? cd(a.dt_bias)[d] : 0.0;
  double G[kMaxState], dAacc[kMaxState];
  for (int n = 0; n < N; ++n) G[n] = g.dlast_state ? cd(g.dlast_state)[row * N + n] : 0.0, dAacc[n] = 0.0;
  double dDacc = 0.0, dBiasAcc = 0.0;
  for (int t = L - 1; t >= 0; --t) {
    const double pre = dl[t] + bias;
    const double dt = a.delta_softplus ? softplus_d(pre) : pre;
    const double ut = u[t];
    const double* hc = states + (row * L + t) * N;
    double ypre = Dv * ut;
    for (int n = 0; n < N; ++n) ypre += Cm[(int64_t)n * a.c_sn + (int64_t)t * a.c_st] * hc[n];
    double dy = dout[t];
    if (z) {
      dz[t] = dout[t] * ypre * silu_grad_d(z[t]);
      dy = dout[t] * silu_d(z[t]);
    }
    dDacc += dy * ut;
    double s1 = 0.0, s2 = 0.0;
    for (int n = 0; n < N; ++n) {
      const double hp = t > 0 ? hc[n - N] : (a.initial_state ? cd(a.initial_state)[row * N + n] : 0.0);
      const double Bn = Bm[(int64_t)n * a.b_sn + (int64_t)t * a.b_st], Cn = Cm[(int64_t)n * a.c_sn + (int64_t)t * a.c_st];
      const double Gn = Cn * dy + G[n];
      const double da = exp(dt * A[n]);
      atomicAdd(dC + (int64_t)n * g.dc_sn + (int64_t)t * g.dc_st, dy * hc[n]);
      atomicAdd(dB + (int64_t)n * g.db_sn + (int64_t)t * g.db_st, Gn * dt * ut);
      s1 += Gn * Bn;
      const double gha = Gn * hp * da;
      s2 += gha * A[n];
      dAacc[n] += gha * dt;
      G[n] = da * Gn;
    }
    du[t] = s1 * dt + Dv * dy;
    double dd = s1 * ut + s2;
    if (a.delta_softplus) dd *= softplus_grad_d(pre);
    ddl[t] = dd;
    dBiasAcc += dd;
  }
  for (int n = 0; n < N; ++n) {
    if (g.dinitial_state) md(g.dinitial_state)[row * N + n] = G[n];
    atomicAdd(md(g.dA) + (int64_t)d * N + n, dAacc[n]);
  }
  if (g.dD) atomicAdd(md(g.dD) + d, dDacc);
  if (g.ddt_bias) atomicAdd(md(g.ddt_bias) + d, dBiasAcc);
}

// ---------------------------------------------------------------------------------------------
// single-token state step: thread = (batch, channel)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) step_kernel(const ssm_step_bwd_args g, bool backward) {
  const ssm_step_args& a = g.fwd;
  const int64_t row = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (row >= (int64_t)a.batch * a.dim) return;
  const int b = (int)(row / a.dim), d = (int)(row % a.dim);
  const int N = a.nstate;
  const int H = a.param_heads;
  const int ph = H > 0 ? d / (a.dim / H) : d;  // index of dt / A / D / dt_bias
  const double x = cd(a.x)[row];
  double pre = H > 0 ? cd(a.dt)[(int64_t)b * H + ph] : cd(a.dt)[row];
  if (a.dt_bias) pre += cd(a.dt_bias)[ph];
  const double dt = a.dt_softplus ? softplus_d(pre) : pre;
  const double zv = a.z ? cd(a.z)[row] : 0.0;
  const int grp = d / (a.dim / a.bc_groups);
  const double* Bm = cd(a.Bm) + (int64_t)b * a.b_sb + (int64_t)grp * a.b_sg;
  const double* Cm = cd(a.Cm) + (int64_t)b * a.c_sb + (int64_t)grp * a.c_sg;
  const double Dv = a.D ? cd(a.D)[ph] : 0.0;
  double* state = md(a.state) + row * N;
  if (!backward) {
    double y = 0.0;
    for (int n = 0; n < N; ++n) {
      const double An = H > 0 ? cd(a.A)[ph] : cd(a.A)[(int64_t)d * N + n];
      const double nw = exp(dt * An) * state[n] + dt * x * Bm[(int64_t)n * a.b_sn];
      state[n] = nw;
      y += Cm[(int64_t)n * a.c_sn] * nw;
    }
    y += Dv * x;
    if (a.z) y *= silu_d(zv);
    md(a.out)[row] = y;
    return;
  }
  const double dout = cd(g.dout)[row];
  const double dy = a.z ? dout * silu_d(zv) : dout;
  double* dBp = md(g.dB) + (int64_t)b * a.b_sb + (int64_t)grp * a.b_sg;
  double* dCp = md(g.dC) + (int64_t)b * a.c_sb + (int64_t)grp * a.c_sg;
  double y = 0.0, sum_gb = 0.0, sum_da = 0.0;
  for (int n = 0; n < N; ++n) {
    const double An = cd(a.A)[(int64_t)d * N + n];
    const double Bn = Bm[(int64_t)n * a.b_sn], Cn = Cm[(int64_t)n * a.c_sn];
    const double s = state[n];
    const double da = exp(dt * An);
    const double nw = da * s + dt * x * Bn;
    y += Cn * nw;
    const double G = Cn * dy + (g.dnew_state ? cd(g.dnew_state)[row * N + n] : 0.0);
    md(g.dstate)[row * N + n] = G * da;
    atomicAdd(dCp + (int64_t)n * a.c_sn, dy * nw);
    atomicAdd(dBp + (int64_t)n * a.b_sn, G * dt * x);
    atomicAdd(md(g.dA) + (int64_t)d * N + n, G * s * da * dt);
    sum_gb += G * Bn;
    sum_da += G * s * da * An;
  }
  const double yfull = Dv * x + y;
  if (g.dz) md(g.dz)[row] = dout * yfull * silu_grad_d(zv);
  md(g.dx)[row] = dy * Dv + sum_gb * dt;
  const double ddl = sum_gb * x + sum_da;
  const double dpre = a.dt_softplus ? ddl * softplus_grad_d(pre) : ddl;
  md(g.ddt)[row] = dpre;
  if (g.dD) atomicAdd(md(g.dD) + d, dy * x);
  if (g.ddt_bias) atomicAdd(md(g.ddt_bias) + d, dpre);
}

// ---------------------------------------------------------------------------------------------
// element-wise chunked recurrence: thread = (batch, head, proj); the chunk size has no numerical effect
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ double bc4(const ssm_bcast4& p, int b, int t, int h, int q) {
  return cd(p.ptr)[(int64_t)b * p.sb + (int64_t)t * p.st + (int64_t)h * p.sh + (int64_t)q * p.sq];
}
__device__ __forceinline__ double* bc4p(const ssm_bcast4& p, int b, int t, int h, int q) {
  return md(p.ptr) + (int64_t)b * p.sb + (int64_t)t * p.st + (int64_t)h * p.sh + (int64_t)q * p.sq;
}

__global__ void __launch_bounds__(kThreads) chunk_kernel(const ssm_chunk_bwd_args g, bool backward) {
  const ssm_chunk_args& a = g.fwd;
  const int HP = a.heads * a.proj;
  const int64_t id = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (id >= (int64_t)a.batch * HP) return;
  const int b = (int)(id / HP), hp = (int)(id % HP), h = hp / a.proj, q = hp % a.proj;
  int valid = a.len;
  if (a.seq_lens) {
    const int64_t v = a.seq_lens[b];
    valid = (int)(v < 0 ? 0 : (v > a.len ? a.len : v));
  }
  const double Av = bc4(a.A, 0, 0, h, q);
  const double Dv = a.D.ptr ? bc4(a.D, 0, 0, h, q) : 0.0;
  const double* X = cd(a.X) + (int64_t)b * a.len * HP + hp;
  const double* dt = cd(a.dt) + (int64_t)b * a.len * a.heads + h;
  const double s0 = a.initial.ptr ? bc4(a.initial, b, 0, h, q) : 0.0;
  if (!backward) {
    double* Y = md(a.Y) + (int64_t)b * a.len * HP + hp;
    double s = s0;
    for (int t = 0; t < valid; ++t) {
      const double d = dt[(int64_t)t * a.heads], x = X[(int64_t)t * HP];
      s = exp(d * Av) * s + d * bc4(a.Bm, b, t, h, q) * x;
      double y = Dv * x + s * bc4(a.Cm, b, t, h, q);
      if (a.z.ptr) y *= silu_d(bc4(a.z, b, t, h, q));
      Y[(int64_t)t * HP] = y;
    }
    for (int t = valid; t < a.len; ++t) Y[(int64_t)t * HP] = 0.0;
    if (a.final_state) md(a.final_state)[(int64_t)b * HP + hp] = s;
    return;
  }
  double* hist = md(g.history) + (int64_t)b * a.len * HP + hp;
  double* dX = md(g.dX) + (int64_t)b * a.len * HP + hp;
  const double* dY = cd(g.dY) + (int64_t)b * a.len * HP + hp;
  {
    double s = s0;
    for (int t = 0; t < valid; ++t) {
      const double d = dt[(int64_t)t * a.heads];
      s = exp(d * Av) * s + d * bc4(a.Bm, b, t, h, q) * X[(int64_t)t * HP];
      hist[(int64_t)t * HP] = s;
    }
  }
  for (int t = valid; t < a.len; ++t) dX[(int64_t)t * HP] = 0.0;
  double carry = 0.0, dA_acc = 0.0, dD_acc = 0.0;
  for (int t = valid - 1; t >= 0; --t) {
    const double d = dt[(int64_t)t * a.heads], x = X[(int64_t)t * HP];
    const double bv = bc4(a.Bm, b, t, h, q), cv = bc4(a.Cm, b, t, h, q);
    const double st = hist[(int64_t)t * HP], sp = t > 0 ? hist[(int64_t)(t - 1) * HP] : s0;
    const double dout = dY[(int64_t)t * HP];
    double dyv = dout;
    if (a.z.ptr) {
      const double zv = bc4(a.z, b, t, h, q);
      atomicAdd(bc4p(g.dz, b, t, h, q), dout * (Dv * x + st * cv) * silu_grad_d(zv));
      dyv = dout * silu_d(zv);
    }
    const double da = exp(d * Av);
    const double G = cv * dyv + carry;
    atomicAdd(bc4p(g.dC, b, t, h, q), dyv * st);
    atomicAdd(bc4p(g.dB, b, t, h, q), G * d * x);
    dX[(int64_t)t * HP] = dyv * Dv + G * d * bv;
    const double gsa = G * sp * da;
    atomicAdd(md(g.ddt) + ((int64_t)b * a.len + t) * a.heads + h, G * bv * x + gsa * Av);
    dA_acc += gsa * d;
    dD_acc += dyv * x;
    carry = G * da;
  }
  atomicAdd(bc4p(g.dA, 0, 0, h, q), dA_acc);
  if (g.dD.ptr) atomicAdd(bc4p(g.dD, 0, 0, h, q), dD_acc);
  if (g.dinitial.ptr) atomicAdd(bc4p(g.dinitial, b, 0, h, q), carry);
}

// ---------------------------------------------------------------------------------------------
// depthwise causal conv: thread = (batch, channel, step)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int64_t conv_at(const ssm_conv_args& a, int b, int c, int t) {
  return a.channels_first ? (int64_t)b * a.row_sb + (int64_t)c * a.row_sc + t : ((int64_t)b * a.len + t) * a.channels + c;
}
__device__ __forceinline__ double conv_x(const ssm_conv_args& a, int b, int c, int t) {
  if (t >= 0) return cd(a.x)[conv_at(a, b, c, t)];
  if (a.halo && t >= -(a.width - 1)) return cd(a.halo)[((int64_t)b * a.channels + c) * (a.width - 1) + (a.width - 1) + t];
  return 0.0;
}
__device__ __forceinline__ double conv_pre(const ssm_conv_args& a, int b, int c, int t) {
  double acc = a.bias ? cd(a.bias)[c] : 0.0;
  for (int j = 0; j < a.width; ++j) acc += cd(a.weight)[(int64_t)c * a.width + j] * conv_x(a, b, c, t - (a.width - 1) + j);
  return acc;
}
__global__ void __launch_bounds__(kThreads) conv_kernel(const ssm_conv_bwd_args g, bool backward) {
  const ssm_conv_args& a = g.fwd;
  const int64_t id = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (id >= (int64_t)a.batch * a.channels * a.len) return;
  const int t = (int)(id % a.len), c = (int)((id / a.len) % a.channels), b = (int)(id / ((int64_t)a.len * a.channels));
  if (!backward) {
    const double pre = conv_pre(a, b, c, t);
    md(a.y)[conv_at(a, b, c, t)] = a.silu ? silu_d(pre) : pre;
    return;
  }
  // dpre[s] = dy[s] * act'(pre[s]);  dx[t] = sum_j w[j] dpre[t + (K - 1) - j];  dw[j] += dpre[t] x[t - (K - 1) + j];  db += dpre[t]
  auto dpre = [&](int s) {
    const double dyv = cd(g.dy)[conv_at(a, b, c, s)];
    return a.silu ? dyv * silu_grad_d(conv_pre(a, b, c, s)) : dyv;
  };
  double dx = 0.0;
  for (int j = 0; j < a.width; ++j) {
    const int s = t + (a.width - 1) - j;
    if (s < a.len) dx += cd(a.weight)[(int64_t)c * a.width + j] * dpre(s);
  }
  md(g.dx)[conv_at(a, b, c, t)] = dx;
  const double dp = dpre(t);
  for (int j = 0; j < a.width; ++j) atomicAdd(md(g.dweight) + (int64_t)c * a.width + j, dp * conv_x(a, b, c, t - (a.width - 1) + j));
  if (g.dbias) atomicAdd(md(g.dbias) + c, dp);
}

// ---------------------------------------------------------------------------------------------
// residual add + LayerNorm / RMSNorm: thread = row
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) norm_kernel(const ssm_norm_bwd_args g, bool backward) {
  const ssm_norm_args& a = g.fwd;
  const int64_t row = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (row >= a.rows) return;
  const int H = a.hidden;
  const double* x = cd(a.x) + row * H;
  const double* res = a.residual ? cd(a.residual) + row * H : nullptr;
  const double eps = (double)a.eps;
  auto sv = [&](int i) { return (res && a.prenorm) ? x[i] + res[i] : x[i]; };
  double mean = 0.0;
  if (!a.is_rms) {
    for (int i = 0; i < H; ++i) mean += sv(i);
    mean /= H;
  }
  double var = 0.0;
  for (int i = 0; i < H; ++i) var += (sv(i) - mean) * (sv(i) - mean);
  const double rstd = rsqrt(var / H + eps);
  if (!backward) {
    double* y = md(a.y) + row * H;
    for (int i = 0; i < H; ++i) {
      double v = (sv(i) - mean) * rstd * cd(a.weight)[i] + (a.bias ? cd(a.bias)[i] : 0.0);
      if (res && !a.prenorm) v += res[i];
      y[i] = v;
      if (a.residual_out) md(a.residual_out)[row * H + i] = res ? x[i] + res[i] : x[i];
    }
    return;
  }
  const double* dy = cd(g.dy) + row * H;
  const double* gro = g.dresidual_out ? cd(g.dresidual_out) + row * H : nullptr;
  double c1 = 0.0, c2 = 0.0;
  for (int i = 0; i < H; ++i) {
    const double xh = (sv(i) - mean) * rstd, wdy = dy[i] * cd(a.weight)[i];
    c1 += wdy * xh;
    c2 += wdy;
    atomicAdd(md(g.dweight) + i, dy[i] * xh);
    if (g.dbias) atomicAdd(md(g.dbias) + i, dy[i]);
  }
  c1 /= H;
  c2 = a.is_rms ? 0.0 : c2 / H;
  for (int i = 0; i < H; ++i) {
    const double xh = (sv(i) - mean) * rstd;
    double ds = (dy[i] * cd(a.weight)[i] - xh * c1 - c2) * rstd;
    double dres = a.prenorm ? ds : dy[i];
    if (gro) ds += gro[i], dres += gro[i];
    md(g.dx)[row * H + i] = ds;
    if (g.dresidual) md(g.dresidual)[row * H + i] = dres;
  }
}

static unsigned blocks(int64_t n) { return (unsigned)((n + kThreads - 1) / kThreads); }

}  // namespace f64

// ---- host side: called from the ordinary entry points when io_dtype == SSM_F64 -------------------------------------------
int f64_scan_fwd(const ssm_scan_fwd_args& a, cudaStream_t st) {
  SSM_REQUIRE(a.batch >= 0 && a.dim >= 0 && a.len >= 0 && a.nstate >= 1 && a.nstate <= f64::kMaxState, SSM_ERR_SHAPE, "selective_scan (fp64): bad shape");
  if (a.batch == 0 || a.dim == 0) return SSM_OK;
  SSM_REQUIRE(a.u && a.delta && a.A && a.Bm && a.Cm && a.out, SSM_ERR_NULL, "selective_scan (fp64): missing pointer");
  SSM_REQUIRE(a.bc_groups >= 1 && a.dim % a.bc_groups == 0, SSM_ERR_SHAPE, "B group dimension must divide D.");
  f64::scan_fwd_kernel<false><<<f64::blocks((int64_t)a.batch * a.dim), f64::kThreads, 0, st>>>(a, nullptr, true);
  return launch_status("f64::scan_fwd_kernel");
}

// fwd.checkpoints addresses the scratch of batch * dim * len * nstate doubles that holds the state after every step
int f64_scan_bwd(const ssm_scan_bwd_args& g, cudaStream_t st) {
  const ssm_scan_fwd_args& a = g.fwd;
  SSM_REQUIRE(a.batch >= 0 && a.dim >= 0 && a.len >= 0 && a.nstate >= 1 && a.nstate <= f64::kMaxState, SSM_ERR_SHAPE, "selective_scan_backward (fp64): bad shape");
  if (a.batch == 0 || a.dim == 0 || a.len == 0) return SSM_OK;
  SSM_REQUIRE(a.u && a.delta && a.A && a.Bm && a.Cm && a.checkpoints && g.dout && g.du && g.ddelta && g.dA && g.dB && g.dC, SSM_ERR_NULL,
              "selective_scan_backward (fp64): missing pointer");
  SSM_REQUIRE(!a.z == !g.dz, SSM_ERR_NULL, "selective_scan_backward: dz must be given exactly when z is");
  SSM_REQUIRE(a.bc_groups >= 1 && a.dim % a.bc_groups == 0, SSM_ERR_SHAPE, "B group dimension must divide D.");
  double* states = reinterpret_cast<double*>(a.checkpoints);
  f64::scan_fwd_kernel<true><<<f64::blocks((int64_t)a.batch * a.dim), f64::kThreads, 0, st>>>(a, states, false);
  if (int rc = launch_status("f64::scan_fwd_kernel<states>")) return rc;
  f64::scan_bwd_kernel<<<f64::blocks((int64_t)a.batch * a.dim), f64::kThreads, 0, st>>>(g, states);
  return launch_status("f64::scan_bwd_kernel");
}

int f64_step(const ssm_step_bwd_args& g, bool backward, cudaStream_t st) {
  const ssm_step_args& a = g.fwd;
  SSM_REQUIRE(a.batch >= 0 && a.dim >= 0 && a.nstate >= 1, SSM_ERR_SHAPE, "selective_state_step (fp64): bad shape");
  if (a.batch == 0 || a.dim == 0) return SSM_OK;
  SSM_REQUIRE(a.state && a.x && a.dt && a.A && a.Bm && a.Cm, SSM_ERR_NULL, "selective_state_step (fp64): missing pointer");
  SSM_REQUIRE(a.bc_groups >= 1 && a.dim % a.bc_groups == 0, SSM_ERR_SHAPE, "B group dimension must divide D.");
  SSM_REQUIRE(a.param_heads >= 0 && (a.param_heads == 0 || a.dim % a.param_heads == 0), SSM_ERR_SHAPE, "selective_state_step: param_heads must divide dim");
  if (backward) {
    SSM_REQUIRE(a.param_heads == 0, SSM_ERR_UNSUPPORTED, "selective_state_step_backward: per-head parameters have no backward");
    SSM_REQUIRE(g.dout && g.dstate && g.dx && g.ddt && g.dA && g.dB && g.dC, SSM_ERR_NULL, "selective_state_step_backward (fp64): missing pointer");
  } else {
    SSM_REQUIRE(a.out, SSM_ERR_NULL, "selective_state_step (fp64): missing pointer");
  }
  f64::step_kernel<<<f64::blocks((int64_t)a.batch * a.dim), f64::kThreads, 0, st>>>(g, backward);
  return launch_status("f64::step_kernel");
}

int f64_chunk(const ssm_chunk_bwd_args& g, bool backward, cudaStream_t st) {
  const ssm_chunk_args& a = g.fwd;
  SSM_REQUIRE(a.batch >= 0 && a.len >= 0 && a.heads >= 1 && a.proj >= 1, SSM_ERR_SHAPE, "ssd_chunk_scan (fp64): bad shape");
  if (a.batch == 0) return SSM_OK;
  SSM_REQUIRE(a.X && a.dt && a.A.ptr && a.Bm.ptr && a.Cm.ptr, SSM_ERR_NULL, "ssd_chunk_scan (fp64): missing pointer");
  if (backward) {
    SSM_REQUIRE(g.dY && g.dX && g.ddt && g.dA.ptr && g.dB.ptr && g.dC.ptr && g.history, SSM_ERR_NULL, "ssd_chunk_scan_backward (fp64): missing pointer");
    SSM_REQUIRE(!a.z.ptr || g.dz.ptr, SSM_ERR_NULL, "ssd_chunk_scan_backward (fp64): dz is required with z");
  } else {
    SSM_REQUIRE(a.Y, SSM_ERR_NULL, "ssd_chunk_scan (fp64): missing pointer");
  }
  f64::chunk_kernel<<<f64::blocks((int64_t)a.batch * a.heads * a.proj), f64::kThreads, 0, st>>>(g, backward);
  return launch_status("f64::chunk_kernel");
}

int f64_conv(const ssm_conv_bwd_args& g, bool backward, cudaStream_t st) {
  const ssm_conv_args& a = g.fwd;
  SSM_REQUIRE(a.batch >= 0 && a.channels >= 0 && a.len >= 0 && a.width >= 1 && a.width <= 8, SSM_ERR_SHAPE, "dw_causal_conv (fp64): bad shape");
  if (a.batch == 0 || a.channels == 0 || a.len == 0) return SSM_OK;
  SSM_REQUIRE(a.x && a.weight && (backward ? (g.dy && g.dx && g.dweight) : a.y != nullptr), SSM_ERR_NULL, "dw_causal_conv (fp64): missing pointer");
  f64::conv_kernel<<<f64::blocks((int64_t)a.batch * a.channels * a.len), f64::kThreads, 0, st>>>(g, backward);
  return launch_status("f64::conv_kernel");
}

// dweight / dbias are zero-filled by the caller and accumulated into (the fp32 path writes them instead)
int f64_norm(const ssm_norm_bwd_args& g, bool backward, cudaStream_t st) {
  const ssm_norm_args& a = g.fwd;
  SSM_REQUIRE(a.rows >= 0 && a.hidden >= 1, SSM_ERR_SHAPE, "fused_layer_norm (fp64): bad shape");
  if (a.rows == 0) return SSM_OK;
  SSM_REQUIRE(a.x && a.weight && (backward ? (g.dy && g.dx && g.dweight) : a.y != nullptr), SSM_ERR_NULL, "fused_layer_norm (fp64): missing pointer");
  f64::norm_kernel<<<f64::blocks(a.rows), f64::kThreads, 0, st>>>(g, backward);
  return launch_status("f64::norm_kernel");
}

}  // namespace ssmb
