// Single-token selective state step (decode), forward and backward, sm_100a.
//
// HBM-bound on the fp32 state: it is read once and written once per step, as float4, by a
// group of LPR lanes per (batch, channel) row that covers the row's states; everything
// else (softplus, dt bias, grouped B / C lookup, D skip, SiLU gate) is folded into the same
// pass.  No host synchronisation and no allocation.
#include "common.cuh"

namespace ssmb {

constexpr int kStepThreads = 128;

template <typename T, int LPR>
__global__ void __launch_bounds__(kStepThreads) step_fwd_kernel(const ssm_step_args a, int vec) {
  const int64_t gid = (int64_t)blockIdx.x * kStepThreads + threadIdx.x;
  const int64_t rows = (int64_t)a.batch * a.dim;
  const int64_t row_raw = gid / LPR;
  const bool live = row_raw < rows;
  const int64_t row = live ? row_raw : rows - 1;
  const int sg = (int)(gid % LPR);
  const int b = (int)(row / a.dim), d = (int)(row % a.dim);
  const int N = a.nstate;
  const int head = a.param_heads > 0 ? d / (a.dim / a.param_heads) : d;
  const int64_t prow = a.param_heads > 0 ? (int64_t)b * a.param_heads + head : row;

  const float x = to_f<T>(reinterpret_cast<const T*>(a.x)[row]);
  float dt = to_f<T>(reinterpret_cast<const T*>(a.dt)[prow]);
  if (a.dt_bias) dt += __ldg(a.dt_bias + head);
  if (a.dt_softplus) dt = softplus_f(dt);
  const float dtx = dt * x;
  const int g = d / (a.dim / a.bc_groups);
  const int64_t boff = (int64_t)b * a.b_sb + (int64_t)g * a.b_sg;
  const int64_t coff = (int64_t)b * a.c_sb + (int64_t)g * a.c_sg;
  float* st = a.state + row * N;
  float y = 0.f;
  if (vec) {
    for (int n0 = sg * 4; n0 < N; n0 += LPR * 4) {
      float4 s = *reinterpret_cast<const float4*>(st + n0);
      float sv[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int n = n0 + i;
        const float An = a.param_heads > 0 ? __ldg(a.A + head) : __ldg(a.A + (int64_t)d * N + n);
        const float Bn = load_dyn(a.Bm, boff + (int64_t)n * a.b_sn, a.bc_dtype);
        const float Cn = load_dyn(a.Cm, coff + (int64_t)n * a.c_sn, a.bc_dtype);
        sv[i] = fmaf(ex2_approx(dt * An * kLog2e), sv[i], dtx * Bn);
        y = fmaf(Cn, sv[i], y);
      }
      if (live) *reinterpret_cast<float4*>(st + n0) = make_float4(sv[0], sv[1], sv[2], sv[3]);
    }
  } else {
    for (int n = sg; n < N; n += LPR) {
      const float An = a.param_heads > 0 ? __ldg(a.A + head) : __ldg(a.A + (int64_t)d * N + n);
      const float Bn = load_dyn(a.Bm, boff + (int64_t)n * a.b_sn, a.bc_dtype);
      const float Cn = load_dyn(a.Cm, coff + (int64_t)n * a.c_sn, a.bc_dtype);
      const float s = fmaf(ex2_approx(dt * An * kLog2e), st[n], dtx * Bn);
      if (live) st[n] = s;
      y = fmaf(Cn, s, y);
    }
  }
  y = group_sum<LPR, 1>(y);
  if (sg == 0 && live) {
    if (a.D) y = fmaf(__ldg(a.D + head), x, y);
    if (a.z) y *= silu_fast(to_f<T>(reinterpret_cast<const T*>(a.z)[row]));
    reinterpret_cast<T*>(a.out)[row] = from_f<T>(y);
  }
}

// Fast path: every lane owns NV float4 groups of its row's state, all loaded before any is used so
// that each thread keeps NV * 16 bytes of the dominant stream in flight; the LPR lanes of a row
// read adjacent groups.  Needs nstate == 4 * NV * LPR.
template <typename T, int NV, int LPR>
__global__ void __launch_bounds__(kStepThreads) step_fwd_vec_kernel(const ssm_step_args a) {
  const int64_t gid = (int64_t)blockIdx.x * kStepThreads + threadIdx.x;
  const int64_t rows = (int64_t)a.batch * a.dim;
  const int64_t row_raw = gid / LPR;
  const bool live = row_raw < rows;
  const int64_t row = live ? row_raw : rows - 1;
  const int sg = (int)(gid % LPR);
  const int b = (int)(row / a.dim), d = (int)(row % a.dim);
  constexpr int N = 4 * NV * LPR;
  const int head = a.param_heads > 0 ? d / (a.dim / a.param_heads) : d;
  const int64_t prow = a.param_heads > 0 ? (int64_t)b * a.param_heads + head : row;
  float* st = a.state + row * N;
  float4 s[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) s[v] = *reinterpret_cast<const float4*>(st + (sg + v * LPR) * 4);
  const float x = to_f<T>(reinterpret_cast<const T*>(a.x)[row]);
  float dt = to_f<T>(reinterpret_cast<const T*>(a.dt)[prow]);
  if (a.dt_bias) dt += __ldg(a.dt_bias + head);
  if (a.dt_softplus) dt = softplus_fast(dt);
  const float dtx = dt * x;
  const int g = d / (a.dim / a.bc_groups);
  const int64_t boff = (int64_t)b * a.b_sb + (int64_t)g * a.b_sg;
  const int64_t coff = (int64_t)b * a.c_sb + (int64_t)g * a.c_sg;
  const float Ahead = a.param_heads > 0 ? __ldg(a.A + head) * kLog2e : 0.f;
  float y = 0.f;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int n0 = (sg + v * LPR) * 4;
    float An[4];
    if (a.param_heads > 0) {
      An[0] = An[1] = An[2] = An[3] = Ahead;
    } else {
      const float4 q = __ldg(reinterpret_cast<const float4*>(a.A + (int64_t)d * N + n0));
      An[0] = q.x * kLog2e, An[1] = q.y * kLog2e, An[2] = q.z * kLog2e, An[3] = q.w * kLog2e;
    }
    float sv[4] = {s[v].x, s[v].y, s[v].z, s[v].w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float Bn = load_dyn(a.Bm, boff + (int64_t)(n0 + i) * a.b_sn, a.bc_dtype);
      const float Cn = load_dyn(a.Cm, coff + (int64_t)(n0 + i) * a.c_sn, a.bc_dtype);
      sv[i] = fmaf(ex2_approx(dt * An[i]), sv[i], dtx * Bn);
      y = fmaf(Cn, sv[i], y);
    }
    if (live) *reinterpret_cast<float4*>(st + n0) = make_float4(sv[0], sv[1], sv[2], sv[3]);
  }
  y = group_sum<LPR, 1>(y);
  if (sg == 0 && live) {
    if (a.D) y = fmaf(__ldg(a.D + head), x, y);
    if (a.z) y *= silu_fast(to_f<T>(reinterpret_cast<const T*>(a.z)[row]));
    reinterpret_cast<T*>(a.out)[row] = from_f<T>(y);
  }
}

// Four consecutive B or C values of compile-time element type BT as fp32 (one 8- or 16-byte load).
template <typename BT>
__device__ __forceinline__ void load_bc4(const void* base, int64_t off, float (&v)[4]) {
  if constexpr (sizeof(BT) == 4) {
    const float4 q = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off));
    v[0] = q.x, v[1] = q.y, v[2] = q.z, v[3] = q.w;
  } else {
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const BT*>(base) + off));
    const BT* e = reinterpret_cast<const BT*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = to_f<BT>(e[i]);
  }
}

// The same fast path with B / C rows read as vectors: unit state stride, every (batch, group) row of B and C aligned to the
// vector, element type BT known at compile time.  This is the layout decoding uses (B, C of shape (batch, groups, nstate));
// it replaces 2 x nstate scalar loads with run-time type dispatch per thread by 2 x nstate / 4 vector loads.
template <typename T, typename BT, int NV, int LPR>
__global__ void __launch_bounds__(kStepThreads) step_fwd_fast_kernel(const ssm_step_args a) {
  const int64_t gid = (int64_t)blockIdx.x * kStepThreads + threadIdx.x;
  const int64_t rows = (int64_t)a.batch * a.dim;
  const int64_t row_raw = gid / LPR;
  const bool live = row_raw < rows;
  const int64_t row = live ? row_raw : rows - 1;
  const int sg = (int)(gid % LPR);
  const int b = (int)(row / a.dim), d = (int)(row % a.dim);
  constexpr int N = 4 * NV * LPR;
  const int head = a.param_heads > 0 ? d / (a.dim / a.param_heads) : d;
  const int64_t prow = a.param_heads > 0 ? (int64_t)b * a.param_heads + head : row;
  float* st = a.state + row * N;
  float4 s[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) s[v] = __ldcs(reinterpret_cast<const float4*>(st + (sg + v * LPR) * 4));
  const int g = d / (a.dim / a.bc_groups);
  const int64_t boff = (int64_t)b * a.b_sb + (int64_t)g * a.b_sg;
  const int64_t coff = (int64_t)b * a.c_sb + (int64_t)g * a.c_sg;
  float Bv[NV][4], Cv[NV][4], An[NV][4];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int n0 = (sg + v * LPR) * 4;
    load_bc4<BT>(a.Bm, boff + n0, Bv[v]);
    load_bc4<BT>(a.Cm, coff + n0, Cv[v]);
    if (a.param_heads == 0) {
      const float4 q = __ldg(reinterpret_cast<const float4*>(a.A + (int64_t)d * N + n0));
      An[v][0] = q.x * kLog2e, An[v][1] = q.y * kLog2e, An[v][2] = q.z * kLog2e, An[v][3] = q.w * kLog2e;
    }
  }
  const float x = to_f<T>(reinterpret_cast<const T*>(a.x)[row]);
  float dt = to_f<T>(reinterpret_cast<const T*>(a.dt)[prow]);
  if (a.dt_bias) dt += __ldg(a.dt_bias + head);
  if (a.dt_softplus) dt = softplus_fast(dt);
  const float dtx = dt * x;
  float y = 0.f;
  if (a.param_heads > 0) {  // one decay for the whole head: a single ex2 per thread
    const float da = ex2_approx(dt * __ldg(a.A + head) * kLog2e);
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      float sv[4] = {s[v].x, s[v].y, s[v].z, s[v].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        sv[i] = fmaf(da, sv[i], dtx * Bv[v][i]);
        y = fmaf(Cv[v][i], sv[i], y);
      }
      if (live) __stcs(reinterpret_cast<float4*>(st + (sg + v * LPR) * 4), make_float4(sv[0], sv[1], sv[2], sv[3]));
    }
  } else {
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      float sv[4] = {s[v].x, s[v].y, s[v].z, s[v].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        sv[i] = fmaf(ex2_approx(dt * An[v][i]), sv[i], dtx * Bv[v][i]);
        y = fmaf(Cv[v][i], sv[i], y);
      }
      if (live) __stcs(reinterpret_cast<float4*>(st + (sg + v * LPR) * 4), make_float4(sv[0], sv[1], sv[2], sv[3]));
    }
  }
  y = group_sum<LPR, 1>(y);
  if (sg == 0 && live) {
    if (a.D) y = fmaf(__ldg(a.D + head), x, y);
    if (a.z) y *= silu_fast(to_f<T>(reinterpret_cast<const T*>(a.z)[row]));
    reinterpret_cast<T*>(a.out)[row] = from_f<T>(y);
  }
}

// Backward of the plain step.  One group of LPR lanes per row, parameter gradients by atomics.
template <typename T, int LPR>
__global__ void __launch_bounds__(kStepThreads) step_bwd_kernel(const ssm_step_bwd_args g) {
  const ssm_step_args& a = g.fwd;
  const int64_t gid = (int64_t)blockIdx.x * kStepThreads + threadIdx.x;
  const int64_t rows = (int64_t)a.batch * a.dim;
  const int64_t row_raw = gid / LPR;
  const bool live = row_raw < rows;
  const int64_t row = live ? row_raw : rows - 1;
  const int sg = (int)(gid % LPR);
  const int b = (int)(row / a.dim), d = (int)(row % a.dim);
  const int N = a.nstate;
  const float x = to_f<T>(reinterpret_cast<const T*>(a.x)[row]);
  float pre = to_f<T>(reinterpret_cast<const T*>(a.dt)[row]);
  if (a.dt_bias) pre += __ldg(a.dt_bias + d);
  const float dt = a.dt_softplus ? softplus_f(pre) : pre;
  const float zv = a.z ? to_f<T>(reinterpret_cast<const T*>(a.z)[row]) : 0.f;
  const float gate = a.z ? silu_f(zv) : 1.f;
  const float dout = to_f<T>(reinterpret_cast<const T*>(g.dout)[row]);
  const float dy = dout * gate;
  const int grp = d / (a.dim / a.bc_groups);
  const int64_t boff = (int64_t)b * a.b_sb + (int64_t)grp * a.b_sg;
  const int64_t coff = (int64_t)b * a.c_sb + (int64_t)grp * a.c_sg;
  float y = 0.f, sum_gb = 0.f, sum_da = 0.f;
  for (int n = sg; n < N; n += LPR) {
    const float An = __ldg(a.A + (int64_t)d * N + n);
    const float Bn = load_dyn(a.Bm, boff + (int64_t)n * a.b_sn, a.bc_dtype);
    const float Cn = load_dyn(a.Cm, coff + (int64_t)n * a.c_sn, a.bc_dtype);
    const float s = a.state[row * N + n];
    const float da = expf(dt * An);
    const float nw = fmaf(da, s, dt * x * Bn);
    y = fmaf(Cn, nw, y);
    const float G = fmaf(Cn, dy, g.dnew_state ? g.dnew_state[row * N + n] : 0.f);
    if (live) {
      g.dstate[row * N + n] = G * da;
      atomicAdd(g.dC + coff + (int64_t)n * a.c_sn, dy * nw);
      atomicAdd(g.dB + boff + (int64_t)n * a.b_sn, G * dt * x);
      atomicAdd(g.dA + (int64_t)d * N + n, G * s * da * dt);
    }
    sum_gb = fmaf(G, Bn, sum_gb);
    sum_da = fmaf(G * s * da, An, sum_da);
  }
  y = group_sum<LPR, 1>(y);
  sum_gb = group_sum<LPR, 1>(sum_gb);
  sum_da = group_sum<LPR, 1>(sum_da);
  if (sg == 0 && live) {
    const float Dv = a.D ? __ldg(a.D + d) : 0.f;
    const float yfull = fmaf(Dv, x, y);
    if (g.dz) {
      const float s = sigmoid_f(zv);
      reinterpret_cast<T*>(g.dz)[row] = from_f<T>(dout * yfull * s * (1.f + zv * (1.f - s)));
    }
    reinterpret_cast<T*>(g.dx)[row] = from_f<T>(fmaf(dy, Dv, sum_gb * dt));
    const float ddl = fmaf(sum_gb, x, sum_da);
    const float dpre = a.dt_softplus ? ddl * softplus_grad_f(pre) : ddl;
    reinterpret_cast<T*>(g.ddt)[row] = from_f<T>(dpre);
    if (g.dD) atomicAdd(g.dD + d, dy * x);
    if (g.ddt_bias) atomicAdd(g.ddt_bias + d, dpre);
  }
}

static int step_validate(const ssm_step_args* a) {
  SSM_REQUIRE(a != nullptr, SSM_ERR_NULL, "selective_state_step: args is NULL");
  SSM_REQUIRE(a->batch >= 0 && a->dim >= 0 && a->nstate >= 1, SSM_ERR_SHAPE, "selective_state_step: bad shape");
  SSM_REQUIRE(valid_dtype(a->io_dtype) && valid_dtype(a->bc_dtype), SSM_ERR_DTYPE, "selective_state_step: unknown dtype");
  if (a->batch == 0 || a->dim == 0) return SSM_OK;
  SSM_REQUIRE(a->state && a->x && a->dt && a->A && a->Bm && a->Cm, SSM_ERR_NULL, "selective_state_step: missing pointer");
  SSM_REQUIRE(a->bc_groups >= 1 && a->dim % a->bc_groups == 0, SSM_ERR_SHAPE, "B group dimension must divide D.");
  SSM_REQUIRE(a->param_heads >= 0 && (a->param_heads == 0 || a->dim % a->param_heads == 0), SSM_ERR_SHAPE,
              "selective_state_step: param_heads must divide dim");
  return SSM_OK;
}

static int step_lpr(int n, bool vec) {
  const int per = vec ? (n + 3) / 4 : n;
  int l = 1;
  while (l < per && l < 32) l <<= 1;
  return l;
}

template <typename T, int LPR>
static int step_fwd_launch(const ssm_step_args& a, int vec, cudaStream_t st) {
  const int64_t threads = (int64_t)a.batch * a.dim * LPR;
  step_fwd_kernel<T, LPR><<<(unsigned)((threads + kStepThreads - 1) / kStepThreads), kStepThreads, 0, st>>>(a, vec);
  return launch_status("step_fwd_kernel");
}
template <typename T, int LPR>
static int step_bwd_launch(const ssm_step_bwd_args& g, cudaStream_t st) {
  const int64_t threads = (int64_t)g.fwd.batch * g.fwd.dim * LPR;
  step_bwd_kernel<T, LPR><<<(unsigned)((threads + kStepThreads - 1) / kStepThreads), kStepThreads, 0, st>>>(g);
  return launch_status("step_bwd_kernel");
}

template <typename T, int NV, int LPR>
static int step_fwd_vec_launch(const ssm_step_args& a, cudaStream_t st) {
  const int64_t threads = (int64_t)a.batch * a.dim * LPR;
  step_fwd_vec_kernel<T, NV, LPR><<<(unsigned)((threads + kStepThreads - 1) / kStepThreads), kStepThreads, 0, st>>>(a);
  return launch_status("step_fwd_vec_kernel");
}

template <typename T, typename BT, int NV, int LPR>
static int step_fwd_fast_launch(const ssm_step_args& a, cudaStream_t st) {
  const int64_t threads = (int64_t)a.batch * a.dim * LPR;
  step_fwd_fast_kernel<T, BT, NV, LPR><<<(unsigned)((threads + kStepThreads - 1) / kStepThreads), kStepThreads, 0, st>>>(a);
  return launch_status("step_fwd_fast_kernel");
}
template <typename T, typename BT>
static int step_fwd_fast_n(const ssm_step_args& a, cudaStream_t st) {
  switch (a.nstate) {
    case 16: return step_fwd_fast_launch<T, BT, 4, 1>(a, st);
    case 32: return step_fwd_fast_launch<T, BT, 4, 2>(a, st);
    case 64: return step_fwd_fast_launch<T, BT, 4, 4>(a, st);
    case 128: return step_fwd_fast_launch<T, BT, 4, 8>(a, st);
    default: return step_fwd_fast_launch<T, BT, 4, 16>(a, st);
  }
}

template <typename T>
static int step_fwd_t(const ssm_step_args& a, cudaStream_t st) {
  if (aligned_to(a.state, 16) && aligned_to(a.A, 16)) {
    // vector loads of B / C: unit state stride and rows that start on a vector boundary
    const int bcb = dtype_size(a.bc_dtype);
    const int64_t per = 16 / bcb / (bcb == 4 ? 1 : 2);  // elements per load: 4 (one 16-byte or one 8-byte load)
    const bool n_ok = a.nstate == 16 || a.nstate == 32 || a.nstate == 64 || a.nstate == 128 || a.nstate == 256;
    const bool bc_ok = a.b_sn == 1 && a.c_sn == 1 && a.b_sb % per == 0 && a.b_sg % per == 0 && a.c_sb % per == 0 && a.c_sg % per == 0 &&
                       aligned_to(a.Bm, 4 * bcb) && aligned_to(a.Cm, 4 * bcb);
    if (n_ok && bc_ok) {
      switch (a.bc_dtype) {
        case SSM_F32: return step_fwd_fast_n<T, float>(a, st);
        case SSM_BF16: return step_fwd_fast_n<T, __nv_bfloat16>(a, st);
        default: return step_fwd_fast_n<T, __half>(a, st);
      }
    }
    switch (a.nstate) {
      case 4: return step_fwd_vec_launch<T, 1, 1>(a, st);
      case 8: return step_fwd_vec_launch<T, 2, 1>(a, st);
      case 16: return step_fwd_vec_launch<T, 4, 1>(a, st);
      case 32: return step_fwd_vec_launch<T, 4, 2>(a, st);
      case 64: return step_fwd_vec_launch<T, 4, 4>(a, st);
      case 128: return step_fwd_vec_launch<T, 4, 8>(a, st);
      case 256: return step_fwd_vec_launch<T, 4, 16>(a, st);
      default: break;
    }
  }
  const int vec = (a.nstate % 4 == 0) && aligned_to(a.state, 16);
  switch (step_lpr(a.nstate, vec != 0)) {
    case 1: return step_fwd_launch<T, 1>(a, vec, st);
    case 2: return step_fwd_launch<T, 2>(a, vec, st);
    case 4: return step_fwd_launch<T, 4>(a, vec, st);
    case 8: return step_fwd_launch<T, 8>(a, vec, st);
    case 16: return step_fwd_launch<T, 16>(a, vec, st);
    default: return step_fwd_launch<T, 32>(a, vec, st);
  }
}
template <typename T>
static int step_bwd_t(const ssm_step_bwd_args& g, cudaStream_t st) {
  switch (step_lpr(g.fwd.nstate, false)) {
    case 1: return step_bwd_launch<T, 1>(g, st);
    case 2: return step_bwd_launch<T, 2>(g, st);
    case 4: return step_bwd_launch<T, 4>(g, st);
    case 8: return step_bwd_launch<T, 8>(g, st);
    case 16: return step_bwd_launch<T, 16>(g, st);
    default: return step_bwd_launch<T, 32>(g, st);
  }
}

}  // namespace ssmb

using namespace ssmb;

extern "C" int ssm_selective_state_step(const ssm_step_args* a, ssm_stream_t stream) {
  if (a && a->io_dtype == SSM_F64) {
    ssm_step_bwd_args g{};
    g.fwd = *a;
    return f64_step(g, false, reinterpret_cast<cudaStream_t>(stream));
  }
  if (int rc = step_validate(a)) return rc;
  if (a->batch == 0 || a->dim == 0) return SSM_OK;
  SSM_REQUIRE(a->out, SSM_ERR_NULL, "selective_state_step: out is required");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (a->io_dtype) {
    case SSM_F32: return step_fwd_t<float>(*a, st);
    case SSM_BF16: return step_fwd_t<__nv_bfloat16>(*a, st);
    default: return step_fwd_t<__half>(*a, st);
  }
}

extern "C" int ssm_selective_state_step_bwd(const ssm_step_bwd_args* g, ssm_stream_t stream) {
  SSM_REQUIRE(g != nullptr, SSM_ERR_NULL, "selective_state_step_backward: args is NULL");
  const ssm_step_args* a = &g->fwd;
  if (a->io_dtype == SSM_F64) return f64_step(*g, true, reinterpret_cast<cudaStream_t>(stream));
  if (int rc = step_validate(a)) return rc;
  SSM_REQUIRE(a->param_heads == 0, SSM_ERR_UNSUPPORTED, "selective_state_step_backward: per-head parameters have no backward");
  if (a->batch == 0 || a->dim == 0) return SSM_OK;
  SSM_REQUIRE(g->dout && g->dstate && g->dx && g->ddt && g->dA && g->dB && g->dC, SSM_ERR_NULL,
              "selective_state_step_backward: missing pointer");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (a->io_dtype) {
    case SSM_F32: return step_bwd_t<float>(*g, st);
    case SSM_BF16: return step_bwd_t<__nv_bfloat16>(*g, st);
    default: return step_bwd_t<__half>(*g, st);
  }
}
