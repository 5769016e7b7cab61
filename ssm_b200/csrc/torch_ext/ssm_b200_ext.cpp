// Thin PyTorch extension over the C ABI of include/ssm_b200.h.
//
// It exports the ten callables that upstream's facade (src/ssm/ops/__init__.py) invokes on
// its compiled CUDA backend, with the names, keyword arguments, defaults and return tuples
// that src/ssm/ops/cuda/bindings.cpp:96-152 fixes (selective_scan -> 3-tuple,
// selective_scan_backward -> 8-tuple, selective_state_step_backward -> the 9 values the
// facade zips with its nine requires_grad flags at src/ssm/ops/__init__.py:669-676, ...).
// Each function validates shapes the way the specification does (reference.py:22-84 and the
// operator bodies), allocates its outputs with ATen, fills the plain C struct of the matching
// entry point from data_ptr() / stride(), and launches on the current CUDA stream of the
// tensors' device.  Violations are reported with TORCH_CHECK, i.e. as RuntimeError, which the
// facade turns into ValueError (src/ssm/ops/__init__.py:1244-1252).  There is no fallback of
// any kind: CPU tensors are rejected.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <string>
#include <tuple>
#include <vector>

#include "../../../include/ssm_b200.h"

namespace {

using at::Tensor;
using OptTensor = c10::optional<at::Tensor>;

int dtype_code(const Tensor& t, const char* what) {
  switch (t.scalar_type()) {
    case at::kFloat: return SSM_F32;
    case at::kBFloat16: return SSM_BF16;
    case at::kHalf: return SSM_F16;
    default: TORCH_CHECK(false, what, ": dtype ", t.scalar_type(), " is not built (float32, bfloat16 and float16 are)");
  }
  return -1;
}
bool io_dtype_ok(const Tensor& t) { return t.scalar_type() == at::kFloat || t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kHalf; }

void need_cuda(const Tensor& ref, std::initializer_list<const OptTensor*> rest) {
  TORCH_CHECK(ref.is_cuda(), "ssm_b200 operators run on CUDA tensors only; there is no CPU fallback");
  for (const OptTensor* t : rest)
    if (t->has_value()) TORCH_CHECK((*t)->is_cuda() && (*t)->device() == ref.device(), "all tensors must be on the same CUDA device");
}
void same_device(const Tensor& ref, std::initializer_list<const Tensor*> rest) {
  TORCH_CHECK(ref.is_cuda(), "ssm_b200 operators run on CUDA tensors only; there is no CPU fallback");
  for (const Tensor* t : rest) TORCH_CHECK(t->is_cuda() && t->device() == ref.device(), "all tensors must be on the same CUDA device");
}

Tensor f32c(const Tensor& t) { return t.detach().to(at::kFloat).contiguous(); }
OptTensor f32c(const OptTensor& t) { return t.has_value() ? OptTensor(f32c(*t)) : OptTensor(); }
Tensor like(const Tensor& t, const Tensor& ref) { return t.detach().to(ref.scalar_type()).contiguous(); }
const void* ptr(const OptTensor& t) { return t.has_value() ? t->data_ptr() : nullptr; }
const float* fptr(const OptTensor& t) { return t.has_value() ? t->data_ptr<float>() : nullptr; }
float* fptr_mut(OptTensor& t) { return t.has_value() ? t->data_ptr<float>() : nullptr; }

void run(int rc) {
  if (rc == 0) return;
  const char* msg = ssm_b200_last_error();
  TORCH_CHECK(false, (msg && *msg) ? msg : "libssm_b200 call failed", " (code ", rc, ")");
}
ssm_stream_t stream_of(const Tensor& t) { return reinterpret_cast<ssm_stream_t>(at::cuda::getCurrentCUDAStream(t.get_device()).stream()); }

// ---------------------------------------------------------------------------------------------
// selective scan
// ---------------------------------------------------------------------------------------------
struct Coeff {
  Tensor t;
  int groups;
  int64_t sb, sg, sn, st;
};

// B / C in one of the layouts of reference.py:22-56 -> tensor + group count + element strides
Coeff scan_coeff(const char* name, const Tensor& p, int64_t nb, int64_t nd, int64_t nn, int64_t nl) {
  if (p.dim() == 2) {
    TORCH_CHECK(p.size(0) == nd && p.size(1) == nn, name, " must have shape (D, N).");
    return {f32c(p), (int)nd, 0, nn, 1, 0};
  }
  if (p.dim() == 3) {
    TORCH_CHECK(p.size(0) == nb && p.size(1) == nd && p.size(2) == nn, name, " must have shape (B, D, N) when 3-D.");
    return {f32c(p), (int)nd, nd * nn, nn, 1, 0};
  }
  TORCH_CHECK(p.dim() == 4, "Unsupported rank for ", name, ".");
  TORCH_CHECK(p.size(0) == nb && p.size(3) == nl, name, " must have shape (B, G, N, L) when 4-D.");
  const int64_t g = p.size(1);
  TORCH_CHECK(g > 0 && nd % g == 0, "Group dimension must divide D.");
  TORCH_CHECK(p.size(2) == nn, name, " has mismatched state dimension.");
  Tensor t = io_dtype_ok(p) ? p.detach().contiguous() : f32c(p);
  return {t, (int)g, g * nn * nl, nn * nl, nl, 1};
}

struct ScanCtx {
  int64_t nb, nd, nl, nn;
  Tensor u, delta, A;
  OptTensor z, D, bias;
  Coeff B, C;
  bool softplus;

  ScanCtx(const Tensor& u_, const Tensor& delta_, const Tensor& A_, const Tensor& B_, const Tensor& C_, const OptTensor& D_, const OptTensor& z_,
          const OptTensor& bias_, bool softplus_)
      : softplus(softplus_) {
    TORCH_CHECK(u_.dim() == 3 && delta_.dim() == 3, "u and delta must have shape (B, D, L).");
    nb = u_.size(0), nd = u_.size(1), nl = u_.size(2);
    TORCH_CHECK(delta_.sizes() == u_.sizes(), "delta must match the shape of u.");
    TORCH_CHECK(A_.dim() == 2 && A_.size(0) == nd, "A must have shape (D, N).");
    TORCH_CHECK(!A_.is_complex(), "selective_scan: complex A is not built");
    nn = A_.size(1);
    TORCH_CHECK(nn >= 1 && nn <= 256, "selective_scan: the state dimension must be in [1, 256].");
    same_device(u_, {&delta_, &A_, &B_, &C_});
    need_cuda(u_, {&D_, &z_, &bias_});
    dtype_code(u_, "selective_scan");
    u = u_.detach().contiguous();
    delta = like(delta_, u);
    A = f32c(A_);
    B = scan_coeff("B", B_, nb, nd, nn, nl);
    C = scan_coeff("C", C_, nb, nd, nn, nl);
    if (B.groups != C.groups) {  // expand the coarser grouping so that one group map serves both
      const int g = std::max(B.groups, C.groups);
      TORCH_CHECK(g % std::min(B.groups, C.groups) == 0, "B and C group dimensions must nest.");
      Coeff& low = B.groups < g ? B : C;
      TORCH_CHECK(low.st != 0, "B and C group dimensions must nest.");
      low.t = low.t.repeat_interleave(g / low.groups, 1).contiguous();
      low.groups = g, low.sb = g * nn * nl, low.sg = nn * nl, low.sn = nl, low.st = 1;
    }
    if (B.t.scalar_type() != C.t.scalar_type()) B.t = B.t.to(at::kFloat), C.t = C.t.to(at::kFloat);
    if (D_.has_value()) TORCH_CHECK(D_->dim() == 1 && D_->size(0) == nd, "D must have shape (D,).");
    if (z_.has_value()) TORCH_CHECK(z_->sizes() == u_.sizes(), "z must have shape (B, D, L).");
    if (bias_.has_value()) TORCH_CHECK(bias_->dim() == 1 && bias_->size(0) == nd, "dt_bias must have shape (D,).");
    D = f32c(D_), bias = f32c(bias_);
    if (z_.has_value()) z = like(*z_, u);
  }

  void fill(ssm_scan_fwd_args& a) const {
    a.batch = (int)nb, a.dim = (int)nd, a.len = (int)nl, a.nstate = (int)nn;
    a.io_dtype = dtype_code(u, "selective_scan"), a.bc_dtype = dtype_code(B.t, "selective_scan B/C");
    a.delta_softplus = softplus;
    a.u = u.data_ptr(), a.delta = delta.data_ptr(), a.z = ptr(z), a.A = A.data_ptr<float>();
    a.Bm = B.t.data_ptr(), a.Cm = C.t.data_ptr(), a.bc_groups = B.groups;
    a.b_sb = B.sb, a.b_sg = B.sg, a.b_sn = B.sn, a.b_st = B.st;
    a.c_sb = C.sb, a.c_sg = C.sg, a.c_sn = C.sn, a.c_st = C.st;
    a.D = fptr(D), a.dt_bias = fptr(bias), a.initial_state = nullptr;
    a.row_sb = nd * nl, a.row_sd = nl;
  }
};

Tensor scan_checkpoints(const ScanCtx& c) {
  const int iv = ssm_scan_checkpoint_interval();
  return at::empty({c.nb, c.nd, std::max<int64_t>(1, (c.nl + iv - 1) / iv), c.nn}, c.u.options().dtype(at::kFloat));
}

std::tuple<Tensor, Tensor, Tensor> selective_scan(const Tensor& u, const Tensor& delta, const Tensor& A, const Tensor& B, const Tensor& C,
                                                  const OptTensor& D, const OptTensor& z, const OptTensor& dt_bias, bool softplus,
                                                  bool return_last_state) {
  ScanCtx c(u, delta, A, B, C, D, z, dt_bias, softplus);
  c10::cuda::CUDAGuard guard(c.u.device());
  Tensor out = at::empty_like(c.u);
  Tensor last = return_last_state ? at::empty({c.nb, c.nd, c.nn}, c.u.options()) : at::empty({0}, c.u.options());
  Tensor cache = scan_checkpoints(c);
  ssm_scan_fwd_args a{};
  c.fill(a);
  a.out = out.data_ptr();
  a.last_state = return_last_state ? last.data_ptr() : nullptr;
  a.last_dtype = a.io_dtype;
  a.checkpoints = cache.data_ptr<float>();
  const int nseg = ssm_scan_split_segments((int)c.nb, (int)c.nd, (int)c.nl, (int)c.nn);  // > 1: cut the sequence into parallel segments
  Tensor split;
  if (nseg > 1) {
    split = at::empty({2 * c.nb * c.nd * nseg * c.nn}, c.u.options().dtype(at::kFloat));
    a.split_scratch = split.data_ptr<float>(), a.split_segments = nseg;
  }
  run(ssm_selective_scan_fwd(&a, stream_of(c.u)));
  return {out, last, cache};
}

// gradient buffer of a coefficient, folded back to the shape / dtype of the tensor the caller passed
Tensor fold_coeff_grad(const Tensor& grad, const Tensor& like_) {
  Tensor g = grad;
  if (g.sizes() != like_.sizes()) {  // the coefficient had been regrouped: sum the repeats back
    const int64_t rep = g.size(1) / like_.size(1);
    g = g.view({like_.size(0), like_.size(1), rep, like_.size(2), like_.size(3)}).sum(2);
  }
  return g.to(like_.scalar_type());
}

std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor, OptTensor, OptTensor, OptTensor> selective_scan_backward(
    const Tensor& grad_output, const OptTensor& grad_last_state, const Tensor& u, const Tensor& delta, const Tensor& A, const Tensor& B,
    const Tensor& C, const OptTensor& D, const OptTensor& z, const OptTensor& dt_bias, bool softplus, const OptTensor& forward_output,
    const OptTensor& cache) {
  (void)forward_output;  // the kernel rebuilds what it needs from the checkpoints
  ScanCtx c(u, delta, A, B, C, D, z, dt_bias, softplus);
  c10::cuda::CUDAGuard guard(c.u.device());
  TORCH_CHECK(grad_output.sizes() == c.u.sizes(), "grad_output must have the shape of u.");
  Tensor ck;
  ssm_scan_bwd_args g{};
  c.fill(g.fwd);
  if (cache.has_value() && cache->numel() > 0) {
    ck = f32c(*cache);
  } else {  // no checkpoints handed over: one forward pass produces them
    ck = scan_checkpoints(c);
    Tensor scratch_out = at::empty_like(c.u);
    ssm_scan_fwd_args f = g.fwd;
    f.out = scratch_out.data_ptr(), f.checkpoints = ck.data_ptr<float>();
    run(ssm_selective_scan_fwd(&f, stream_of(c.u)));
  }
  g.fwd.checkpoints = ck.data_ptr<float>();
  const auto f32 = c.u.options().dtype(at::kFloat);
  Tensor go = like(grad_output, c.u);
  OptTensor gl = f32c(grad_last_state);
  if (gl.has_value()) TORCH_CHECK(gl->dim() == 3 && gl->size(0) == c.nb && gl->size(1) == c.nd && gl->size(2) == c.nn, "grad_last_state must have shape (B, D, N).");
  Tensor du = at::empty_like(c.u), dd = at::empty_like(c.u);
  OptTensor dz = c.z.has_value() ? OptTensor(at::empty_like(c.u)) : OptTensor();
  Tensor dA = at::zeros({c.nd, c.nn}, f32), dB = at::zeros(c.B.t.sizes(), f32), dC = at::zeros(c.C.t.sizes(), f32);
  OptTensor dD = c.D.has_value() ? OptTensor(at::zeros({c.nd}, f32)) : OptTensor();
  OptTensor db = c.bias.has_value() ? OptTensor(at::zeros({c.nd}, f32)) : OptTensor();
  g.dout = go.data_ptr(), g.dlast_state = fptr(gl);
  g.du = du.data_ptr(), g.ddelta = dd.data_ptr(), g.dz = dz.has_value() ? dz->data_ptr() : nullptr;
  g.dA = dA.data_ptr<float>(), g.dB = dB.data_ptr<float>(), g.dC = dC.data_ptr<float>();
  g.db_sb = c.B.sb, g.db_sg = c.B.sg, g.db_sn = c.B.sn, g.db_st = c.B.st;
  g.dc_sb = c.C.sb, g.dc_sg = c.C.sg, g.dc_sn = c.C.sn, g.dc_st = c.C.st;
  g.dD = fptr_mut(dD), g.ddt_bias = fptr_mut(db), g.dinitial_state = nullptr;
  if (c.nb * c.nd * c.nl > 0) run(ssm_selective_scan_bwd(&g, stream_of(c.u)));
  else du.zero_(), dd.zero_();
  auto cast = [](const OptTensor& grad, const OptTensor& src) { return grad.has_value() ? OptTensor(grad->to(src->scalar_type())) : OptTensor(); };
  return {du.to(u.scalar_type()), dd.to(delta.scalar_type()), dA.to(A.scalar_type()), fold_coeff_grad(dB, B.dim() == 4 ? B : dB).to(B.scalar_type()),
          fold_coeff_grad(dC, C.dim() == 4 ? C : dC).to(C.scalar_type()), cast(dD, D), cast(dz, z), cast(db, dt_bias)};
}

// ---------------------------------------------------------------------------------------------
// single-token state step
// ---------------------------------------------------------------------------------------------
struct StepCoeff {
  int groups;
  int64_t sb, sg, sn;
};
StepCoeff step_coeff(const char* name, const Tensor& p, int64_t nb, int64_t nd, int64_t nn) {
  if (p.dim() == 2) {
    TORCH_CHECK(p.size(0) == nd && p.size(1) == nn, name, " must have shape (D, N).");
    return {(int)nd, 0, nn, 1};
  }
  TORCH_CHECK(p.dim() == 3 && p.size(0) == nb, name, " must have shape (D, N), (B, D, N) or (B, G, N).");
  const int64_t g = p.size(1);
  TORCH_CHECK(p.size(2) == nn, name, " must have matching state dimension.");
  TORCH_CHECK(g > 0 && nd % g == 0, name, " group dimension must divide D.");
  return {(int)g, g * nn, nn, 1};
}

struct StepCtx {
  int64_t nb, nd, nn;
  Tensor x, dt, A, B, C;
  OptTensor z, D, bias;
  StepCoeff cb, cc;
  bool softplus;

  StepCtx(const Tensor& state, const Tensor& x_, const Tensor& dt_, const Tensor& A_, const Tensor& B_, const Tensor& C_, const OptTensor& D_,
          const OptTensor& z_, const OptTensor& bias_, bool softplus_)
      : softplus(softplus_) {
    TORCH_CHECK(state.dim() == 3, "state must have shape (B, D, N).");
    TORCH_CHECK(x_.dim() == 2 && dt_.dim() == 2, "x and dt must have shape (B, D).");
    nb = state.size(0), nd = state.size(1), nn = state.size(2);
    TORCH_CHECK(x_.size(0) == nb && x_.size(1) == nd && dt_.sizes() == x_.sizes(), "x and dt must match the first two dimensions of state.");
    TORCH_CHECK(A_.dim() == 2 && A_.size(0) == nd && A_.size(1) == nn, "A must have shape (D, N).");
    same_device(state, {&x_, &dt_, &A_, &B_, &C_});
    need_cuda(state, {&D_, &z_, &bias_});
    dtype_code(x_, "selective_state_step");
    cb = step_coeff("B", B_, nb, nd, nn), cc = step_coeff("C", C_, nb, nd, nn);
    B = B_.detach().contiguous(), C = C_.detach().contiguous();
    if (cb.groups != cc.groups || B.scalar_type() != C.scalar_type() || !io_dtype_ok(B)) {
      auto expand = [&](Tensor t, StepCoeff& sc) {  // bring to per-channel fp32 (B, D, N) / (D, N)
        t = t.to(at::kFloat);
        if (t.dim() == 3 && sc.groups != nd) t = t.repeat_interleave(nd / sc.groups, 1);
        sc = t.dim() == 2 ? StepCoeff{(int)nd, 0, nn, 1} : StepCoeff{(int)nd, nd * nn, nn, 1};
        return t.contiguous();
      };
      B = expand(B, cb), C = expand(C, cc);
    }
    if (D_.has_value()) TORCH_CHECK(D_->dim() == 1 && D_->size(0) == nd, "D must have shape (D,).");
    if (z_.has_value()) TORCH_CHECK(z_->sizes() == x_.sizes(), "z must have shape (B, D).");
    if (bias_.has_value()) TORCH_CHECK(bias_->dim() == 1 && bias_->size(0) == nd, "dt_bias must have shape (D,).");
    x = x_.detach().contiguous(), dt = like(dt_, x), A = f32c(A_), D = f32c(D_), bias = f32c(bias_);
    if (z_.has_value()) z = like(*z_, x);
  }

  void fill(ssm_step_args& a, Tensor& state32) const {
    a.batch = (int)nb, a.dim = (int)nd, a.nstate = (int)nn, a.io_dtype = dtype_code(x, "selective_state_step");
    a.bc_dtype = dtype_code(B, "selective_state_step B/C"), a.bc_groups = cb.groups, a.dt_softplus = softplus, a.param_heads = 0;
    a.state = state32.data_ptr<float>(), a.x = x.data_ptr(), a.dt = dt.data_ptr(), a.z = ptr(z), a.A = A.data_ptr<float>();
    a.Bm = B.data_ptr(), a.Cm = C.data_ptr();
    a.b_sb = cb.sb, a.b_sg = cb.sg, a.b_sn = cb.sn, a.c_sb = cc.sb, a.c_sg = cc.sg, a.c_sn = cc.sn;
    a.D = fptr(D), a.dt_bias = fptr(bias);
  }
};

Tensor selective_state_step(Tensor state, const Tensor& x, const Tensor& dt, const Tensor& A, const Tensor& B, const Tensor& C, const OptTensor& D,
                            const OptTensor& z, const OptTensor& dt_bias, bool softplus) {
  StepCtx c(state, x, dt, A, B, C, D, z, dt_bias, softplus);
  c10::cuda::CUDAGuard guard(state.device());
  const bool direct = state.scalar_type() == at::kFloat && state.is_contiguous();
  Tensor work = direct ? state.detach() : f32c(state);
  Tensor out = at::empty_like(c.x);
  ssm_step_args a{};
  c.fill(a, work);
  a.out = out.data_ptr();
  if (c.nb * c.nd > 0) run(ssm_selective_state_step(&a, stream_of(state)));
  if (!direct) state.detach().copy_(work);
  return out;
}

std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, OptTensor, OptTensor, OptTensor> selective_state_step_backward(
    const Tensor& grad_output, const OptTensor& grad_state, const Tensor& state, const Tensor& x, const Tensor& dt, const Tensor& A, const Tensor& B,
    const Tensor& C, const OptTensor& D, const OptTensor& z, const OptTensor& dt_bias, bool softplus) {
  StepCtx c(state, x, dt, A, B, C, D, z, dt_bias, softplus);
  c10::cuda::CUDAGuard guard(state.device());
  const auto f32 = c.x.options().dtype(at::kFloat);
  Tensor old = f32c(state);  // the state BEFORE the step
  Tensor go = like(grad_output, c.x);
  OptTensor gs = f32c(grad_state);
  Tensor dstate = at::empty({c.nb, c.nd, c.nn}, f32), dx = at::empty_like(c.x), ddt = at::empty_like(c.x);
  OptTensor dz = c.z.has_value() ? OptTensor(at::empty_like(c.x)) : OptTensor();
  Tensor dA = at::zeros({c.nd, c.nn}, f32), dB = at::zeros(c.B.sizes(), f32), dC = at::zeros(c.C.sizes(), f32);
  OptTensor dD = c.D.has_value() ? OptTensor(at::zeros({c.nd}, f32)) : OptTensor();
  OptTensor db = c.bias.has_value() ? OptTensor(at::zeros({c.nd}, f32)) : OptTensor();
  ssm_step_bwd_args g{};
  c.fill(g.fwd, old);
  g.dout = go.data_ptr(), g.dnew_state = fptr(gs), g.dstate = dstate.data_ptr<float>();
  g.dx = dx.data_ptr(), g.ddt = ddt.data_ptr(), g.dz = dz.has_value() ? dz->data_ptr() : nullptr;
  g.dA = dA.data_ptr<float>(), g.dB = dB.data_ptr<float>(), g.dC = dC.data_ptr<float>(), g.dD = fptr_mut(dD), g.ddt_bias = fptr_mut(db);
  if (c.nb * c.nd > 0) run(ssm_selective_state_step_bwd(&g, stream_of(state)));
  else dstate.zero_();
  auto fold = [&](Tensor grad, const Tensor& src) {
    if (grad.sizes() != src.sizes()) {  // grouped (B, G, N) had been expanded to (B, D, N)
      const int64_t rep = grad.size(1) / src.size(1);
      grad = grad.view({src.size(0), src.size(1), rep, src.size(2)}).sum(2);
    }
    return grad.to(src.scalar_type());
  };
  auto cast = [](const OptTensor& grad, const OptTensor& src) { return grad.has_value() ? OptTensor(grad->to(src->scalar_type())) : OptTensor(); };
  return {dstate.to(state.scalar_type()), dx, ddt.to(dt.scalar_type()), dA.to(A.scalar_type()), fold(dB, B), fold(dC, C), cast(dD, D), cast(dz, z),
          cast(db, dt_bias)};
}

// ---------------------------------------------------------------------------------------------
// element-wise chunked recurrence
// ---------------------------------------------------------------------------------------------
enum class Kind { H, HP, BHP, BLH, BLHP };
void set_bc4(ssm_bcast4& d, const OptTensor& t, Kind k) {
  d.ptr = nullptr, d.sb = d.st = d.sh = d.sq = 0;
  if (!t.has_value()) return;
  d.ptr = t->data_ptr();
  switch (k) {
    case Kind::H: d.sh = 1; break;
    case Kind::HP: d.sh = t->size(1), d.sq = 1; break;
    case Kind::BHP: d.sb = t->size(1) * t->size(2), d.sh = t->size(2), d.sq = 1; break;
    case Kind::BLH: d.sb = t->size(1) * t->size(2), d.st = t->size(2), d.sh = 1; break;
    case Kind::BLHP: d.sb = t->size(1) * t->size(2) * t->size(3), d.st = t->size(2) * t->size(3), d.sh = t->size(3), d.sq = 1; break;
  }
}

struct ChunkCtx {
  int64_t nb, nl, nh, np;
  int chunk;
  Tensor X, dt;
  OptTensor A, B, C, D, z, init, lens;
  Kind kA, kB, kC, kD = Kind::H, kz = Kind::BLH;
  int par;

  ChunkCtx(const Tensor& X_, const Tensor& dt_, const Tensor& A_, const Tensor& B_, const Tensor& C_, int64_t chunk_size, const OptTensor& D_,
           const OptTensor& z_, const OptTensor& seq_lens, const OptTensor& cu_seqlens, const OptTensor& init_) {
    TORCH_CHECK(X_.dim() == 4, "X must have shape (B, L, H, P).");
    TORCH_CHECK(dt_.dim() == 3, "dt must have shape (B, L, H).");
    nb = X_.size(0), nl = X_.size(1), nh = X_.size(2), np = X_.size(3);
    TORCH_CHECK(dt_.size(0) == nb && dt_.size(1) == nl && dt_.size(2) == nh, "dt must align with (B, L, H).");
    TORCH_CHECK(chunk_size > 0, "chunk_size must be positive.");
    chunk = (int)std::min<int64_t>(chunk_size, 1 << 30);
    same_device(X_, {&dt_, &A_, &B_, &C_});
    need_cuda(X_, {&D_, &z_, &init_});
    dtype_code(X_, "ssd_chunk_scan");
    X = X_.detach().contiguous(), dt = like(dt_, X);
    if (A_.dim() == 1) {
      TORCH_CHECK(A_.size(0) == nh, "A must have shape (H,) when 1-D.");
      kA = Kind::H;
    } else {
      TORCH_CHECK(A_.dim() == 2, "A must be 1-D or 2-D.");
      TORCH_CHECK(A_.size(0) == nh && A_.size(1) == np, "A must have shape (H, P) when 2-D.");
      kA = Kind::HP;
    }
    A = f32c(A_);
    auto coeff = [&](const char* name, const Tensor& p) {
      if (p.dim() == 2) {
        TORCH_CHECK(p.size(0) == nh && p.size(1) == np, name, " must have shape (H, P).");
        return Kind::HP;
      }
      if (p.dim() == 3) {
        TORCH_CHECK(p.size(0) == nb && p.size(1) == nh && p.size(2) == np, name, " must be (B, H, P) when 3-D.");
        return Kind::BHP;
      }
      TORCH_CHECK(p.dim() == 4, "Unsupported rank for ", name, ".");
      TORCH_CHECK(p.sizes() == X_.sizes(), name, " must have shape (B, L, H, P) when 4-D.");
      return Kind::BLHP;
    };
    kB = coeff("B", B_), kC = coeff("C", C_);
    if (D_.has_value()) {
      if (D_->dim() == 1 && D_->size(0) == nh) kD = Kind::H;
      else if (D_->dim() == 2 && D_->size(0) == nh && D_->size(1) == np) kD = Kind::HP;
      else TORCH_CHECK(false, "D must have shape (H,) or (H, P).");
    }
    if (z_.has_value()) {
      if (z_->dim() == 3 && z_->size(0) == nb && z_->size(1) == nl && z_->size(2) == nh) kz = Kind::BLH;
      else if (z_->dim() == 4 && z_->sizes() == X_.sizes()) kz = Kind::BLHP;
      else TORCH_CHECK(false, "z must have shape (B, L, H) or (B, L, H, P).");
    }
    if (init_.has_value()) TORCH_CHECK(init_->dim() == 3 && init_->size(0) == nb && init_->size(1) == nh && init_->size(2) == np, "initial_states must have shape (B, H, P).");
    // B, C and z share one run-time element type inside the kernel
    at::ScalarType pd = X_.scalar_type();  // the kernels take X's element type or fp32
    const bool same = B_.scalar_type() == pd && C_.scalar_type() == pd && (!z_.has_value() || z_->scalar_type() == pd);
    if (!same) pd = at::kFloat;
    par = pd == at::kFloat ? SSM_F32 : pd == at::kBFloat16 ? SSM_BF16 : SSM_F16;
    B = B_.detach().to(pd).contiguous(), C = C_.detach().to(pd).contiguous();
    if (z_.has_value()) z = z_->detach().to(pd).contiguous();
    D = f32c(D_), init = f32c(init_);
    // valid lengths per row, on the device (reference.py:413-428); never copied to the host
    if (cu_seqlens.has_value()) {
      TORCH_CHECK(cu_seqlens->numel() == nb + 1, "cu_seqlens must have length B + 1.");
      Tensor cu = cu_seqlens->to(X.device(), at::kLong);
      lens = (cu.slice(0, 1) - cu.slice(0, 0, nb)).contiguous();
    } else if (seq_lens.has_value()) {
      TORCH_CHECK(seq_lens->numel() == nb, "seq_lens must have length B.");
      lens = seq_lens->to(X.device(), at::kLong).contiguous();
    }
  }

  void fill(ssm_chunk_args& a) const {
    a.batch = (int)nb, a.len = (int)nl, a.heads = (int)nh, a.proj = (int)np;
    a.io_dtype = dtype_code(X, "ssd_chunk_scan"), a.par_dtype = par, a.chunk_size = chunk;
    a.X = X.data_ptr(), a.dt = dt.data_ptr();
    set_bc4(a.A, A, kA), set_bc4(a.Bm, B, kB), set_bc4(a.Cm, C, kC), set_bc4(a.D, D, kD), set_bc4(a.z, z, kz), set_bc4(a.initial, init, Kind::BHP);
    a.seq_lens = lens.has_value() ? lens->data_ptr<int64_t>() : nullptr;
  }
};

Tensor ssd_chunk_scan(const Tensor& X, const Tensor& dt, const Tensor& A, const Tensor& B, const Tensor& C, int64_t chunk_size, const OptTensor& D,
                      const OptTensor& z, const OptTensor& seq_lens, const OptTensor& cu_seqlens, const OptTensor& initial_states) {
  ChunkCtx c(X, dt, A, B, C, chunk_size, D, z, seq_lens, cu_seqlens, initial_states);
  c10::cuda::CUDAGuard guard(c.X.device());
  Tensor Y = at::empty_like(c.X);
  const int64_t n = ssm_chunk_scan_scratch_floats((int)c.nb, (int)c.nl, (int)c.nh, (int)c.np, c.chunk);
  Tensor scratch = at::empty({std::max<int64_t>(n, 1)}, c.X.options().dtype(at::kFloat));
  ssm_chunk_args a{};
  c.fill(a);
  a.Y = Y.data_ptr(), a.final_state = nullptr, a.scratch = scratch.data_ptr<float>();
  run(ssm_chunk_scan_fwd(&a, stream_of(c.X)));
  return Y;
}

std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor, OptTensor, OptTensor, OptTensor> ssd_chunk_scan_backward(
    const Tensor& grad_output, const Tensor& X, const Tensor& dt, const Tensor& A, const Tensor& B, const Tensor& C, int64_t chunk_size,
    const OptTensor& D, const OptTensor& z, const OptTensor& seq_lens, const OptTensor& cu_seqlens, const OptTensor& initial_states) {
  ChunkCtx c(X, dt, A, B, C, chunk_size, D, z, seq_lens, cu_seqlens, initial_states);
  c10::cuda::CUDAGuard guard(c.X.device());
  TORCH_CHECK(grad_output.sizes() == c.X.sizes(), "grad_output must have the shape of X.");
  const auto f32 = c.X.options().dtype(at::kFloat);
  auto zeros_like = [&](const OptTensor& t) { return t.has_value() ? OptTensor(at::zeros(t->sizes(), f32)) : OptTensor(); };
  Tensor dX = at::empty_like(c.X), ddt = at::zeros({c.nb, c.nl, c.nh}, f32);
  // per-token B / C / z: the kernel writes their gradients in the tensor's own type (no zero-fill, no fp32 copy to convert)
  int typed = 0;
  auto own = [&](const OptTensor& t, Kind k, int bit) {
    if (!t.has_value() || k != Kind::BLHP) return zeros_like(t);
    typed |= bit;
    return OptTensor(at::empty_like(*t));
  };
  OptTensor dA = zeros_like(c.A), dB = own(c.B, c.kB, 1), dC = own(c.C, c.kC, 2), dD = zeros_like(c.D), dz = own(c.z, c.kz, 4), dI = zeros_like(c.init);
  Tensor hist = at::empty({c.nb, std::max<int64_t>(c.nl, 1), c.nh, c.np}, f32);
  Tensor gy = like(grad_output, c.X);
  ssm_chunk_bwd_args g{};
  c.fill(g.fwd);
  g.fwd.typed_grads = typed;
  Tensor scratch = at::empty({std::max<int64_t>(1, ssm_chunk_scan_bwd_scratch_floats((int)c.nb, (int)c.nl, (int)c.nh, (int)c.np, c.chunk))}, f32);
  g.dY = gy.data_ptr(), g.dX = dX.data_ptr(), g.ddt = ddt.data_ptr<float>(), g.history = hist.data_ptr<float>();
  g.scratch = scratch.data_ptr<float>();
  set_bc4(g.dA, dA, c.kA), set_bc4(g.dB, dB, c.kB), set_bc4(g.dC, dC, c.kC), set_bc4(g.dD, dD, c.kD), set_bc4(g.dz, dz, c.kz),
      set_bc4(g.dinitial, dI, Kind::BHP);
  run(ssm_chunk_scan_bwd(&g, stream_of(c.X)));
  auto cast = [](const OptTensor& grad, const OptTensor& src) { return grad.has_value() ? OptTensor(grad->to(src->scalar_type())) : OptTensor(); };
  return {dX, ddt.to(dt.scalar_type()), dA->to(A.scalar_type()), dB->to(B.scalar_type()), dC->to(C.scalar_type()), cast(dD, D), cast(dz, z),
          cast(dI, initial_states)};
}

// ---------------------------------------------------------------------------------------------
// depthwise causal conv
// ---------------------------------------------------------------------------------------------
struct ConvCtx {
  bool first, silu;
  int64_t nb, nc, nl, k;
  Tensor x, w;
  OptTensor b;

  ConvCtx(const Tensor& x_, const Tensor& weight, const OptTensor& bias, const std::string& activation) {
    TORCH_CHECK(x_.dim() == 3, "x must have shape (B, C, L) or (B, L, C).");
    nc = weight.size(0);
    if (x_.size(1) == nc) first = true;
    else if (x_.size(2) == nc) first = false;
    else TORCH_CHECK(false, "weight channel dimension must match x.");
    Tensor w2;
    if (weight.dim() == 3) {
      TORCH_CHECK(weight.size(1) == 1, "Expected depthwise weights with shape (C, 1, K).");
      w2 = weight.select(1, 0);
    } else {
      TORCH_CHECK(weight.dim() == 2, "weight must have 2 or 3 dimensions.");
      w2 = weight;
    }
    if (bias.has_value()) TORCH_CHECK(bias->dim() == 1 && bias->size(0) == nc, "bias must have shape (C,).");
    std::string act = activation;
    for (auto& ch : act) ch = (char)std::tolower((unsigned char)ch);
    TORCH_CHECK(act == "silu" || act == "swish" || act == "identity" || act == "none", "Unsupported activation '", activation, "'.");
    silu = act == "silu" || act == "swish";
    k = w2.size(1);
    TORCH_CHECK(k >= 1 && k <= 8, "dw_causal_conv: kernel width must be in [1, 8].");
    same_device(x_, {&weight});
    need_cuda(x_, {&bias});
    dtype_code(x_, "dw_causal_conv");
    x = x_.detach().contiguous(), w = f32c(w2), b = f32c(bias);
    nb = x_.size(0), nl = first ? x_.size(2) : x_.size(1);
  }
  void fill(ssm_conv_args& a) const {
    a.batch = (int)nb, a.channels = (int)nc, a.len = (int)nl, a.width = (int)k;
    a.io_dtype = dtype_code(x, "dw_causal_conv"), a.channels_first = first, a.silu = silu;
    a.x = x.data_ptr(), a.weight = w.data_ptr<float>(), a.bias = fptr(b), a.halo = nullptr;
    a.row_sb = nc * nl, a.row_sc = nl;
  }
};

Tensor dw_causal_conv(const Tensor& x, const Tensor& weight, const OptTensor& bias, const std::string& activation) {
  ConvCtx c(x, weight, bias, activation);
  c10::cuda::CUDAGuard guard(c.x.device());
  Tensor y = at::empty_like(c.x);
  ssm_conv_args a{};
  c.fill(a);
  a.y = y.data_ptr();
  run(ssm_dw_causal_conv_fwd(&a, stream_of(c.x)));
  return y;
}

std::tuple<Tensor, Tensor, OptTensor> dw_causal_conv_backward(const Tensor& grad_output, const Tensor& x, const Tensor& weight, const OptTensor& bias,
                                                             const std::string& activation) {
  ConvCtx c(x, weight, bias, activation);
  c10::cuda::CUDAGuard guard(c.x.device());
  TORCH_CHECK(grad_output.sizes() == c.x.sizes(), "grad_output must have the shape of x.");
  const auto f32 = c.x.options().dtype(at::kFloat);
  Tensor dx = at::empty_like(c.x), dw = at::zeros({c.nc, c.k}, f32);
  OptTensor db = c.b.has_value() ? OptTensor(at::zeros({c.nc}, f32)) : OptTensor();
  Tensor go = like(grad_output, c.x);
  ssm_conv_bwd_args g{};
  c.fill(g.fwd);
  g.dy = go.data_ptr(), g.dx = dx.data_ptr(), g.dweight = dw.data_ptr<float>(), g.dbias = fptr_mut(db);
  run(ssm_dw_causal_conv_bwd(&g, stream_of(c.x)));
  return {dx, dw.view(weight.sizes()).to(weight.scalar_type()), db.has_value() ? OptTensor(db->to(bias->scalar_type())) : OptTensor()};
}

// ---------------------------------------------------------------------------------------------
// fused residual add + LayerNorm / RMSNorm
// ---------------------------------------------------------------------------------------------
struct NormCtx {
  Tensor x, w;
  OptTensor b, res;
  bool is_rms, prenorm;
  double eps;

  NormCtx(const Tensor& x_, const Tensor& weight, const OptTensor& bias, const OptTensor& residual, bool is_rms_, double eps_, bool prenorm_)
      : is_rms(is_rms_), prenorm(prenorm_), eps(eps_) {
    TORCH_CHECK(x_.dim() == 3, "x must have shape (B, L, D).");
    TORCH_CHECK(weight.dim() == 1 && weight.size(0) == x_.size(2), "weight must match the last dimension of x.");
    if (bias.has_value()) TORCH_CHECK(bias->dim() == 1 && bias->size(0) == x_.size(2), "bias must match the last dimension of x.");
    if (residual.has_value()) TORCH_CHECK(residual->sizes() == x_.sizes(), "residual must match the shape of x.");
    same_device(x_, {&weight});
    need_cuda(x_, {&bias, &residual});
    dtype_code(x_, "fused_layer_norm");
    x = x_.detach().contiguous(), w = f32c(weight), b = f32c(bias);
    if (residual.has_value()) {
      dtype_code(*residual, "fused_layer_norm residual");
      res = residual->detach().contiguous();
    }
  }
  void fill(ssm_norm_args& a) const {
    a.rows = x.size(0) * x.size(1), a.hidden = (int)x.size(2);
    a.io_dtype = dtype_code(x, "fused_layer_norm"), a.res_dtype = res.has_value() ? dtype_code(*res, "fused_layer_norm residual") : 0;
    a.is_rms = is_rms, a.prenorm = prenorm, a.eps = (float)eps;
    a.x = x.data_ptr(), a.residual = ptr(res), a.weight = w.data_ptr<float>(), a.bias = fptr(b);
  }
};

Tensor fused_layer_norm(const Tensor& x, const Tensor& weight, const OptTensor& bias, const OptTensor& residual, bool is_rms, double eps, bool prenorm,
                        bool residual_in_fp32) {
  (void)residual_in_fp32;  // all arithmetic is fp32 for fp32 / bf16 / fp16 inputs, whatever this flag says
  NormCtx c(x, weight, bias, residual, is_rms, eps, prenorm);
  c10::cuda::CUDAGuard guard(c.x.device());
  Tensor y = at::empty_like(c.x);
  ssm_norm_args a{};
  c.fill(a);
  a.y = y.data_ptr(), a.residual_out = nullptr;
  run(ssm_fused_add_norm_fwd(&a, stream_of(c.x)));
  return y;
}

std::tuple<Tensor, Tensor, Tensor, Tensor> fused_layer_norm_backward(const Tensor& grad_output, const Tensor& x, const Tensor& weight, const OptTensor& bias,
                                                                     const OptTensor& residual, bool is_rms, double eps, bool prenorm,
                                                                     bool residual_in_fp32) {
  (void)residual_in_fp32;
  NormCtx c(x, weight, bias, residual, is_rms, eps, prenorm);
  c10::cuda::CUDAGuard guard(c.x.device());
  TORCH_CHECK(grad_output.sizes() == c.x.sizes(), "grad_output must have the shape of x.");
  const auto f32 = c.x.options().dtype(at::kFloat);
  const int64_t rows = c.x.size(0) * c.x.size(1), hidden = c.x.size(2);
  Tensor dx = at::empty_like(c.x), dw = at::empty({hidden}, f32);
  Tensor db = c.b.has_value() ? at::empty({hidden}, f32) : at::empty({0}, c.x.options());
  Tensor dres = c.res.has_value() ? at::empty_like(*c.res) : at::empty({0}, c.x.options());
  Tensor partial = at::empty({ssm_norm_bwd_scratch_floats(rows, (int)hidden)}, f32);
  Tensor go = like(grad_output, c.x);
  ssm_norm_bwd_args g{};
  c.fill(g.fwd);
  g.dy = go.data_ptr(), g.dx = dx.data_ptr(), g.dresidual = c.res.has_value() ? dres.data_ptr() : nullptr;
  g.dweight = dw.data_ptr<float>(), g.dbias = c.b.has_value() ? db.data_ptr<float>() : nullptr, g.partial = partial.data_ptr<float>();
  g.dresidual_out = nullptr;
  run(ssm_fused_add_norm_bwd(&g, stream_of(c.x)));
  // absent inputs give empty tensors, as upstream's extension does
  return {dx, dw.to(weight.scalar_type()), c.b.has_value() ? db.to(bias->scalar_type()) : db, dres};
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  namespace py = pybind11;
  m.doc() = "ssm.ops CUDA backend for B200 (sm_100a): the ten entry points of upstream's compiled extension, on libssm_b200";
  m.def("abi_version", []() { return ssm_b200_abi_version(); });
  m.def("selective_scan", &selective_scan, py::arg("u"), py::arg("delta"), py::arg("A"), py::arg("B"), py::arg("C"), py::arg("D") = c10::nullopt,
        py::arg("z") = c10::nullopt, py::arg("dt_bias") = c10::nullopt, py::arg("softplus") = false, py::arg("return_last_state") = false);
  m.def("selective_scan_backward", &selective_scan_backward, py::arg("grad_output"), py::arg("grad_last_state") = c10::nullopt, py::arg("u"),
        py::arg("delta"), py::arg("A"), py::arg("B"), py::arg("C"), py::arg("D") = c10::nullopt, py::arg("z") = c10::nullopt,
        py::arg("dt_bias") = c10::nullopt, py::arg("softplus") = false, py::arg("forward_output") = c10::nullopt, py::arg("cache") = c10::nullopt);
  m.def("selective_state_step", &selective_state_step, py::arg("state"), py::arg("x"), py::arg("dt"), py::arg("A"), py::arg("B"), py::arg("C"),
        py::arg("D") = c10::nullopt, py::arg("z") = c10::nullopt, py::arg("dt_bias") = c10::nullopt, py::arg("softplus") = true);
  m.def("selective_state_step_backward", &selective_state_step_backward, py::arg("grad_output"), py::arg("grad_state") = c10::nullopt, py::arg("state"),
        py::arg("x"), py::arg("dt"), py::arg("A"), py::arg("B"), py::arg("C"), py::arg("D") = c10::nullopt, py::arg("z") = c10::nullopt,
        py::arg("dt_bias") = c10::nullopt, py::arg("softplus") = true);
  m.def("ssd_chunk_scan", &ssd_chunk_scan, py::arg("X"), py::arg("dt"), py::arg("A"), py::arg("B"), py::arg("C"), py::arg("chunk_size"),
        py::arg("D") = c10::nullopt, py::arg("z") = c10::nullopt, py::arg("seq_lens") = c10::nullopt, py::arg("cu_seqlens") = c10::nullopt,
        py::arg("initial_states") = c10::nullopt);
  m.def("ssd_chunk_scan_backward", &ssd_chunk_scan_backward, py::arg("grad_output"), py::arg("X"), py::arg("dt"), py::arg("A"), py::arg("B"),
        py::arg("C"), py::arg("chunk_size"), py::arg("D") = c10::nullopt, py::arg("z") = c10::nullopt, py::arg("seq_lens") = c10::nullopt,
        py::arg("cu_seqlens") = c10::nullopt, py::arg("initial_states") = c10::nullopt);
  m.def("dw_causal_conv", &dw_causal_conv, py::arg("x"), py::arg("weight"), py::arg("bias") = c10::nullopt, py::arg("activation") = "silu");
  m.def("dw_causal_conv_backward", &dw_causal_conv_backward, py::arg("grad_output"), py::arg("x"), py::arg("weight"), py::arg("bias") = c10::nullopt,
        py::arg("activation") = "silu");
  m.def("fused_layer_norm", &fused_layer_norm, py::arg("x"), py::arg("weight"), py::arg("bias") = c10::nullopt, py::arg("residual") = c10::nullopt,
        py::arg("is_rms") = false, py::arg("eps") = 1e-5, py::arg("prenorm") = true, py::arg("residual_in_fp32") = true);
  m.def("fused_layer_norm_backward", &fused_layer_norm_backward, py::arg("grad_output"), py::arg("x"), py::arg("weight"), py::arg("bias") = c10::nullopt,
        py::arg("residual") = c10::nullopt, py::arg("is_rms") = false, py::arg("eps") = 1e-5, py::arg("prenorm") = true,
        py::arg("residual_in_fp32") = true);
}
