// Shared device/host helpers for the sm_100a operator kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>

#include "../../include/ssm_b200.h"

namespace ssmb {

// ---------------------------------------------------------------------------------------
// host: error reporting
// ---------------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
inline int fail(int code, const char* what) {
  set_error("%s", what);
  return code;
}
#define SSM_REQUIRE(cond, code, what) \
  do {                                \
    if (!(cond)) return ::ssmb::fail((code), (what)); \
  } while (0)

// double-precision variants (fp64_ops.cu), reached from the ordinary entry points when io_dtype == SSM_F64
int f64_scan_fwd(const ssm_scan_fwd_args& a, cudaStream_t st);
int f64_scan_bwd(const ssm_scan_bwd_args& g, cudaStream_t st);
int f64_step(const ssm_step_bwd_args& g, bool backward, cudaStream_t st);
int f64_chunk(const ssm_chunk_bwd_args& g, bool backward, cudaStream_t st);
int f64_conv(const ssm_conv_bwd_args& g, bool backward, cudaStream_t st);
int f64_norm(const ssm_norm_bwd_args& g, bool backward, cudaStream_t st);

inline int launch_status(const char* kernel) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: %s", kernel, cudaGetErrorString(e));
    return (int)e;
  }
  return SSM_OK;
}

inline bool valid_dtype(int d) { return d == SSM_F32 || d == SSM_BF16 || d == SSM_F16; }
inline int dtype_size(int d) { return d == SSM_F32 ? 4 : 2; }
inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ---------------------------------------------------------------------------------------
// device: scalar conversion
// ---------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

// Load element i of an array whose element type is given at run time.
__device__ __forceinline__ float load_dyn(const void* base, int64_t i, int dtype) {
  if (dtype == SSM_F32) return __ldg(reinterpret_cast<const float*>(base) + i);
  if (dtype == SSM_BF16) return __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16*>(base) + i));
  return __half2float(__ldg(reinterpret_cast<const __half*>(base) + i));
}
__device__ __forceinline__ void store_dyn(void* base, int64_t i, int dtype, float v) {
  if (dtype == SSM_F32) reinterpret_cast<float*>(base)[i] = v;
  else if (dtype == SSM_BF16) reinterpret_cast<__nv_bfloat16*>(base)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(base)[i] = __float2half_rn(v);
}

// ---------------------------------------------------------------------------------------
// device: 16-byte vectors of T  (4 x fp32 or 8 x 16-bit)
// ---------------------------------------------------------------------------------------
template <typename T>
struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  uint4 raw;
  __device__ __forceinline__ void load(const T* p) { raw = __ldg(reinterpret_cast<const uint4*>(p)); }
  __device__ __forceinline__ void load_stream(const T* p) { raw = __ldcs(reinterpret_cast<const uint4*>(p)); }
  __device__ __forceinline__ void store(T* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  __device__ __forceinline__ void store_stream(T* p) const { __stcs(reinterpret_cast<uint4*>(p), raw); }
  __device__ __forceinline__ void unpack(float (&f)[N]) const {
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < N; ++i) f[i] = to_f<T>(e[i]);
  }
  __device__ __forceinline__ void pack(const float (&f)[N]) {
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < N; ++i) e[i] = from_f<T>(f[i]);
  }
};

// ---------------------------------------------------------------------------------------
// device: math
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float exp_fast(float x) { return ex2_approx(x * kLog2e); }
// torch.nn.functional.softplus with its defaults: identity above 20, log1p(exp(x)) below.
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float lg2_approx(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// softplus(x) = max(x, 0) + log1p(exp(-|x|)) on the special-function unit.  For small
// t = exp(-|x|) the series t - t^2/2 + t^3/3 - t^4/4 replaces log(1 + t), whose argument would lose
// t's low bits; relative error stays below 4e-6 over the whole range.  Above the switch point
// of torch.nn.functional.softplus (20) the correction is below half an ulp of x, so the
// result equals x there as well.
__device__ __forceinline__ float softplus_fast(float x) {
  const float t = ex2_approx(-fabsf(x) * kLog2e);
  const float series = t * fmaf(t, fmaf(t, fmaf(t, -0.25f, 0.33333334f), -0.5f), 1.f);
  const float l = t < 0.0625f ? series : lg2_approx(1.f + t) * kLn2;
  return fmaxf(x, 0.f) + l;
}
// softplus for kernels whose inputs and outputs are 16-bit: log2(1 + 2^(x log2 e)) ln 2 on the special-function unit, no
// series for small arguments.  The absolute error is that of forming 1 + t in fp32 (6e-8), i.e. a relative error of
// 6e-8 / softplus(x): below the spacing of bf16 / fp16 values down to softplus(x) = 1e-5.
__device__ __forceinline__ float softplus_half_io(float x) {
  const float t = ex2_approx(fminf(x, 88.f) * kLog2e);
  return x > 20.f ? x : lg2_approx(1.f + t) * kLn2;
}
// 1 - exp(-x) for x >= 0 without cancellation for small x (it is sigmoid(pre) when
// x = softplus(pre), i.e. the derivative of softplus).
__device__ __forceinline__ float one_minus_exp_neg(float x) {
  const float series = x * fmaf(x, fmaf(x, fmaf(x, -0.041666668f, 0.16666667f), -0.5f), 1.f);
  return x < 0.0625f ? series : 1.f - ex2_approx(-x * kLog2e);
}
// SiLU through the special-function unit: x * rcp(1 + 2^(-x*log2e)); relative error ~1e-6.
__device__ __forceinline__ float silu_fast(float x) { return x * rcp_approx(1.f + ex2_approx(-x * kLog2e)); }
__device__ __forceinline__ float sigmoid_fast(float x) { return rcp_approx(1.f + ex2_approx(-x * kLog2e)); }
// silu for results that are rounded to 16 bits: x sigmoid(x) = h (1 + tanh(h)), h = x / 2, on the hardware tanh (relative
// error about 2^-11, one special-function instruction instead of two)
__device__ __forceinline__ float silu_half_io(float x) {
  const float h = 0.5f * x;
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(h));
  return fmaf(h, t, h);
}
// d/dx silu for gradients that are rounded to 16 bits: sigmoid(x) = 0.5 + 0.5 tanh(x / 2) on the hardware tanh (one
// special-function instruction instead of two)
__device__ __forceinline__ float silu_grad_half_io(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  const float s = fmaf(0.5f, t, 0.5f);
  return fmaf(x * s, 1.f - s, s);
}
__device__ __forceinline__ float silu_grad_fast(float x) {
  const float s = sigmoid_fast(x);
  return s * (1.f + x * (1.f - s));
}
// d/dx softplus(x) with the same switch point.
__device__ __forceinline__ float softplus_grad_f(float x) { return x > 20.f ? 1.f : sigmoid_f(x); }

// ---------------------------------------------------------------------------------------
// device: reduce-scatter over a group of LANES lanes whose lane ids differ in the bits
// [log2(STRIDE), log2(STRIDE*LANES)).  On entry every lane holds COUNT partial sums
// (COUNT a multiple of LANES).  On exit lane with group index g (= (lane / STRIDE) % LANES)
// holds, in p[0 .. COUNT/LANES), the group-wide totals of entries
// g*(COUNT/LANES) + i.  Costs COUNT*(1-1/LANES) shuffles instead of COUNT*log2(LANES).
// ---------------------------------------------------------------------------------------
template <int LANES, int STRIDE, int COUNT>
__device__ __forceinline__ void reduce_scatter(float (&p)[COUNT], int lane) {
  static_assert(COUNT % LANES == 0, "COUNT must be a multiple of LANES");
#pragma unroll
  for (int off = LANES / 2, len = COUNT / 2; off >= 1; off >>= 1, len >>= 1) {
    const bool upper = (lane & (off * STRIDE)) != 0;
#pragma unroll
    for (int i = 0; i < len; ++i) {
      const float send = upper ? p[i] : p[i + len];
      const float keep = upper ? p[i + len] : p[i];
      p[i] = keep + __shfl_xor_sync(0xffffffffu, send, off * STRIDE);
    }
  }
}

// all-reduce (sum) over the same kind of lane group
template <int LANES, int STRIDE>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int off = LANES / 2; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off * STRIDE);
  return v;
}

__device__ __forceinline__ float warp_sum(float v) { return group_sum<32, 1>(v); }

}  // namespace ssmb
