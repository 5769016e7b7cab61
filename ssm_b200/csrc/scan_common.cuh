// Lane layout and tile staging shared by the selective-scan forward and backward kernels.
//
// A warp works on RPW = 32/LPR channel rows of one batch element; the LPR lanes of a row
// each keep NS of the row's states in registers (NP = NS*LPR >= nstate, padded states have
// A = B = C = 0).  Time is walked sequentially in tiles of TL steps, so the recurrence
// itself needs no parallel prefix: parallelism comes from rows x states.  Per tile the
// warp stages its rows' inputs in shared memory as fp32; in "shared B/C" mode the CTA also
// stages one (NP x TL) tile of B and of C that all of its rows use (rows of one group).
#pragma once

#include "common.cuh"

namespace ssmb {

constexpr int kScanWarps = 4;
constexpr int kScanCkpt = 32;  // checkpoint interval in time steps

template <int NS_, int LPR_>
struct ScanShape {
  static constexpr int NS = NS_;
  static constexpr int LPR = LPR_;
  static constexpr int NP = NS * LPR;
  static constexpr int RPW = 32 / LPR;
  static constexpr int ROWS = kScanWarps * RPW;
  static constexpr int TB = LPR > 4 ? LPR : 4;  // time steps per reduce-scatter batch
};

// Flags computed on the host.
struct ScanFlags {
  int io_vec;      // u/delta/z/out rows start 16-byte aligned and len % (16/sizeof(T)) == 0
  int bc_vec;      // B and C: unit time stride and every (b, g, n) row 16-byte aligned
  int shared_bc;   // all rows of a CTA belong to one B/C group
  int rows_per_group;
};

// Stage one (N x TL) tile of a B/C-like operand into shared memory as fp32, zero beyond len.
template <typename TB_, int TL, int TLP>
__device__ __forceinline__ void stage_bc_typed(float* __restrict__ dst, const TB_* __restrict__ base, int64_t sn, int64_t st,
                                               int nstate, int t0, int len, bool vec, int tid, int nthreads) {
  constexpr int V = 16 / sizeof(TB_);
  if (vec) {
    constexpr int CH = TL / V;
    for (int c = tid; c < nstate * CH; c += nthreads) {
      const int n = c / CH, ch = c % CH;
      const int t = t0 + ch * V;
      float f[V];
      if (t < len) {
        Vec16<TB_> v;
        v.load(base + (int64_t)n * sn + t);
        v.unpack(f);
      } else {
#pragma unroll
        for (int i = 0; i < V; ++i) f[i] = 0.f;
      }
      float* d = dst + n * TLP + ch * V;
#pragma unroll
      for (int i = 0; i < V; i += 4) *reinterpret_cast<float4*>(d + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
    }
  } else {
    for (int i = tid; i < nstate * TL; i += nthreads) {
      const int n = i / TL, tt = i % TL;
      const int t = t0 + tt;
      dst[n * TLP + tt] = t < len ? to_f<TB_>(__ldg(base + (int64_t)n * sn + (int64_t)t * st)) : 0.f;
    }
  }
}

template <int TL, int TLP>
__device__ __forceinline__ void stage_bc(float* dst, const void* base, int dtype, int64_t sn, int64_t st, int nstate, int t0,
                                         int len, bool vec, int tid, int nthreads) {
  if (dtype == SSM_F32)
    stage_bc_typed<float, TL, TLP>(dst, reinterpret_cast<const float*>(base), sn, st, nstate, t0, len, vec, tid, nthreads);
  else if (dtype == SSM_BF16)
    stage_bc_typed<__nv_bfloat16, TL, TLP>(dst, reinterpret_cast<const __nv_bfloat16*>(base), sn, st, nstate, t0, len, vec, tid,
                                          nthreads);
  else
    stage_bc_typed<__half, TL, TLP>(dst, reinterpret_cast<const __half*>(base), sn, st, nstate, t0, len, vec, tid, nthreads);
}

// Element offset of the start of B/C data for batch b and channel d.
__device__ __forceinline__ int64_t bc_row_offset(int b, int d, int rows_per_group, int64_t sb, int64_t sg) {
  return (int64_t)b * sb + (int64_t)(d / rows_per_group) * sg;
}

}  // namespace ssmb
