// Lane layout and tile staging shared by the selective-scan forward and backward kernels.
//
// A warp works on RPW = 32/LPR channel rows of one batch element; the LPR lanes of a row
// each keep NS consecutive states of the row in registers (NP = NS*LPR >= nstate, padded
// states have A = B = C = 0).  Time is walked sequentially in tiles of TL steps, so the
// recurrence itself needs no parallel prefix: parallelism comes from rows x states.
//
// Per tile the raw inputs (u, delta, z, ... rows of the warp; one B and one C tile per CTA
// when all of its rows share a B/C group) are copied global -> shared with 16-byte
// cp.async while the previous tile is being computed, then converted once to fp32 working
// arrays: row arrays [RPW][TL+4] (time fastest) and B/C as [TL][NP] (state fastest, so a
// lane reads its NS states of one step with one 16-byte load and lanes of a row read
// adjacent 16-byte groups).
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

// ---- cp.async -----------------------------------------------------------------------------
// 16-byte asynchronous copy; when !valid the destination is zero-filled and src is not read.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool valid) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

// ---- raw tiles ------------------------------------------------------------------------------
// Rows of a (B, D, L) activation tensor for one warp: raw[rr][TL] elements of T.
template <typename T, int RPW, int TL>
__device__ __forceinline__ void fill_rows_raw(T* __restrict__ raw, const T* __restrict__ g, int b, int D, int L, int drow0, int t0, bool vec,
                                              int lane, int64_t sb, int64_t sd) {
  constexpr int V = 16 / sizeof(T);
  if (vec) {
    constexpr int CH = TL / V;
    for (int c = lane; c < RPW * CH; c += 32) {
      const int rr = c / CH, ch = c % CH;
      const int dd = min(drow0 + rr, D - 1);
      const int t = t0 + ch * V;
      const bool ok = t < L;
      cp_async16(raw + rr * TL + ch * V, g + (int64_t)b * sb + (int64_t)dd * sd + (ok ? t : 0), ok);
    }
  } else {
    for (int i = lane; i < RPW * TL; i += 32) {
      const int rr = i / TL, tt = i % TL;
      const int dd = min(drow0 + rr, D - 1);
      const int t = t0 + tt;
      raw[i] = t < L ? g[(int64_t)b * sb + (int64_t)dd * sd + t] : from_f<T>(0.f);
    }
  }
}

// One (N x TL) tile of B or C for the CTA.  vec: raw bytes in the source dtype, [n][TL].
// Otherwise the elements are converted while loading and stored as fp32 [n][TL].
template <int TL>
__device__ __forceinline__ void fill_bc_raw(void* __restrict__ raw, const char* __restrict__ base, int dtype, int64_t sn, int64_t st, int N, int t0,
                                            int L, bool vec, int tid, int nthreads) {
  if (vec) {
    const int esz = dtype == SSM_F32 ? 4 : 2;
    const int per = 16 / esz;          // elements per 16-byte chunk
    const int CH = TL / per;           // chunks per row
    char* dst = reinterpret_cast<char*>(raw);
    for (int c = tid; c < N * CH; c += nthreads) {
      const int n = c / CH, ch = c % CH;
      const int t = t0 + ch * per;
      const bool ok = t < L;
      cp_async16(dst + ((int64_t)n * TL + ch * per) * esz, base + ((int64_t)n * sn + (ok ? t : 0)) * esz, ok);
    }
  } else {
    float* dst = reinterpret_cast<float*>(raw);
    for (int i = tid; i < N * TL; i += nthreads) {
      const int n = i / TL, tt = i % TL;
      const int t = t0 + tt;
      dst[i] = t < L ? load_dyn(base, (int64_t)n * sn + (int64_t)t * st, dtype) : 0.f;
    }
  }
}

__device__ __forceinline__ float raw_bc_at(const void* raw, int idx, int dtype) {
  if (dtype == SSM_F32) return reinterpret_cast<const float*>(raw)[idx];
  if (dtype == SSM_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(raw)[idx]);
  return __half2float(reinterpret_cast<const __half*>(raw)[idx]);
}

// raw [n][TL] -> fp32 [TL][NP]; states >= N are written as zero.
template <int TL, int NP>
__device__ __forceinline__ void convert_bc(float* __restrict__ dst, const void* __restrict__ raw, int dtype, int N, int tid, int nthreads) {
  constexpr int NQ = NP / 4;
  for (int i = tid; i < NQ * TL; i += nthreads) {
    const int nq = i % NQ, tt = i / NQ;
    float v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int n = nq * 4 + k;
      v[k] = n < N ? raw_bc_at(raw, n * TL + tt, dtype) : 0.f;
    }
    *reinterpret_cast<float4*>(dst + tt * NP + nq * 4) = make_float4(v[0], v[1], v[2], v[3]);
  }
}

// Element offset of the start of B/C data for batch b and channel d.
__device__ __forceinline__ int64_t bc_row_offset(int b, int d, int rows_per_group, int64_t sb, int64_t sg) {
  return (int64_t)b * sb + (int64_t)(d / rows_per_group) * sg;
}

// Load a lane's NS consecutive states of step tt from a [TL][NP] tile.
template <int NS, int NP>
__device__ __forceinline__ void load_states(const float* __restrict__ tile, int tt, int sg, float (&v)[NS]) {
  if constexpr (NS % 4 == 0) {
#pragma unroll
    for (int k = 0; k < NS; k += 4) {
      const float4 q = *reinterpret_cast<const float4*>(tile + tt * NP + sg * NS + k);
      v[k] = q.x, v[k + 1] = q.y, v[k + 2] = q.z, v[k + 3] = q.w;
    }
  } else {
    static_assert(NS == 2, "NS must be 2 or a multiple of 4");
    const float2 q = *reinterpret_cast<const float2*>(tile + tt * NP + sg * NS);
    v[0] = q.x, v[1] = q.y;
  }
}

}  // namespace ssmb
