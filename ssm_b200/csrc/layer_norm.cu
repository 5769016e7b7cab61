// Residual add fused with LayerNorm / RMSNorm, forward and backward, sm_100a.
//
// HBM-bound: each row is read once into registers (x and residual as 16-byte vectors),
// the mean and the centred variance are both computed from those registers (the two-pass
// form of the specification, no E[x^2]-mean^2 cancellation), and y / residual_out are
// written once.  A row is owned by a group of G threads (a warp, or 128 / 512 threads for
// wide rows).  The backward kernel is persistent: every thread keeps the weight / bias
// gradient of its own columns in registers across all rows its CTA visits, the CTA writes
// one partial row, and a second small kernel folds the partials -- no atomics, bitwise
// reproducible.
#include <mutex>

#include "common.cuh"

namespace ssmb {

constexpr int kNormFwdChunks = 4;  // 16-byte chunks of x per thread, forward
constexpr int kNormBwdChunks = 2;  // widest backward configuration: 512 threads x 2 chunks
constexpr int kNormBwdMaxCtas = 592;  // 4 per SM on a 148-SM part

// V consecutive elements of run-time type -> fp32
template <int V>
__device__ __forceinline__ void load_dyn_vec(const void* base, int64_t i, int dtype, float (&f)[V]) {
  if (dtype == SSM_F32) {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + i);
#pragma unroll
    for (int k = 0; k < V / 4; ++k) {
      const float4 v = __ldcs(p + k);
      f[4 * k] = v.x, f[4 * k + 1] = v.y, f[4 * k + 2] = v.z, f[4 * k + 3] = v.w;
    }
  } else if constexpr (V == 8) {
    const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + i));
    if (dtype == SSM_BF16) {
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] = __bfloat162float(e[k]);
    } else {
      const __half* e = reinterpret_cast<const __half*>(&raw);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] = __half2float(e[k]);
    }
  } else {
    const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(base) + i));
    if (dtype == SSM_BF16) {
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
      for (int k = 0; k < 4; ++k) f[k] = __bfloat162float(e[k]);
    } else {
      const __half* e = reinterpret_cast<const __half*>(&raw);
#pragma unroll
      for (int k = 0; k < 4; ++k) f[k] = __half2float(e[k]);
    }
  }
}
template <int V>
__device__ __forceinline__ void store_dyn_vec(void* base, int64_t i, int dtype, const float (&f)[V]) {
  if (dtype == SSM_F32) {
    float4* p = reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + i);
#pragma unroll
    for (int k = 0; k < V / 4; ++k) __stcs(p + k, make_float4(f[4 * k], f[4 * k + 1], f[4 * k + 2], f[4 * k + 3]));
  } else if constexpr (V == 8) {
    uint4 raw;
    if (dtype == SSM_BF16) {
      __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&raw);
#pragma unroll
      for (int k = 0; k < 8; ++k) e[k] = __float2bfloat16_rn(f[k]);
    } else {
      __half* e = reinterpret_cast<__half*>(&raw);
#pragma unroll
      for (int k = 0; k < 8; ++k) e[k] = __float2half_rn(f[k]);
    }
    __stcs(reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(base) + i), raw);
  } else {
    uint2 raw;
    if (dtype == SSM_BF16) {
      __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&raw);
#pragma unroll
      for (int k = 0; k < 4; ++k) e[k] = __float2bfloat16_rn(f[k]);
    } else {
      __half* e = reinterpret_cast<__half*>(&raw);
#pragma unroll
      for (int k = 0; k < 4; ++k) e[k] = __float2half_rn(f[k]);
    }
    __stcs(reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(base) + i), raw);
  }
}

// Sum over the G threads of a row group.  G == 32: shuffles only.  G > 32: one row per CTA.
template <int G>
__device__ __forceinline__ float group_allsum(float v, float* scratch) {
  v = warp_sum(v);
  if constexpr (G > 32) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();  // scratch reuse
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < G / 32; ++w) t += scratch[w];
    v = t;
  }
  return v;
}

template <typename T, int G>
struct NormCfg {
  static constexpr int V = 16 / sizeof(T);
  static constexpr int BLOCK = G < 128 ? 128 : G;
  static constexpr int RPC = BLOCK / G;  // rows per CTA pass
};

// A row's pieces of a tensor of run-time element type, in two steps: every load of the row is issued first (the type switch
// sits outside the loop over chunks, so each arm is a straight run of independent loads), the conversions come afterwards.
// With the load, the conversion and the next load of a chunk in one loop body the loads of a row went out one memory
// latency after the other.  Threads beyond the end of the row read its last chunk (a valid address) and drop the value.
template <int V, int G, int MC>
__device__ __forceinline__ void dyn_issue_row(const void* base, int64_t row_off, int gt, int nchunk, int dtype, uint4 (&a)[MC], uint4 (&b)[MC]) {
  if (dtype == SSM_F32) {
#pragma unroll
    for (int c = 0; c < MC; ++c) {
      const int ch = min(c * G + gt, nchunk - 1);
      const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(base) + row_off + (int64_t)ch * V);
      a[c] = __ldcs(p);
      if constexpr (V == 8) b[c] = __ldcs(p + 1);
    }
  } else if constexpr (V == 8) {
#pragma unroll
    for (int c = 0; c < MC; ++c) {
      const int ch = min(c * G + gt, nchunk - 1);
      a[c] = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + row_off + (int64_t)ch * V));
    }
  } else {
#pragma unroll
    for (int c = 0; c < MC; ++c) {
      const int ch = min(c * G + gt, nchunk - 1);
      const uint2 t = __ldcs(reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(base) + row_off + (int64_t)ch * V));
      a[c] = make_uint4(t.x, t.y, 0u, 0u);
    }
  }
}
template <int V>
__device__ __forceinline__ void dyn_convert(int dtype, const uint4& a, const uint4& b, float (&f)[V]) {
  if (dtype == SSM_F32) {
    f[0] = __uint_as_float(a.x), f[1] = __uint_as_float(a.y), f[2] = __uint_as_float(a.z), f[3] = __uint_as_float(a.w);
    if constexpr (V == 8) f[4] = __uint_as_float(b.x), f[5] = __uint_as_float(b.y), f[6] = __uint_as_float(b.z), f[7] = __uint_as_float(b.w);
  } else if (dtype == SSM_BF16) {
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&a);
#pragma unroll
    for (int k = 0; k < V; ++k) f[k] = __bfloat162float(e[k]);
  } else {
    const __half* e = reinterpret_cast<const __half*>(&a);
#pragma unroll
    for (int k = 0; k < V; ++k) f[k] = __half2float(e[k]);
  }
}
// the row's pieces of a tensor of the io type
template <typename T, int G, int MC>
__device__ __forceinline__ void io_issue_row(const void* base, int64_t row_off, int gt, int nchunk, uint4 (&a)[MC]) {
  constexpr int V = 16 / sizeof(T);
#pragma unroll
  for (int c = 0; c < MC; ++c) {
    const int ch = min(c * G + gt, nchunk - 1);
    a[c] = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(base) + row_off + (int64_t)ch * V));
  }
}

// Raw pieces of a row of x and of the residual, in flight.
template <int MC>
struct NormRowRaw {
  uint4 x[MC], ra[MC], rb[MC];
};
template <typename T, int G, int MC, bool RES = true>
__device__ __forceinline__ void norm_issue_row(const ssm_norm_args& a, int64_t row, int gt, int nchunk, NormRowRaw<MC>& raw) {
  constexpr int V = 16 / sizeof(T);
  io_issue_row<T, G, MC>(a.x, row * a.hidden, gt, nchunk, raw.x);
  if (RES && a.residual) dyn_issue_row<V, G, MC>(a.residual, row * a.hidden, gt, nchunk, a.res_dtype, raw.ra, raw.rb);
}
// s = x (+ residual when prenorm), r = residual; zero beyond the end of the row.
template <typename T, int G, int MC, bool RES = true>
__device__ __forceinline__ void norm_convert_row(const ssm_norm_args& a, int gt, int nchunk, const NormRowRaw<MC>& raw, float (&s)[MC][16 / sizeof(T)],
                                                 float (&r)[MC][16 / sizeof(T)]) {
  constexpr int V = 16 / sizeof(T);
#pragma unroll
  for (int c = 0; c < MC; ++c) {
    if (c * G + gt < nchunk) {
      Vec16<T> v;
      v.raw = raw.x[c];
      v.unpack(s[c]);
      if (RES && a.residual) {
        dyn_convert<V>(a.res_dtype, raw.ra[c], raw.rb[c], r[c]);
        if (a.prenorm) {
#pragma unroll
          for (int i = 0; i < V; ++i) s[c][i] += r[c][i];
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < V; ++i) s[c][i] = 0.f, r[c][i] = 0.f;
    }
  }
}
// Loads the row into registers as s = x (+ residual when prenorm); returns through refs.
template <typename T, int G, int MC, bool RES = true>
__device__ __forceinline__ void norm_load_row(const ssm_norm_args& a, int64_t row, int gt, int nchunk, float (&s)[MC][16 / sizeof(T)],
                                              float (&r)[MC][16 / sizeof(T)]) {
  NormRowRaw<MC> raw;
  norm_issue_row<T, G, MC, RES>(a, row, gt, nchunk, raw);
  norm_convert_row<T, G, MC, RES>(a, gt, nchunk, raw, s, r);
}

template <typename T, int G, int MC>
__device__ __forceinline__ void norm_stats(const ssm_norm_args& a, int gt, int nchunk, const float (&s)[MC][16 / sizeof(T)], float* scratch,
                                           float& mean, float& rstd) {
  constexpr int V = 16 / sizeof(T);
  const float inv = 1.f / (float)a.hidden;
  mean = 0.f;
  if (!a.is_rms) {
    float t = 0.f;
#pragma unroll
    for (int c = 0; c < MC; ++c)
#pragma unroll
      for (int i = 0; i < V; ++i) t += s[c][i];
    mean = group_allsum<G>(t, scratch) * inv;
  }
  float q = 0.f;
#pragma unroll
  for (int c = 0; c < MC; ++c) {
    if (c * G + gt < nchunk) {
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float d = s[c][i] - mean;
        q = fmaf(d, d, q);
      }
    }
  }
  rstd = rsqrtf(group_allsum<G>(q, scratch) * inv + a.eps);
}

// MC = 16-byte chunks of a row per thread.  Rows of up to 768 chunks stay with 128 threads (several rows in flight per SM keep
// more loads outstanding than one wide CTA per row does); only wider rows take 512 threads.
// RES = false: the call has no residual (its registers are then free, which raises the number of rows in flight).
template <typename T, int G, int MC = kNormFwdChunks, bool RES = true>
__global__ void __launch_bounds__(NormCfg<T, G>::BLOCK) norm_fwd_kernel(const ssm_norm_args a) {
  using Cfg = NormCfg<T, G>;
  constexpr int V = Cfg::V;
  constexpr int kNormFwdChunks = MC;
  __shared__ float scratch[32];
  const int gt = threadIdx.x % G;
  const int64_t row = (int64_t)blockIdx.x * Cfg::RPC + threadIdx.x / G;
  if (row >= a.rows) return;  // whole groups leave together (G >= 32; G > 32 has one row per CTA)
  const int nchunk = a.hidden / V;
  float s[kNormFwdChunks][V], r[kNormFwdChunks][V];
  norm_load_row<T, G, kNormFwdChunks, RES>(a, row, gt, nchunk, s, r);
  if (a.residual_out) {
#pragma unroll
    for (int c = 0; c < kNormFwdChunks; ++c) {
      const int ch = c * G + gt;
      if (ch < nchunk) {
        float o[V];
#pragma unroll
        for (int i = 0; i < V; ++i) o[i] = (RES && a.residual && !a.prenorm) ? s[c][i] + r[c][i] : s[c][i];
        store_dyn_vec<V>(a.residual_out, row * a.hidden + (int64_t)ch * V, a.resout_dtype, o);
      }
    }
  }
  float mean, rstd;
  norm_stats<T, G, kNormFwdChunks>(a, gt, nchunk, s, scratch, mean, rstd);
#pragma unroll
  for (int c = 0; c < kNormFwdChunks; ++c) {
    const int ch = c * G + gt;
    if (ch < nchunk) {
      float o[V], wv[V], bv[V];
#pragma unroll
      for (int i = 0; i < V; i += 4) {  // weight / bias are fp32 and 16-byte aligned at every chunk (hidden % V == 0, V >= 4)
        const float4 w4 = __ldg(reinterpret_cast<const float4*>(a.weight + ch * V + i));
        wv[i] = w4.x, wv[i + 1] = w4.y, wv[i + 2] = w4.z, wv[i + 3] = w4.w;
        const float4 b4 = a.bias ? __ldg(reinterpret_cast<const float4*>(a.bias + ch * V + i)) : make_float4(0.f, 0.f, 0.f, 0.f);
        bv[i] = b4.x, bv[i + 1] = b4.y, bv[i + 2] = b4.z, bv[i + 3] = b4.w;
      }
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float y = fmaf((s[c][i] - mean) * rstd, wv[i], bv[i]);
        if (RES && a.residual && !a.prenorm) y += r[c][i];
        o[i] = y;
      }
      Vec16<T> v;
      v.pack(o);
      v.store_stream(reinterpret_cast<T*>(a.y) + row * a.hidden + (int64_t)ch * V);
    }
  }
}

// MC = 16-byte chunks of a row per thread.  A row of up to 32 * MC chunks is owned by ONE warp (G = 32): every reduction is
// a shuffle tree and four rows are in flight per CTA; wider rows take 128 or 512 threads with block-wide reductions.
// The time of a row is a chain of latencies (loads, two reductions, stores), so what counts is how many loads an SM has in
// flight: all loads of a row are issued before the first use, and with 128-thread CTAs the running weight / bias gradients
// of a thread's columns live in shared-memory slots of its own (same additions in the same order) instead of 16 MC registers,
// which leaves the registers to the loads in flight and lets more CTAs fit.
template <int G, int MC>
constexpr int norm_bwd_min_ctas() {
  return G <= 128 ? (MC <= 2 ? 5 : (MC == 3 ? 3 : 2)) : 1;
}
template <typename T, int G, int MC>
__global__ void __launch_bounds__(NormCfg<T, G>::BLOCK, norm_bwd_min_ctas<G, MC>()) norm_bwd_kernel(const ssm_norm_bwd_args g) {
  using Cfg = NormCfg<T, G>;
  constexpr int V = Cfg::V;
  constexpr int kNormBwdChunks = MC;
  constexpr bool kSmemAcc = G <= 128;
  constexpr int kAccRegs = kSmemAcc ? 1 : MC;
  constexpr int kAccRow = MC * V * G + 1;
  const ssm_norm_args& a = g.fwd;
  __shared__ float scratch[32];
  __shared__ float acc_all[kSmemAcc ? Cfg::RPC * 2 * kAccRow : 1];  // [row slot][weight | bias][chunk][element][thread]
  const int gt = threadIdx.x % G, slot = threadIdx.x / G;
  float* acc = acc_all + (kSmemAcc ? slot * 2 * kAccRow : 0);
  const int nchunk = a.hidden / V;
  const float inv = 1.f / (float)a.hidden;
  float dw[kAccRegs][V], db[kAccRegs][V];
#pragma unroll
  for (int c = 0; c < kNormBwdChunks; ++c)
#pragma unroll
    for (int i = 0; i < V; ++i) {
      if constexpr (kSmemAcc) acc[(c * V + i) * G + gt] = 0.f, acc[kAccRow + (c * V + i) * G + gt] = 0.f;
      else dw[c][i] = 0.f, db[c][i] = 0.f;
    }
  // the weights of this thread's columns are re-read from L1 for every row (16-byte loads) instead of occupying registers
  auto load_w = [&](int c, float (&wv)[V]) {
    const int ch = c * G + gt;
#pragma unroll
    for (int i = 0; i < V; i += 4) {
      const float4 w4 = ch < nchunk ? __ldg(reinterpret_cast<const float4*>(a.weight + ch * V + i)) : make_float4(0.f, 0.f, 0.f, 0.f);
      wv[i] = w4.x, wv[i + 1] = w4.y, wv[i + 2] = w4.z, wv[i + 3] = w4.w;
    }
  };
  const int64_t npass = (a.rows + Cfg::RPC - 1) / Cfg::RPC;
  for (int64_t pass = blockIdx.x; pass < npass; pass += gridDim.x) {
    const int64_t row = pass * Cfg::RPC + slot;
    const bool live = row < a.rows;  // G == 32: a dead warp still joins nothing but its own shuffles
    float s[kNormBwdChunks][V], r[kNormBwdChunks][V], dy[kNormBwdChunks][V];
    if (live) {
      // every load of the row goes out before the first value is used: x, the residual, dy and the gradient arriving through
      // the x + residual output (which takes the place of the residual values, dead once the row sum is formed)
      NormRowRaw<kNormBwdChunks> raw;
      uint4 dyr[kNormBwdChunks], ga[kNormBwdChunks], gb[kNormBwdChunks];
      norm_issue_row<T, G, kNormBwdChunks>(a, row, gt, nchunk, raw);
      io_issue_row<T, G, kNormBwdChunks>(g.dy, row * a.hidden, gt, nchunk, dyr);
      if (g.dresidual_out) dyn_issue_row<V, G, kNormBwdChunks>(g.dresidual_out, row * a.hidden, gt, nchunk, a.resout_dtype, ga, gb);
      norm_convert_row<T, G, kNormBwdChunks>(a, gt, nchunk, raw, s, r);
#pragma unroll
      for (int c = 0; c < kNormBwdChunks; ++c) {
        if (c * G + gt < nchunk) {
          Vec16<T> v;
          v.raw = dyr[c];
          v.unpack(dy[c]);
          if (g.dresidual_out) dyn_convert<V>(a.resout_dtype, ga[c], gb[c], r[c]);
        } else {
#pragma unroll
          for (int i = 0; i < V; ++i) dy[c][i] = 0.f;
        }
      }
    } else {
#pragma unroll
      for (int c = 0; c < kNormBwdChunks; ++c)
#pragma unroll
        for (int i = 0; i < V; ++i) s[c][i] = 0.f, r[c][i] = 0.f, dy[c][i] = 0.f;
    }
    float mean, rstd;
    norm_stats<T, G, kNormBwdChunks>(a, gt, nchunk, s, scratch, mean, rstd);
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int c = 0; c < kNormBwdChunks; ++c) {
      float wv[V];
      load_w(c, wv);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float xh = (s[c][i] - mean) * rstd;
        const float wdy = dy[c][i] * wv[i];
        s[c][i] = xh;  // keep xhat
        c1 = fmaf(wdy, xh, c1);
        c2 += wdy;
        if (live && (c * G + gt) < nchunk) {
          if constexpr (kSmemAcc) {
            float* pw = acc + (c * V + i) * G + gt;
            float* pb = acc + kAccRow + (c * V + i) * G + gt;
            *pw = fmaf(dy[c][i], xh, *pw);
            *pb += dy[c][i];
          } else {
            dw[c][i] = fmaf(dy[c][i], xh, dw[c][i]);
            db[c][i] += dy[c][i];
          }
        }
      }
    }
    c1 = group_allsum<G>(c1, scratch) * inv;
    c2 = a.is_rms ? 0.f : group_allsum<G>(c2, scratch) * inv;
    if (live) {
#pragma unroll
      for (int c = 0; c < kNormBwdChunks; ++c) {
        const int ch = c * G + gt;
        if (ch < nchunk) {
          float dsv[V], wv[V];
          load_w(c, wv);
#pragma unroll
          for (int i = 0; i < V; ++i) dsv[i] = (dy[c][i] * wv[i] - s[c][i] * c1 - c2) * rstd;
          const int64_t off = row * a.hidden + (int64_t)ch * V;
          if (g.dresidual_out) {  // gradient arriving through the x + residual output reaches x and residual unchanged
#pragma unroll
            for (int i = 0; i < V; ++i) dsv[i] += r[c][i], dy[c][i] += r[c][i];
          }
          Vec16<T> v;
          v.pack(dsv);
          v.store_stream(reinterpret_cast<T*>(g.dx) + off);
          if (g.dresidual) {
            if (a.prenorm) store_dyn_vec<V>(g.dresidual, off, a.res_dtype, dsv);
            else store_dyn_vec<V>(g.dresidual, off, a.res_dtype, dy[c]);
          }
        }
      }
    }
  }
  // fold the RPC row slots of this CTA, then write the CTA's partial rows
  if constexpr (Cfg::RPC > 1) __syncthreads();
  if (slot == 0) {
    float* pw = g.partial + (int64_t)blockIdx.x * 2 * a.hidden;
    float* pb = pw + a.hidden;
#pragma unroll
    for (int c = 0; c < kNormBwdChunks; ++c) {
      const int ch = c * G + gt;
      if (ch < nchunk) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          if constexpr (kSmemAcc) {
            float tw = 0.f, tb = 0.f;
#pragma unroll
            for (int q = 0; q < Cfg::RPC; ++q) {
              tw += acc_all[q * 2 * kAccRow + (c * V + i) * G + gt];
              tb += acc_all[q * 2 * kAccRow + kAccRow + (c * V + i) * G + gt];
            }
            pw[ch * V + i] = tw, pb[ch * V + i] = tb;
          } else {
            pw[ch * V + i] = dw[c][i], pb[ch * V + i] = db[c][i];
          }
        }
      }
    }
  }
}

// Column sums of the per-CTA partial rows: 32 columns x kFoldLanes partial-row lanes per CTA,
// so the loads of a column are spread over many threads instead of one serial chain.
constexpr int kFoldLanes = 16;
__global__ void __launch_bounds__(32 * kFoldLanes) norm_fold_kernel(const float* __restrict__ partial, int nctas, int hidden,
                                                                   float* __restrict__ dweight, float* __restrict__ dbias) {
  __shared__ float sw[kFoldLanes][33], sb[kFoldLanes][33];
  const int cx = threadIdx.x & 31, ky = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + cx;
  float tw = 0.f, tb = 0.f;
  if (col < hidden) {
#pragma unroll 4
    for (int k = ky; k < nctas; k += kFoldLanes) {
      tw += __ldg(partial + (int64_t)k * 2 * hidden + col);
      tb += __ldg(partial + (int64_t)k * 2 * hidden + hidden + col);
    }
  }
  sw[ky][cx] = tw, sb[ky][cx] = tb;
  __syncthreads();
  if (ky == 0 && col < hidden) {
#pragma unroll
    for (int k = 1; k < kFoldLanes; ++k) tw += sw[k][cx], tb += sb[k][cx];
    dweight[col] = tw;
    if (dbias) dbias[col] = tb;
  }
}

// ---- fallback for rows that cannot be vectorised (hidden not a multiple of the vector, or
// ---- misaligned pointers): one CTA per row, strided scalar accesses, atomics for dw / db.
template <typename T>
__device__ __forceinline__ float norm_s_at(const ssm_norm_args& a, int64_t off) {
  float v = to_f<T>(reinterpret_cast<const T*>(a.x)[off]);
  if (a.residual && a.prenorm) v += load_dyn(a.residual, off, a.res_dtype);
  return v;
}
__device__ __forceinline__ float block_allsum128(float v, float* scratch) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  return scratch[0] + scratch[1] + scratch[2] + scratch[3];
}
template <typename T, bool BWD>
__global__ void __launch_bounds__(128) norm_scalar_kernel(const ssm_norm_bwd_args g) {
  const ssm_norm_args& a = g.fwd;
  __shared__ float scratch[4];
  const int64_t row = blockIdx.x;
  const int64_t base = row * a.hidden;
  const float inv = 1.f / (float)a.hidden;
  float mean = 0.f;
  if (!a.is_rms) {
    float t = 0.f;
    for (int c = threadIdx.x; c < a.hidden; c += 128) t += norm_s_at<T>(a, base + c);
    mean = block_allsum128(t, scratch) * inv;
  }
  float q = 0.f;
  for (int c = threadIdx.x; c < a.hidden; c += 128) {
    const float d = norm_s_at<T>(a, base + c) - mean;
    q = fmaf(d, d, q);
  }
  const float rstd = rsqrtf(block_allsum128(q, scratch) * inv + a.eps);
  if (!BWD) {
    for (int c = threadIdx.x; c < a.hidden; c += 128) {
      const float sv = norm_s_at<T>(a, base + c);
      float y = (sv - mean) * rstd * __ldg(a.weight + c);
      if (a.bias) y += __ldg(a.bias + c);
      if (a.residual && !a.prenorm) y += load_dyn(a.residual, base + c, a.res_dtype);
      reinterpret_cast<T*>(a.y)[base + c] = from_f<T>(y);
      if (a.residual_out) {
        float ro = to_f<T>(reinterpret_cast<const T*>(a.x)[base + c]);
        if (a.residual) ro += load_dyn(a.residual, base + c, a.res_dtype);
        store_dyn(a.residual_out, base + c, a.resout_dtype, ro);
      }
    }
  } else {
    float c1 = 0.f, c2 = 0.f;
    for (int c = threadIdx.x; c < a.hidden; c += 128) {
      const float xh = (norm_s_at<T>(a, base + c) - mean) * rstd;
      const float dyv = to_f<T>(reinterpret_cast<const T*>(g.dy)[base + c]);
      const float wdy = dyv * __ldg(a.weight + c);
      c1 = fmaf(wdy, xh, c1);
      c2 += wdy;
      atomicAdd(g.dweight + c, dyv * xh);
      if (g.dbias) atomicAdd(g.dbias + c, dyv);
    }
    c1 = block_allsum128(c1, scratch) * inv;
    c2 = a.is_rms ? 0.f : block_allsum128(c2, scratch) * inv;
    for (int c = threadIdx.x; c < a.hidden; c += 128) {
      const float xh = (norm_s_at<T>(a, base + c) - mean) * rstd;
      const float dyv = to_f<T>(reinterpret_cast<const T*>(g.dy)[base + c]);
      const float gro = g.dresidual_out ? load_dyn(g.dresidual_out, base + c, a.resout_dtype) : 0.f;
      const float ds = (dyv * __ldg(a.weight + c) - xh * c1 - c2) * rstd + gro;
      reinterpret_cast<T*>(g.dx)[base + c] = from_f<T>(ds);
      if (g.dresidual) store_dyn(g.dresidual, base + c, a.res_dtype, a.prenorm ? ds : dyv + gro);
    }
  }
}

static int norm_validate(const ssm_norm_args* a) {
  SSM_REQUIRE(a != nullptr, SSM_ERR_NULL, "fused_layer_norm: args is NULL");
  SSM_REQUIRE(a->rows >= 0 && a->hidden >= 1, SSM_ERR_SHAPE, "fused_layer_norm: bad shape");
  SSM_REQUIRE(valid_dtype(a->io_dtype), SSM_ERR_DTYPE, "fused_layer_norm: unknown dtype");
  SSM_REQUIRE(!a->residual || valid_dtype(a->res_dtype), SSM_ERR_DTYPE, "fused_layer_norm: unknown residual dtype");
  SSM_REQUIRE(!a->residual_out || valid_dtype(a->resout_dtype), SSM_ERR_DTYPE, "fused_layer_norm: unknown residual_out dtype");
  SSM_REQUIRE(a->rows < (1ll << 31), SSM_ERR_TOO_LARGE, "fused_layer_norm: too many rows");
  return SSM_OK;
}

static bool norm_vec_ok(const ssm_norm_args& a, int maxchunks, const void* p1, const void* p2, const void* p3) {
  const int V = 16 / dtype_size(a.io_dtype);
  if (a.hidden % V != 0) return false;
  if (a.hidden > 512 * maxchunks * V) return false;
  auto ok = [](const void* p) { return p == nullptr || aligned_to(p, 16); };
  // residual / residual_out / dresidual rows of fp32 with hidden % V == 0 are 16-byte aligned too
  return ok(a.x) && ok(a.y) && ok(a.residual) && ok(a.residual_out) && ok(a.weight) && ok(a.bias) && ok(p1) && ok(p2) && ok(p3);
}

static int norm_group(const ssm_norm_args& a, int maxchunks) {
  const int V = 16 / dtype_size(a.io_dtype);
  const int nchunk = a.hidden / V;
  if (nchunk <= 32 * maxchunks) return 32;
  if (nchunk <= 128 * maxchunks) return 128;
  return 512;
}

static int norm_bwd_ctas(const ssm_norm_args& a, int rpc) {
  const int64_t npass = (a.rows + rpc - 1) / rpc;
  return (int)(npass < kNormBwdMaxCtas ? npass : kNormBwdMaxCtas);
}

template <typename T, int G, int MC = kNormFwdChunks>
static int norm_fwd_launch(const ssm_norm_args& a, cudaStream_t st) {
  using Cfg = NormCfg<T, G>;
  const unsigned grid = (unsigned)((a.rows + Cfg::RPC - 1) / Cfg::RPC);
  if (a.residual) norm_fwd_kernel<T, G, MC, true><<<grid, Cfg::BLOCK, 0, st>>>(a);
  else norm_fwd_kernel<T, G, MC, false><<<grid, Cfg::BLOCK, 0, st>>>(a);
  return launch_status("norm_fwd_kernel");
}
template <typename T, int G, int MC>
static int norm_bwd_launch(const ssm_norm_bwd_args& g, cudaStream_t st, int max_ctas = kNormBwdMaxCtas) {
  using Cfg = NormCfg<T, G>;
  // persistent grid: exactly one resident wave (a second, partial wave would double the time)
  static const int resident = [] {
    int per_sm = 1, sms = 148, dev = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, norm_bwd_kernel<T, G, MC>, Cfg::BLOCK, 0);
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return (per_sm < 1 ? 1 : per_sm) * sms;
  }();
  int nctas = norm_bwd_ctas(g.fwd, Cfg::RPC);
  if (nctas > max_ctas) nctas = max_ctas;
  if (nctas > resident) nctas = resident;
  norm_bwd_kernel<T, G, MC><<<nctas, Cfg::BLOCK, 0, st>>>(g);
  if (int rc = launch_status("norm_bwd_kernel")) return rc;
  norm_fold_kernel<<<(g.fwd.hidden + 31) / 32, 32 * kFoldLanes, 0, st>>>(g.partial, nctas, g.fwd.hidden, g.dweight, g.dbias);
  return launch_status("norm_fold_kernel");
}

// rows of up to 128 chunks go to one warp each (1 .. 4 chunks per lane), wider ones to 128 or 512 threads
template <typename T>
static int norm_bwd_dispatch(const ssm_norm_bwd_args& g, cudaStream_t st, int max_ctas) {
  const int V = 16 / (int)sizeof(T);
  const int nchunk = g.fwd.hidden / V;
  if (nchunk <= 32) return norm_bwd_launch<T, 32, 1>(g, st, max_ctas);
  if (nchunk <= 64) return norm_bwd_launch<T, 32, 2>(g, st, max_ctas);
  if (nchunk <= 96) return norm_bwd_launch<T, 32, 3>(g, st, max_ctas);
  if (nchunk <= 128) return norm_bwd_launch<T, 32, 4>(g, st, max_ctas);
  if (nchunk <= 256) return norm_bwd_launch<T, 128, 2>(g, st, max_ctas);
  if (nchunk <= 384) return norm_bwd_launch<T, 128, 3>(g, st, max_ctas);  // e.g. 2560 columns of 16 bits: three CTAs per SM, not two
  if (nchunk <= 512) return norm_bwd_launch<T, 128, 4>(g, st, max_ctas);
  return norm_bwd_launch<T, 512, 2>(g, st, max_ctas);
}

template <typename T>
static int norm_fwd_t(const ssm_norm_args& a, cudaStream_t st) {
  if (!norm_vec_ok(a, kNormFwdChunks, nullptr, nullptr, nullptr)) {
    ssm_norm_bwd_args g{};
    g.fwd = a;
    norm_scalar_kernel<T, false><<<(unsigned)a.rows, 128, 0, st>>>(g);
    return launch_status("norm_scalar_kernel");
  }
  const int nchunk = a.hidden / (16 / (int)sizeof(T));
  switch (norm_group(a, kNormFwdChunks)) {
    case 32: return norm_fwd_launch<T, 32>(a, st);
    case 128: return norm_fwd_launch<T, 128>(a, st);
    default: return nchunk <= 128 * 6 ? norm_fwd_launch<T, 128, 6>(a, st) : norm_fwd_launch<T, 512>(a, st);
  }
}
template <typename T>
static int norm_bwd_t(const ssm_norm_bwd_args& g, cudaStream_t st) {
  const ssm_norm_args& a = g.fwd;
  if (!norm_vec_ok(a, kNormBwdChunks, g.dy, g.dx, g.dresidual) || !aligned_to(g.dresidual_out, 16)) {
    cudaMemsetAsync(g.dweight, 0, sizeof(float) * a.hidden, st);
    if (g.dbias) cudaMemsetAsync(g.dbias, 0, sizeof(float) * a.hidden, st);
    norm_scalar_kernel<T, true><<<(unsigned)a.rows, 128, 0, st>>>(g);
    return launch_status("norm_scalar_kernel");
  }
  return norm_bwd_dispatch<T>(g, st, kNormBwdMaxCtas);
}


// ---------------------------------------------------------------------------------------
// Backward variant for callers that must not allocate device memory.
//
// The persistent backward kernel needs a scratch area for its per-CTA partial weight / bias
// gradients.  Here that area is a fixed array that lives in the library's device image, so
// the call performs no cudaMalloc / cudaFree and asks no allocator for anything.  The price
// is a fixed capacity (hidden <= kNoAllocMaxHidden, at most kNoAllocCtas partial rows) and
// 9.25 MiB of device memory held on every GPU that loads the library until the process ends.
// ---------------------------------------------------------------------------------------
constexpr int kNoAllocMaxHidden = 8192;
constexpr int kNoAllocCtas = 148;  // one partial row per SM
constexpr size_t kNoAllocFloats = (size_t)2 * kNoAllocMaxHidden * kNoAllocCtas;
static __device__ __align__(256) float g_norm_noalloc_scratch[kNoAllocFloats];

constexpr int kNoAllocMaxDevices = 64;
static float* g_noalloc_addr[kNoAllocMaxDevices];  // device address of the array, per device; set once
static std::mutex g_noalloc_mutex;

// In host code the array's name is only a handle: the address a kernel can use has to be
// asked for, per device, with that device current.
static int noalloc_scratch_address(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    set_error("fused_layer_norm_backward_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    return (int)e;
  }
  if (dev < 0 || dev >= kNoAllocMaxDevices) return fail(SSM_ERR_UNSUPPORTED, "fused_layer_norm_backward_noalloc: device index out of range");
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_norm_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_error("fused_layer_norm_backward_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      return e != cudaSuccess ? (int)e : SSM_ERR_DEVICE;
    }
    g_noalloc_addr[dev] = static_cast<float*>(p);
  }
  *out = g_noalloc_addr[dev];
  return SSM_OK;
}

template <typename T>
static int norm_bwd_noalloc_t(const ssm_norm_bwd_args& g, float* scratch, cudaStream_t st) {
  const ssm_norm_args& a = g.fwd;
  if (!norm_vec_ok(a, kNormBwdChunks, g.dy, g.dx, g.dresidual) || !aligned_to(g.dresidual_out, 16)) {
    // rows that cannot be vectorised take the scalar kernel, which needs no scratch at all
    cudaMemsetAsync(g.dweight, 0, sizeof(float) * a.hidden, st);
    if (g.dbias) cudaMemsetAsync(g.dbias, 0, sizeof(float) * a.hidden, st);
    norm_scalar_kernel<T, true><<<(unsigned)a.rows, 128, 0, st>>>(g);
    return launch_status("norm_scalar_kernel");
  }
  ssm_norm_bwd_args h = g;
  h.partial = scratch;
  return norm_bwd_dispatch<T>(h, st, kNoAllocCtas);
}

}  // namespace ssmb

using namespace ssmb;

extern "C" int ssm_fused_add_norm_fwd(const ssm_norm_args* a, ssm_stream_t stream) {
  if (a && a->io_dtype == SSM_F64) {
    ssm_norm_bwd_args g{};
    g.fwd = *a;
    return f64_norm(g, false, reinterpret_cast<cudaStream_t>(stream));
  }
  if (int rc = norm_validate(a)) return rc;
  if (a->rows == 0) return SSM_OK;
  SSM_REQUIRE(a->x && a->y && a->weight, SSM_ERR_NULL, "fused_layer_norm: x, weight and y are required");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (a->io_dtype) {
    case SSM_F32: return norm_fwd_t<float>(*a, st);
    case SSM_BF16: return norm_fwd_t<__nv_bfloat16>(*a, st);
    default: return norm_fwd_t<__half>(*a, st);
  }
}

extern "C" int64_t ssm_norm_bwd_scratch_floats(int64_t rows, int32_t hidden) {
  (void)rows;
  return (int64_t)2 * hidden * kNormBwdMaxCtas;
}

extern "C" int ssm_fused_add_norm_bwd(const ssm_norm_bwd_args* g, ssm_stream_t stream) {
  SSM_REQUIRE(g != nullptr, SSM_ERR_NULL, "fused_layer_norm_backward: args is NULL");
  const ssm_norm_args* a = &g->fwd;
  if (a->io_dtype == SSM_F64) return f64_norm(*g, true, reinterpret_cast<cudaStream_t>(stream));
  if (int rc = norm_validate(a)) return rc;
  SSM_REQUIRE(g->dweight, SSM_ERR_NULL, "fused_layer_norm_backward: dweight is required");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a->rows == 0) {
    cudaMemsetAsync(g->dweight, 0, sizeof(float) * a->hidden, st);
    if (g->dbias) cudaMemsetAsync(g->dbias, 0, sizeof(float) * a->hidden, st);
    return SSM_OK;
  }
  SSM_REQUIRE(a->x && a->weight && g->dy && g->dx && g->partial, SSM_ERR_NULL, "fused_layer_norm_backward: missing pointer");
  SSM_REQUIRE(!a->residual == !g->dresidual || !g->dresidual, SSM_ERR_NULL, "fused_layer_norm_backward: dresidual without residual");
  SSM_REQUIRE(!g->dresidual_out || valid_dtype(a->resout_dtype), SSM_ERR_DTYPE, "fused_layer_norm_backward: dresidual_out needs resout_dtype");
  switch (a->io_dtype) {
    case SSM_F32: return norm_bwd_t<float>(*g, st);
    case SSM_BF16: return norm_bwd_t<__nv_bfloat16>(*g, st);
    default: return norm_bwd_t<__half>(*g, st);
  }
}

extern "C" int ssm_fused_add_norm_bwd_noalloc(const ssm_norm_bwd_args* g, ssm_stream_t stream) {
  SSM_REQUIRE(g != nullptr, SSM_ERR_NULL, "fused_layer_norm_backward_noalloc: args is NULL");
  const ssm_norm_args* a = &g->fwd;
  if (int rc = norm_validate(a)) return rc;
  SSM_REQUIRE(a->hidden <= kNoAllocMaxHidden, SSM_ERR_TOO_LARGE,
              "fused_layer_norm_backward_noalloc: hidden exceeds the built-in scratch capacity (8192); use ssm_fused_add_norm_bwd");
  SSM_REQUIRE(g->dweight, SSM_ERR_NULL, "fused_layer_norm_backward_noalloc: dweight is required");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a->rows == 0) {
    cudaMemsetAsync(g->dweight, 0, sizeof(float) * a->hidden, st);
    if (g->dbias) cudaMemsetAsync(g->dbias, 0, sizeof(float) * a->hidden, st);
    return SSM_OK;
  }
  SSM_REQUIRE(a->x && a->weight && g->dy && g->dx, SSM_ERR_NULL, "fused_layer_norm_backward_noalloc: missing pointer");
  SSM_REQUIRE(a->residual || !g->dresidual, SSM_ERR_NULL, "fused_layer_norm_backward_noalloc: dresidual without residual");
  SSM_REQUIRE(!g->dresidual_out || valid_dtype(a->resout_dtype), SSM_ERR_DTYPE, "fused_layer_norm_backward_noalloc: dresidual_out needs resout_dtype");
  {
    // the built-in scratch is looked up for the CURRENT device; tensors that live on another one would be paired with the wrong GPU's array
    int cur = -1;
    cudaPointerAttributes attr{};
    if (cudaGetDevice(&cur) == cudaSuccess && cudaPointerGetAttributes(&attr, g->dy) == cudaSuccess && attr.type == cudaMemoryTypeDevice)
      SSM_REQUIRE(attr.device == cur, SSM_ERR_DEVICE, "fused_layer_norm_backward_noalloc: the tensors are not on the current device");
    else
      (void)cudaGetLastError();
  }
  float* scratch = nullptr;
  if (int rc = noalloc_scratch_address(&scratch)) return rc;
  switch (a->io_dtype) {
    case SSM_F32: return norm_bwd_noalloc_t<float>(*g, scratch, st);
    case SSM_BF16: return norm_bwd_noalloc_t<__nv_bfloat16>(*g, scratch, st);
    default: return norm_bwd_noalloc_t<__half>(*g, scratch, st);
  }
}
