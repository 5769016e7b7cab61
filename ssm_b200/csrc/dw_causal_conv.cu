// Depthwise causal conv1d (+ optional SiLU), forward and backward, both layouts, sm_100a.
//
// The operator is HBM-bound: x is read once and y written once (backward: x, dy read once,
// dx written once).  Channels-first: one CTA per (batch, channel) row, 16-byte vector
// accesses along time, the K-1 element halo re-read through L1.  Channels-last: a thread
// owns a 16-byte group of channels and slides along time keeping the window in registers,
// so adjacent threads touch adjacent 16-byte groups of the same time step.
//
// Taps are held newest-first: wr[m] = weight[K-1-m] multiplies x[t-m], so that every
// register-array index below is a compile-time constant for any run-time width K <= 8.
#include <type_traits>

#include "common.cuh"

namespace ssmb {

__device__ __forceinline__ bool aligned_to_dev(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

constexpr int kConvMaxK = 8;  // widest supported kernel; kernels are built for KM = 4 and KM = 8
constexpr int kConvThreads = 128;
constexpr int kConvTimeTile = 128;  // channels-last: time steps per thread walk

// x[t] of one (batch, channel) row; before t = 0 the halo (or zero), beyond len zero.
template <typename T>
__device__ __forceinline__ float conv_x_at(const T* __restrict__ row, const float* __restrict__ halo, int K, int t, int L) {
  if (t >= 0) return t < L ? to_f<T>(row[t]) : 0.f;
  return (halo && t >= -(K - 1)) ? __ldg(halo + (K - 1) + t) : 0.f;
}

// ---------------------------------------------------------------------------------------
// channels-first forward
// ---------------------------------------------------------------------------------------
template <typename T, int KM>
__global__ void __launch_bounds__(kConvThreads) conv_cf_fwd_kernel(const ssm_conv_args a, int vec) {
  constexpr int KH = KM - 1;
  constexpr int V = 16 / sizeof(T);
  const int64_t rowi = blockIdx.x;  // b * C + c
  const int c = (int)(rowi % a.channels);
  const int64_t roff = (rowi / a.channels) * a.row_sb + (int64_t)c * a.row_sc;
  const int L = a.len, K = a.width;
  const T* __restrict__ x = reinterpret_cast<const T*>(a.x) + roff;
  T* __restrict__ y = reinterpret_cast<T*>(a.y) + roff;
  const float* halo = a.halo ? a.halo + rowi * (K - 1) : nullptr;
  float wr[KM];
#pragma unroll
  for (int m = 0; m < KM; ++m) wr[m] = m < K ? __ldg(a.weight + (int64_t)c * K + (K - 1 - m)) : 0.f;
  const float bias = a.bias ? __ldg(a.bias + c) : 0.f;

  if (vec) {
    // A thread takes UB vectors of 16 bytes per pass and issues their loads, and those of the vectors before them (the K - 1
    // earlier inputs: the neighbouring thread's vector, served by the L1), before the first value is used.  Vectors beyond the
    // end of the row are read at the last valid address and dropped.
    constexpr int UB = 4;
    const int nch = L / V;
    for (int base = threadIdx.x; base < nch; base += kConvThreads * UB) {
      uint4 curr[UB], prvr[UB];
#pragma unroll
      for (int j = 0; j < UB; ++j) {
        const int ch = min(base + j * kConvThreads, nch - 1);
        curr[j] = __ldcs(reinterpret_cast<const uint4*>(x + (int64_t)ch * V));
        prvr[j] = __ldg(reinterpret_cast<const uint4*>(x + (int64_t)max(ch - 1, 0) * V));
      }
#pragma unroll
      for (int j = 0; j < UB; ++j) {
        const int ch = base + j * kConvThreads;
        if (ch >= nch) break;
        const int t0 = ch * V;
        Vec16<T> v;
        float cur[V], prv[V], hist[KH > 0 ? KH : 1];  // hist[m] = x[t0 - 1 - m]
        v.raw = curr[j];
        v.unpack(cur);
        v.raw = prvr[j];
        v.unpack(prv);
#pragma unroll
        for (int m = 0; m < KH; ++m) {
          float hv = 0.f;
          if (m < K - 1) hv = (ch > 0 && m < V) ? prv[m < V ? V - 1 - m : 0] : conv_x_at<T>(x, halo, K, t0 - 1 - m, L);
          hist[m] = hv;
        }
        float out[V];
#pragma unroll
        for (int i = 0; i < V; ++i) {
          float acc = bias;
#pragma unroll
          for (int m = 0; m < KM; ++m) {
            if (m < K) acc = fmaf(wr[m], (i - m >= 0) ? cur[(i - m >= 0) ? i - m : 0] : hist[(m - i - 1 >= 0) ? m - i - 1 : 0], acc);
          }
          out[i] = a.silu ? (sizeof(T) == 2 ? silu_half_io(acc) : silu_fast(acc)) : acc;
        }
        v.pack(out);
        v.store_stream(y + t0);
      }
    }
  } else {
    for (int t = threadIdx.x; t < L; t += kConvThreads) {
      float acc = bias;
#pragma unroll
      for (int m = 0; m < KM; ++m)
        if (m < K) acc = fmaf(wr[m], conv_x_at<T>(x, halo, K, t - m, L), acc);
      y[t] = from_f<T>(a.silu ? silu_fast(acc) : acc);
    }
  }
}

// ---------------------------------------------------------------------------------------
// channels-first backward.  pre[t] = bias + sum_m wr[m] x[t-m];  dpre = dy * act'(pre)
//   dx[t] = sum_m wr[m] dpre[t+m];  dwr[m] += sum_t dpre[t] x[t-m];  dbias += sum_t dpre[t]
// ---------------------------------------------------------------------------------------
template <typename T, int KM>
__global__ void __launch_bounds__(kConvThreads) conv_cf_bwd_kernel(const ssm_conv_bwd_args g, int vec) {
  constexpr int KH = KM - 1;
  const ssm_conv_args& a = g.fwd;
  const int64_t rowi = blockIdx.x;
  const int c = (int)(rowi % a.channels);
  const int64_t roff = (rowi / a.channels) * a.row_sb + (int64_t)c * a.row_sc;
  const int L = a.len, K = a.width;
  const T* __restrict__ x = reinterpret_cast<const T*>(a.x) + roff;
  const T* __restrict__ dy = reinterpret_cast<const T*>(g.dy) + roff;
  T* __restrict__ dx = reinterpret_cast<T*>(g.dx) + roff;
  const float* halo = a.halo ? a.halo + rowi * (K - 1) : nullptr;
  float wr[KM], dwr[KM];
#pragma unroll
  for (int m = 0; m < KM; ++m) wr[m] = m < K ? __ldg(a.weight + (int64_t)c * K + (K - 1 - m)) : 0.f, dwr[m] = 0.f;
  const float bias = a.bias ? __ldg(a.bias + c) : 0.f;
  float db = 0.f;

  if (vec) {
    // 16-byte accesses: a thread owns one vector of outputs and reads the neighbouring
    // vectors of x (both sides) and dy (later side) through L1.
    constexpr int V = 16 / sizeof(T);
    constexpr int NB = (KH + V - 1) / V;  // neighbour vectors per side
    const int last = L - V;  // start of the row's last vector: what out-of-range neighbours read (and drop)
    for (int t0 = threadIdx.x * V; t0 < L; t0 += kConvThreads * V) {
      // every load of the pass is issued before the first value is used
      uint4 xr[2 * NB + 1], dyr[NB + 1];
#pragma unroll
      for (int j = 0; j <= 2 * NB; ++j) xr[j] = __ldg(reinterpret_cast<const uint4*>(x + min(max(t0 + (j - NB) * V, 0), last)));
#pragma unroll
      for (int j = 0; j <= NB; ++j) dyr[j] = __ldg(reinterpret_cast<const uint4*>(dy + min(t0 + j * V, last)));
      float xa[(2 * NB + 1) * V];  // xa[q] = x[t0 - NB * V + q]
#pragma unroll
      for (int j = 0; j <= 2 * NB; ++j) {
        const int tv = t0 + (j - NB) * V;
        if (tv >= 0 && tv < L) {
          Vec16<T> v;
          v.raw = xr[j];
          float f[V];
          v.unpack(f);
#pragma unroll
          for (int i = 0; i < V; ++i) xa[j * V + i] = f[i];
        } else {
#pragma unroll
          for (int i = 0; i < V; ++i) xa[j * V + i] = tv < 0 ? conv_x_at<T>(x, halo, K, tv + i, L) : 0.f;
        }
      }
      float dya[(NB + 1) * V];  // dy[t0 + q], zero beyond the row
#pragma unroll
      for (int j = 0; j <= NB; ++j) {
        const int tv = t0 + j * V;
        float f[V];
        if (tv < L) {
          Vec16<T> v;
          v.raw = dyr[j];
          v.unpack(f);
        } else {
#pragma unroll
          for (int i = 0; i < V; ++i) f[i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < V; ++i) dya[j * V + i] = f[i];
      }
      float dp[V + KH];  // dpre[t0 + i]
#pragma unroll
      for (int i = 0; i < V + KH; ++i) {
        float pre = bias;
#pragma unroll
        for (int m = 0; m < KM; ++m)
          if (m < K) pre = fmaf(wr[m], xa[NB * V + i - m], pre);
        float v = dya[i];
        if (a.silu) v *= sizeof(T) == 2 ? silu_grad_half_io(pre) : silu_grad_fast(pre);
        dp[i] = (i < V + K - 1) ? v : 0.f;
      }
      float out[V];
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float acc = 0.f;
#pragma unroll
        for (int m = 0; m < KM; ++m)
          if (m < K) {
            acc = fmaf(wr[m], dp[i + m], acc);
            dwr[m] = fmaf(dp[i], xa[NB * V + i - m], dwr[m]);
          }
        out[i] = acc;
        db += dp[i];
      }
      Vec16<T> v;
      v.pack(out);
      v.store_stream(dx + t0);
    }
  }
  constexpr int S = 4;  // scalar path: outputs per thread per pass; x / dy re-reads hit L1
  for (int t0 = vec ? L : threadIdx.x * S; t0 < L; t0 += kConvThreads * S) {
    float xw[S + 2 * KH];  // xw[q] = x[t0 - KH + q]
#pragma unroll
    for (int q = 0; q < S + 2 * KH; ++q) {
      const int t = t0 - KH + q;
      xw[q] = (t >= t0 - (K - 1) && t <= t0 + S - 1 + (K - 1)) ? conv_x_at<T>(x, halo, K, t, L) : 0.f;
    }
    float dp[S + KH];  // dpre[t0 + i]
#pragma unroll
    for (int i = 0; i < S + KH; ++i) {
      const int t = t0 + i;
      float v = 0.f;
      if (i < S + K - 1 && t < L) {
        float pre = bias;
#pragma unroll
        for (int m = 0; m < KM; ++m)
          if (m < K) pre = fmaf(wr[m], xw[i - m + KH], pre);
        v = to_f<T>(dy[t]);
        if (a.silu) v *= silu_grad_fast(pre);
      }
      dp[i] = v;
    }
#pragma unroll
    for (int i = 0; i < S; ++i) {
      const int t = t0 + i;
      if (t < L) {
        float acc = 0.f;
#pragma unroll
        for (int m = 0; m < KM; ++m)
          if (m < K) {
            acc = fmaf(wr[m], dp[i + m], acc);
            dwr[m] = fmaf(dp[i], xw[i - m + KH], dwr[m]);
          }
        dx[t] = from_f<T>(acc);
        db += dp[i];
      }
    }
  }
  // block reduce -> one atomic per CTA and tap
  __shared__ float red[kConvThreads / 32][KM + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int m = 0; m < KM; ++m) dwr[m] = warp_sum(dwr[m]);
  db = warp_sum(db);
  if (lane == 0) {
#pragma unroll
    for (int m = 0; m < KM; ++m) red[warp][m] = dwr[m];
    red[warp][KM] = db;
  }
  __syncthreads();
  if (threadIdx.x <= KM) {
    float s = 0.f;
    for (int wv = 0; wv < kConvThreads / 32; ++wv) s += red[wv][threadIdx.x];
    const int m = threadIdx.x;
    if (m < K) atomicAdd(g.dweight + (int64_t)c * K + (K - 1 - m), s);
    if (m == KM && g.dbias) atomicAdd(g.dbias + c, s);
  }
}

// ---------------------------------------------------------------------------------------
// channels-last: x (B, L, C); a thread owns V consecutive channels (V*sizeof(T) = 16 or 8 bytes)
// ---------------------------------------------------------------------------------------
template <typename T, int V>
__device__ __forceinline__ void load_group(const T* __restrict__ p, bool vec, int nvalid, float (&f)[V]) {
  if (vec) {
    if constexpr (V * sizeof(T) == 16) {
      const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(p));
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int i = 0; i < V; ++i) f[i] = to_f<T>(e[i]);
    } else {
      static_assert(V * sizeof(T) == 8, "group must be 8 or 16 bytes");
      const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(p));
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int i = 0; i < V; ++i) f[i] = to_f<T>(e[i]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i) f[i] = i < nvalid ? to_f<T>(p[i]) : 0.f;
  }
}
template <typename T, int V>
__device__ __forceinline__ void store_group(T* __restrict__ p, bool vec, int nvalid, const float (&f)[V]) {
  if (vec) {
    if constexpr (V * sizeof(T) == 16) {
      uint4 raw;
      T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
      for (int i = 0; i < V; ++i) e[i] = from_f<T>(f[i]);
      __stcs(reinterpret_cast<uint4*>(p), raw);
    } else {
      uint2 raw;
      T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
      for (int i = 0; i < V; ++i) e[i] = from_f<T>(f[i]);
      __stcs(reinterpret_cast<uint2*>(p), raw);
    }
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i)
      if (i < nvalid) p[i] = from_f<T>(f[i]);
  }
}

// x[b, t, c0 .. c0+V) with halo / zero outside [0, L); xb already points at (b, 0, c0)
template <typename T, int V>
__device__ __forceinline__ void load_x_cl(const ssm_conv_args& a, const T* __restrict__ xb, int b, int c0, int t, bool vec, int nvalid,
                                          float (&f)[V]) {
  const int K = a.width;
  if (t >= 0 && t < a.len) {
    load_group<T, V>(xb + (int64_t)t * a.channels, vec, nvalid, f);
    return;
  }
#pragma unroll
  for (int i = 0; i < V; ++i) f[i] = 0.f;
  if (t < 0 && t >= -(K - 1) && a.halo) {
#pragma unroll
    for (int i = 0; i < V; ++i)
      if (i < nvalid) f[i] = __ldg(a.halo + ((int64_t)b * a.channels + c0 + i) * (K - 1) + (K - 1) + t);
  }
}

// Channels-last forward: thread = V channels, walking `tile` consecutive steps with the K - 1 previous inputs in registers.
// Eight steps' loads are issued before their results are formed, so every thread keeps eight 16-byte loads in flight; the
// host picks `tile` so that narrow tensors (the 128-channel B / C inputs of a Mamba-2 layer) still fill the machine.
template <typename T, int KM>
__global__ void __launch_bounds__(kConvThreads, 3) conv_cl_fwd_kernel(const ssm_conv_args a, int vec, int tile) {
  constexpr int KH = KM - 1;
  constexpr int V = 16 / sizeof(T);
  constexpr int U = 8;  // steps per batch of loads
  const int C = a.channels, L = a.len, K = a.width;
  // work item = (time tile, channel vector), channel vectors fastest: a narrow tensor packs several time tiles into one CTA
  const int nvec = (C + V - 1) / V;
  const int64_t item = (int64_t)blockIdx.x * kConvThreads + threadIdx.x;
  const int c0 = (int)(item % nvec) * V;
  const int64_t tile_idx = item / nvec;
  const int64_t ts64 = tile_idx * tile;
  if (ts64 >= L) return;
  const int ts = (int)ts64, te = min(L, ts + tile);
  const int nvalid = min(V, C - c0);
  const int b = blockIdx.z;
  const T* __restrict__ x = reinterpret_cast<const T*>(a.x) + (int64_t)b * L * C + c0;
  T* __restrict__ y = reinterpret_cast<T*>(a.y) + (int64_t)b * L * C + c0;
  // channel pairs as float2 for the packed-fp32 multiply-adds
  float2 wr[KM][V / 2], bias[V / 2];
  if (K == KM && nvalid == V && (reinterpret_cast<uintptr_t>(a.weight) & 15) == 0 && (!a.bias || (reinterpret_cast<uintptr_t>(a.bias) & 15) == 0)) {
    // the thread's V x K weights are one contiguous run: 16-byte loads (a scalar load per weight costs a sector request per lane,
    // more of them than the whole tile of x)
    float wf[V * KM];
    const float4* wp = reinterpret_cast<const float4*>(a.weight + (int64_t)c0 * KM);
#pragma unroll
    for (int q = 0; q < V * KM / 4; ++q) {
      const float4 w4 = __ldg(wp + q);
      wf[4 * q] = w4.x, wf[4 * q + 1] = w4.y, wf[4 * q + 2] = w4.z, wf[4 * q + 3] = w4.w;
    }
    float bf[V];
#pragma unroll
    for (int q = 0; q < V / 4; ++q) {
      const float4 b4 = a.bias ? __ldg(reinterpret_cast<const float4*>(a.bias + c0) + q) : make_float4(0.f, 0.f, 0.f, 0.f);
      bf[4 * q] = b4.x, bf[4 * q + 1] = b4.y, bf[4 * q + 2] = b4.z, bf[4 * q + 3] = b4.w;
    }
#pragma unroll
    for (int i = 0; i < V; i += 2) {
      bias[i / 2] = make_float2(bf[i], bf[i + 1]);
#pragma unroll
      for (int m = 0; m < KM; ++m) wr[m][i / 2] = make_float2(wf[i * KM + (KM - 1 - m)], wf[(i + 1) * KM + (KM - 1 - m)]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < V; i += 2) {
      const int c1 = min(c0 + i, C - 1), c2 = min(c0 + i + 1, C - 1);
      bias[i / 2] = a.bias ? make_float2(__ldg(a.bias + c1), __ldg(a.bias + c2)) : make_float2(0.f, 0.f);
#pragma unroll
      for (int m = 0; m < KM; ++m)
        wr[m][i / 2] = m < K ? make_float2(__ldg(a.weight + (int64_t)c1 * K + (K - 1 - m)), __ldg(a.weight + (int64_t)c2 * K + (K - 1 - m))) : make_float2(0.f, 0.f);
    }
  }
  float2 hist[KH > 0 ? KH : 1][V / 2];  // hist[m] = x[t - 1 - m]
  // Where the K - 1 steps before the tile lie inside the tensor (every tile but the first of a sequence) and the rows can be
  // read as 16-byte pieces, they are not fetched here, one dependent load after the other, but run through the pipelined loop
  // below as steps without output.
  const bool warm = vec && ts >= K - 1;
#pragma unroll
  for (int m = 0; m < KH; ++m) {
    float f[V];
    if (m < K - 1 && !warm) {
      load_x_cl<T, V>(a, x, b, c0, ts - 1 - m, vec, nvalid, f);
    } else {
#pragma unroll
      for (int i = 0; i < V; ++i) f[i] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < V; i += 2) hist[m][i / 2] = make_float2(f[i], f[i + 1]);
  }
  // one step: inputs f of step tt -> output row, then the window moves on
  auto step = [&](int tt, const float (&f)[V]) {
    if (tt < ts) {  // a step before the tile: it only enters the window
#pragma unroll
      for (int m = KH - 1; m >= 1; --m)
        if (m < K - 1) {
#pragma unroll
          for (int i = 0; i < V / 2; ++i) hist[m][i] = hist[m - 1][i];
        }
      if (KH > 0) {
#pragma unroll
        for (int i = 0; i < V / 2; ++i) hist[0][i] = make_float2(f[2 * i], f[2 * i + 1]);
      }
      return;
    }
    float out[V];
    float2 c2[V / 2];
#pragma unroll
    for (int i = 0; i < V; i += 2) {
      c2[i / 2] = make_float2(f[i], f[i + 1]);
      float2 acc = __ffma2_rn(wr[0][i / 2], c2[i / 2], bias[i / 2]);
#pragma unroll
      for (int m = 1; m < KM; ++m)
        if (m < K) acc = __ffma2_rn(wr[m][i / 2], hist[m - 1][i / 2], acc);
      if (a.silu) {
        out[i] = sizeof(T) == 2 ? silu_half_io(acc.x) : silu_fast(acc.x);
        out[i + 1] = sizeof(T) == 2 ? silu_half_io(acc.y) : silu_fast(acc.y);
      } else {
        out[i] = acc.x, out[i + 1] = acc.y;
      }
    }
    store_group<T, V>(y + (int64_t)tt * C, vec, nvalid, out);
#pragma unroll
    for (int m = KH - 1; m >= 1; --m)
      if (m < K - 1) {
#pragma unroll
        for (int i = 0; i < V / 2; ++i) hist[m][i] = hist[m - 1][i];
      }
    if (KH > 0) {
#pragma unroll
      for (int i = 0; i < V / 2; ++i) hist[0][i] = c2[i];
    }
  };
  if (vec) {
    // The loads of U steps are issued together and stay packed (16 bytes each) until their step is formed; the loads of the
    // next U steps go out before the current ones are used, so a thread always has loads in flight.
    uint4 raw[U], nxt[U];
    const int tb = warm ? ts - (K - 1) : ts;
#pragma unroll
    for (int j = 0; j < U; ++j)
      if (tb + j < te) nxt[j] = __ldcs(reinterpret_cast<const uint4*>(x + (int64_t)(tb + j) * C));
    for (int t = tb; t < te; t += U) {
#pragma unroll
      for (int j = 0; j < U; ++j) raw[j] = nxt[j];
#pragma unroll
      for (int j = 0; j < U; ++j)
        if (t + U + j < te) nxt[j] = __ldcs(reinterpret_cast<const uint4*>(x + (int64_t)(t + U + j) * C));
#pragma unroll
      for (int j = 0; j < U; ++j) {
        if (t + j < te) {
          float f[V];
          const T* e = reinterpret_cast<const T*>(&raw[j]);
#pragma unroll
          for (int i = 0; i < V; ++i) f[i] = to_f<T>(e[i]);
          step(t + j, f);
        }
      }
    }
  } else {
    for (int t = ts; t < te; ++t) {
      float f[V];
      load_group<T, V>(x + (int64_t)t * C, false, nvalid, f);
      step(t, f);
    }
  }
}

// channels-last backward.  Walk s over [ts, te + K - 1): dpre[s] needs x[s-(K-1) .. s];
// dx[t = s-(K-1)] = sum_q w[q] dpre[s - q] (w in stored order) needs dpre[s-(K-1) .. s].
// Four channels per thread keep both windows, both tap orders and the weight-gradient
// accumulators in registers.
template <typename T, int KM>
__global__ void __launch_bounds__(kConvThreads) conv_cl_bwd_kernel(const ssm_conv_bwd_args g, int vec) {
  constexpr int KH = KM - 1;
  const ssm_conv_args& a = g.fwd;
  constexpr int V = 4;
  const int C = a.channels, L = a.len, K = a.width;
  const int c0 = (blockIdx.x * kConvThreads + threadIdx.x) * V;
  if (c0 >= C) return;
  const int nvalid = min(V, C - c0);
  const int b = blockIdx.z;
  const int ts = blockIdx.y * kConvTimeTile, te = min(L, ts + kConvTimeTile);
  const T* __restrict__ x = reinterpret_cast<const T*>(a.x) + (int64_t)b * L * C + c0;
  const T* __restrict__ dy = reinterpret_cast<const T*>(g.dy) + (int64_t)b * L * C + c0;
  T* __restrict__ dx = reinterpret_cast<T*>(g.dx) + (int64_t)b * L * C + c0;
  float w[KM][V], wr[KM][V], bias[V];  // w[q] = weight[c][q];  wr[m] = weight[c][K-1-m]
  if (K == KM && nvalid == V && (reinterpret_cast<uintptr_t>(a.weight) & 15) == 0 && (!a.bias || (reinterpret_cast<uintptr_t>(a.bias) & 15) == 0)) {
    // the thread's V x K weights are one contiguous run: 16-byte loads instead of a sector request per lane and weight
    float wf[V * KM];
    const float4* wp = reinterpret_cast<const float4*>(a.weight + (int64_t)c0 * KM);
#pragma unroll
    for (int q = 0; q < V * KM / 4; ++q) {
      const float4 w4 = __ldg(wp + q);
      wf[4 * q] = w4.x, wf[4 * q + 1] = w4.y, wf[4 * q + 2] = w4.z, wf[4 * q + 3] = w4.w;
    }
    const float4 b4 = a.bias ? __ldg(reinterpret_cast<const float4*>(a.bias + c0)) : make_float4(0.f, 0.f, 0.f, 0.f);
    bias[0] = b4.x, bias[1] = b4.y, bias[2] = b4.z, bias[3] = b4.w;
#pragma unroll
    for (int i = 0; i < V; ++i)
#pragma unroll
      for (int q = 0; q < KM; ++q) w[q][i] = wf[i * KM + q], wr[q][i] = wf[i * KM + (KM - 1 - q)];
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int cc = min(c0 + i, C - 1);
      bias[i] = a.bias ? __ldg(a.bias + cc) : 0.f;
#pragma unroll
      for (int q = 0; q < KM; ++q) {
        w[q][i] = q < K ? __ldg(a.weight + (int64_t)cc * K + q) : 0.f;
        wr[q][i] = q < K ? __ldg(a.weight + (int64_t)cc * K + (K - 1 - q)) : 0.f;
      }
    }
  }
  float dwr[KM][V], db[V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    db[i] = 0.f;
#pragma unroll
    for (int m = 0; m < KM; ++m) dwr[m][i] = 0.f;
  }
  float xh[KH > 0 ? KH : 1][V], dph[KH > 0 ? KH : 1][V];  // xh[m] = x[s-1-m], dph[m] = dpre[s-1-m]
  // Where the K - 1 steps before the tile lie inside the tensor and the rows can be read as whole pieces, they run through the
  // batched loop below as steps that only enter the window, instead of being fetched here one dependent load after the other.
  const bool warm = vec && ts >= K - 1;
#pragma unroll
  for (int m = 0; m < KH; ++m) {
#pragma unroll
    for (int i = 0; i < V; ++i) dph[m][i] = 0.f;  // dx[ts..] never needs dpre before ts
    if (m < K - 1 && !warm) load_x_cl<T, V>(a, x, b, c0, ts - 1 - m, vec, nvalid, xh[m]);
    else {
#pragma unroll
      for (int i = 0; i < V; ++i) xh[m][i] = 0.f;
    }
  }
  // the loads of U steps (x and dy, as packed pieces) go out together; steps beyond the sequence read its last row and drop it
  constexpr int U = 8;
  using Raw = typename std::conditional<sizeof(T) == 2, uint2, uint4>::type;
  const int sb = warm ? ts - (K - 1) : ts, se = te + K - 1;
  for (int s0 = sb; s0 < se; s0 += U) {
    Raw xr[U], gr[U];
    if (vec) {
#pragma unroll
      for (int j = 0; j < U; ++j) {
        const int sc = min(s0 + j, L - 1);
        xr[j] = __ldcs(reinterpret_cast<const Raw*>(x + (int64_t)sc * C));
        gr[j] = __ldcs(reinterpret_cast<const Raw*>(dy + (int64_t)sc * C));
      }
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
    const int s = s0 + j;
    if (s >= se) break;
    float cur[V], dyv[V], dp[V];
    if (vec) {
      const T* ex = reinterpret_cast<const T*>(&xr[j]);
      const T* eg = reinterpret_cast<const T*>(&gr[j]);
#pragma unroll
      for (int i = 0; i < V; ++i) cur[i] = s < L ? to_f<T>(ex[i]) : 0.f, dyv[i] = (s < L && s >= ts) ? to_f<T>(eg[i]) : 0.f;
    } else {
      load_x_cl<T, V>(a, x, b, c0, s, vec, nvalid, cur);
      if (s < L) load_group<T, V>(dy + (int64_t)s * C, vec, nvalid, dyv);
      else {
#pragma unroll
        for (int i = 0; i < V; ++i) dyv[i] = 0.f;
      }
    }
#pragma unroll
    for (int i = 0; i < V; ++i) {
      float pre = fmaf(wr[0][i], cur[i], bias[i]);
#pragma unroll
      for (int m = 1; m < KM; ++m)
        if (m < K) pre = fmaf(wr[m][i], xh[m - 1][i], pre);
      dp[i] = s < L ? (a.silu ? dyv[i] * (sizeof(T) == 2 ? silu_grad_half_io(pre) : silu_grad_fast(pre)) : dyv[i]) : 0.f;
      if (s >= ts && s < te) {  // each position's parameter gradient is counted by the tile that owns it
        db[i] += dp[i];
        dwr[0][i] = fmaf(dp[i], cur[i], dwr[0][i]);
#pragma unroll
        for (int m = 1; m < KM; ++m)
          if (m < K) dwr[m][i] = fmaf(dp[i], xh[m - 1][i], dwr[m][i]);
      }
    }
    const int t = s - (K - 1);
    if (t >= ts && t < te) {
      float out[V];
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float acc = w[0][i] * dp[i];
#pragma unroll
        for (int q = 1; q < KM; ++q)
          if (q < K) acc = fmaf(w[q][i], dph[q - 1][i], acc);
        out[i] = acc;
      }
      store_group<T, V>(dx + (int64_t)t * C, vec, nvalid, out);
    }
#pragma unroll
    for (int m = KH - 1; m >= 1; --m)
      if (m < K - 1) {
#pragma unroll
        for (int i = 0; i < V; ++i) xh[m][i] = xh[m - 1][i], dph[m][i] = dph[m - 1][i];
      }
    if (KH > 0) {
#pragma unroll
      for (int i = 0; i < V; ++i) xh[0][i] = cur[i], dph[0][i] = dp[i];
    }
    }
  }
#pragma unroll
  for (int i = 0; i < V; ++i) {
    if (i < nvalid) {
      if (g.dbias) atomicAdd(g.dbias + c0 + i, db[i]);
#pragma unroll
      for (int m = 0; m < KM; ++m)
        if (m < K) atomicAdd(g.dweight + (int64_t)(c0 + i) * K + (K - 1 - m), dwr[m][i]);
    }
  }
}

// decode-time update: one thread per (batch, channel)
template <typename T>
__global__ void __launch_bounds__(256) conv_update_kernel(const ssm_conv_update_args a) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= (int64_t)a.batch * a.channels) return;
  const int c = (int)(i % a.channels), K = a.width;
  float* cs = a.conv_state + i * K;
  const float xn = to_f<T>(reinterpret_cast<const T*>(a.x)[i]);
  float acc = a.bias ? __ldg(a.bias + c) : 0.f;
  if (K == 4 && aligned_to_dev(cs)) {
    float4 v = *reinterpret_cast<float4*>(cs);
    v = make_float4(v.y, v.z, v.w, xn);
    *reinterpret_cast<float4*>(cs) = v;
    const float4 w = __ldg(reinterpret_cast<const float4*>(a.weight + (int64_t)c * 4));
    acc = fmaf(v.x, w.x, fmaf(v.y, w.y, fmaf(v.z, w.z, fmaf(v.w, w.w, acc))));
  } else {
    for (int j = 0; j < K; ++j) {
      const float v = j + 1 < K ? cs[j + 1] : xn;
      cs[j] = v;
      acc = fmaf(v, __ldg(a.weight + (int64_t)c * K + j), acc);
    }
  }
  reinterpret_cast<T*>(a.out)[i] = from_f<T>(a.silu ? silu_fast(acc) : acc);
}

static int conv_validate(const ssm_conv_args* a) {
  SSM_REQUIRE(a != nullptr, SSM_ERR_NULL, "dw_causal_conv: args is NULL");
  SSM_REQUIRE(a->batch >= 0 && a->channels >= 0 && a->len >= 0, SSM_ERR_SHAPE, "dw_causal_conv: negative size");
  SSM_REQUIRE(a->width >= 1 && a->width <= kConvMaxK, SSM_ERR_UNSUPPORTED, "dw_causal_conv: kernel width must be in [1, 8]");
  SSM_REQUIRE(valid_dtype(a->io_dtype), SSM_ERR_DTYPE, "dw_causal_conv: unknown dtype");
  SSM_REQUIRE(a->batch <= 65535, SSM_ERR_TOO_LARGE, "dw_causal_conv: batch exceeds 65535");
  SSM_REQUIRE(!a->channels_first || (a->row_sb >= 0 && a->row_sc >= a->len), SSM_ERR_SHAPE, "dw_causal_conv: bad row strides");
  SSM_REQUIRE((int64_t)a->batch * a->channels < (1ll << 31), SSM_ERR_TOO_LARGE, "dw_causal_conv: batch*channels too large");
  return SSM_OK;
}

static dim3 conv_cl_grid(const ssm_conv_args& a, int V) {
  return dim3(((a.channels + V - 1) / V + kConvThreads - 1) / kConvThreads, (a.len + kConvTimeTile - 1) / kConvTimeTile, a.batch);
}

// Steps per thread of the channels-last forward: the full tile when that still gives the GPU eight or more waves of CTAs
// (a ragged last wave then costs little), shorter walks otherwise, down to 8 steps (every walk re-reads K - 1 earlier inputs).
static int64_t conv_cl_fwd_ctas(const ssm_conv_args& a, int V, int tile) {
  const int64_t items = (int64_t)((a.channels + V - 1) / V) * ((a.len + tile - 1) / tile);
  return (items + kConvThreads - 1) / kConvThreads;
}
static int conv_cl_fwd_tile(const ssm_conv_args& a, int V) {
  int tile = kConvTimeTile;
  while (tile > 8 && conv_cl_fwd_ctas(a, V, tile) * a.batch < 4 * 3 * 148) tile >>= 1;  // four waves of three CTAs per SM
  while (conv_cl_fwd_ctas(a, V, tile) >= (1ll << 31)) tile <<= 1;
  return tile;
}

template <typename T, int KM>
static int conv_fwd_launch(const ssm_conv_args& a, cudaStream_t st) {
  constexpr int V = 16 / sizeof(T);
  if (a.channels_first) {
    const int vec = (a.len % V == 0) && (a.row_sb % V == 0) && (a.row_sc % V == 0) && aligned_to(a.x, 16) && aligned_to(a.y, 16);
    conv_cf_fwd_kernel<T, KM><<<(unsigned)((int64_t)a.batch * a.channels), kConvThreads, 0, st>>>(a, vec);
  } else {
    const int vec = (a.channels % V == 0) && aligned_to(a.x, 16) && aligned_to(a.y, 16);
    const int tile = conv_cl_fwd_tile(a, V);
    conv_cl_fwd_kernel<T, KM><<<dim3((unsigned)conv_cl_fwd_ctas(a, V, tile), 1, a.batch), kConvThreads, 0, st>>>(a, vec, tile);
  }
  return launch_status("dw_causal_conv_fwd");
}

template <typename T, int KM>
static int conv_bwd_launch(const ssm_conv_bwd_args& g, cudaStream_t st) {
  const ssm_conv_args& a = g.fwd;
  if (a.channels_first) {
    constexpr int VT = 16 / sizeof(T);
    const int vec = (a.len % VT == 0) && (a.row_sb % VT == 0) && (a.row_sc % VT == 0) && aligned_to(a.x, 16) && aligned_to(g.dy, 16) &&
                    aligned_to(g.dx, 16);
    conv_cf_bwd_kernel<T, KM><<<(unsigned)((int64_t)a.batch * a.channels), kConvThreads, 0, st>>>(g, vec);
  } else {
    constexpr int V = 4;
    const size_t gb = V * sizeof(T);
    const int vec = (a.channels % V == 0) && aligned_to(a.x, gb) && aligned_to(g.dy, gb) && aligned_to(g.dx, gb);
    conv_cl_bwd_kernel<T, KM><<<conv_cl_grid(a, V), kConvThreads, 0, st>>>(g, vec);
  }
  return launch_status("dw_causal_conv_bwd");
}

template <typename T>
static int conv_fwd_k(const ssm_conv_args& a, cudaStream_t st) {
  return a.width <= 4 ? conv_fwd_launch<T, 4>(a, st) : conv_fwd_launch<T, 8>(a, st);
}
template <typename T>
static int conv_bwd_k(const ssm_conv_bwd_args& g, cudaStream_t st) {
  return g.fwd.width <= 4 ? conv_bwd_launch<T, 4>(g, st) : conv_bwd_launch<T, 8>(g, st);
}

}  // namespace ssmb

using namespace ssmb;

extern "C" int ssm_dw_causal_conv_fwd(const ssm_conv_args* a, ssm_stream_t stream) {
  if (a && a->io_dtype == SSM_F64) {
    ssm_conv_bwd_args g{};
    g.fwd = *a;
    return f64_conv(g, false, reinterpret_cast<cudaStream_t>(stream));
  }
  if (int rc = conv_validate(a)) return rc;
  if (a->batch == 0 || a->channels == 0 || a->len == 0) return SSM_OK;
  SSM_REQUIRE(a->x && a->y && a->weight, SSM_ERR_NULL, "dw_causal_conv: x, weight and y are required");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (a->io_dtype) {
    case SSM_F32: return conv_fwd_k<float>(*a, st);
    case SSM_BF16: return conv_fwd_k<__nv_bfloat16>(*a, st);
    default: return conv_fwd_k<__half>(*a, st);
  }
}

extern "C" int ssm_dw_causal_conv_bwd(const ssm_conv_bwd_args* g, ssm_stream_t stream) {
  SSM_REQUIRE(g != nullptr, SSM_ERR_NULL, "dw_causal_conv_backward: args is NULL");
  const ssm_conv_args* a = &g->fwd;
  if (a->io_dtype == SSM_F64) return f64_conv(*g, true, reinterpret_cast<cudaStream_t>(stream));
  if (int rc = conv_validate(a)) return rc;
  if (a->batch == 0 || a->channels == 0 || a->len == 0) return SSM_OK;
  SSM_REQUIRE(a->x && a->weight && g->dy && g->dx && g->dweight, SSM_ERR_NULL, "dw_causal_conv_backward: missing pointer");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (a->io_dtype) {
    case SSM_F32: return conv_bwd_k<float>(*g, st);
    case SSM_BF16: return conv_bwd_k<__nv_bfloat16>(*g, st);
    default: return conv_bwd_k<__half>(*g, st);
  }
}

extern "C" int ssm_dw_causal_conv_update(const ssm_conv_update_args* a, ssm_stream_t stream) {
  SSM_REQUIRE(a != nullptr, SSM_ERR_NULL, "dw_causal_conv_update: args is NULL");
  SSM_REQUIRE(a->batch >= 0 && a->channels >= 0 && a->width >= 1, SSM_ERR_SHAPE, "dw_causal_conv_update: bad shape");
  SSM_REQUIRE(valid_dtype(a->io_dtype), SSM_ERR_DTYPE, "dw_causal_conv_update: unknown dtype");
  const int64_t n = (int64_t)a->batch * a->channels;
  if (n == 0) return SSM_OK;
  SSM_REQUIRE(a->conv_state && a->x && a->weight && a->out, SSM_ERR_NULL, "dw_causal_conv_update: missing pointer");
  SSM_REQUIRE(a->width != 4 || aligned_to(a->weight, 16), SSM_ERR_ALIGN, "dw_causal_conv_update: weight must be 16-byte aligned");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((n + 255) / 256);
  switch (a->io_dtype) {
    case SSM_F32: conv_update_kernel<float><<<grid, 256, 0, st>>>(*a); break;
    case SSM_BF16: conv_update_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(*a); break;
    default: conv_update_kernel<__half><<<grid, 256, 0, st>>>(*a); break;
  }
  return launch_status("conv_update_kernel");
}
