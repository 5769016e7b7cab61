// Element-wise chunked diagonal recurrence over (batch, len, heads, proj), forward and
// backward, sm_100a.
//
//   s_t = exp(dt_t A) s_{t-1} + dt_t B_t X_t;   y_t = s_t C_t + D X_t;   y_t *= silu(z_t)
//
// Each (batch, head, proj) lane is an independent scalar recurrence, so with (head, proj)
// fastest in memory consecutive threads read consecutive addresses at every step; the kernels
// are HBM-bound streams.  The sequence axis is split into chunks that run in parallel:
//   forward   (1) every chunk integrates from a zero state and records its decay product,
//             (2) a short serial pass over chunks turns those into each chunk's incoming state,
//             (3) every chunk is replayed from its true incoming state and writes Y;
//   backward  the same three phases give every chunk its incoming state, their mirror image
//             gives every chunk the adjoint that enters it from the right
//             (g_t = C_t dy_t + exp(dt_{t+1} A) g_{t+1} is a linear recurrence too), and one
//             final pass per chunk replays the states into the history scratch and walks back
//             through them producing every gradient.
// Every thread keeps raw pointers that advance by one time stride per step, and the loads of
// eight steps are issued before the first of them is used, so that enough bytes are in flight.
// Without scratch memory a single serial pass is used instead.
#include <type_traits>

#include "common.cuh"

namespace ssmb {

constexpr int kChunkThreads = 128;
constexpr int kChunkUnroll = 8;

__device__ __forceinline__ int64_t bc4_off(const ssm_bcast4& p, int b, int t, int h, int q) {
  return (int64_t)b * p.sb + (int64_t)t * p.st + (int64_t)h * p.sh + (int64_t)q * p.sq;
}
__device__ __forceinline__ float bc4_load_f32(const ssm_bcast4& p, int b, int t, int h, int q) {
  return __ldg(reinterpret_cast<const float*>(p.ptr) + bc4_off(p, b, t, h, q));
}
__device__ __forceinline__ float* bc4_ptr(const ssm_bcast4& p, int b, int t, int h, int q) {
  return const_cast<float*>(reinterpret_cast<const float*>(p.ptr)) + bc4_off(p, b, t, h, q);
}
// true when every (b, t, h, q) of a gradient buffer is a distinct element (no broadcast axis): plain stores suffice
__device__ __forceinline__ bool bc4_dense(const ssm_bcast4& p) { return p.sb != 0 && p.st != 0 && p.sh != 0 && p.sq != 0; }

__device__ __forceinline__ int chunk_valid_len(const ssm_chunk_args& a, int b) {
  if (!a.seq_lens) return a.len;
  const int64_t v = a.seq_lens[b];
  return (int)(v < 0 ? 0 : (v > a.len ? a.len : v));
}

// A time-strided stream of one lane: element offset at the lane's first step, stride per step (0: constant in time).
template <typename E>
struct Stream {
  const E* p;
  int64_t st;
  __device__ __forceinline__ float at(int k) const { return to_f<E>(__ldg(p + (int64_t)k * st)); }
};
// B / C / z stream of element type PT at (b, t, h, q)
template <typename PT>
__device__ __forceinline__ Stream<PT> par_stream(const ssm_bcast4& c, int b, int t, int h, int q) {
  return {reinterpret_cast<const PT*>(c.ptr) + bc4_off(c, b, t, h, q), c.st};
}

// per-lane context shared by all kernels
template <typename T>
struct Lane {
  int b, h, q, hp, HP, valid;
  float Av, Dv;
  __device__ __forceinline__ bool init(const ssm_chunk_args& a) {
    HP = a.heads * a.proj;
    hp = blockIdx.x * kChunkThreads + threadIdx.x;
    if (hp >= HP) return false;
    h = hp / a.proj, q = hp % a.proj;
    b = blockIdx.z;
    valid = chunk_valid_len(a, b);
    Av = bc4_load_f32(a.A, 0, 0, h, q) * kLog2e;
    Dv = a.D.ptr ? bc4_load_f32(a.D, 0, 0, h, q) : 0.f;
    return true;
  }
  __device__ __forceinline__ Stream<T> x(const ssm_chunk_args& a, int t) const {
    return {reinterpret_cast<const T*>(a.X) + ((int64_t)b * a.len + t) * HP + hp, HP};
  }
  __device__ __forceinline__ Stream<T> dt(const ssm_chunk_args& a, int t) const {
    return {reinterpret_cast<const T*>(a.dt) + ((int64_t)b * a.len + t) * a.heads + h, a.heads};
  }
};

// ---------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------
// mode 0: serial over the whole sequence (no scratch).  mode 1: phase 1 (local state + decay).  mode 3: phase 3.
template <typename T, typename PT, int MODE>
__global__ void __launch_bounds__(kChunkThreads) chunk_fwd_kernel(const ssm_chunk_args a, int nchunks, int chunk_len) {
  Lane<T> ln;
  if (!ln.init(a)) return;
  const int c = MODE == 0 ? 0 : blockIdx.y;
  const int t0 = MODE == 0 ? 0 : c * chunk_len;
  const int t1 = MODE == 0 ? a.len : min(a.len, t0 + chunk_len);
  const int te = max(t0, min(t1, ln.valid));
  float* P = a.scratch;                                                             // [batch][nchunks][HP] decay products
  float* S = a.scratch ? a.scratch + (int64_t)a.batch * nchunks * ln.HP : nullptr;  // local end state, then incoming state
  const int64_t slot = ((int64_t)ln.b * nchunks + c) * ln.HP + ln.hp;
  const Stream<T> sx = ln.x(a, t0), sdt = ln.dt(a, t0);
  const Stream<PT> sB = par_stream<PT>(a.Bm, ln.b, t0, ln.h, ln.q);
  const int n = te - t0;
  if (MODE == 1) {
    float s = 0.f, sumdt = 0.f;
    int k = 0;
    for (; k + kChunkUnroll <= n; k += kChunkUnroll) {
      float x[kChunkUnroll], d[kChunkUnroll], bv[kChunkUnroll];
#pragma unroll
      for (int i = 0; i < kChunkUnroll; ++i) x[i] = sx.at(k + i), d[i] = sdt.at(k + i), bv[i] = sB.at(k + i);
#pragma unroll
      for (int i = 0; i < kChunkUnroll; ++i) {
        s = fmaf(ex2_approx(d[i] * ln.Av), s, d[i] * bv[i] * x[i]);
        sumdt += d[i];
      }
    }
    for (; k < n; ++k) {
      const float d = sdt.at(k);
      s = fmaf(ex2_approx(d * ln.Av), s, d * sB.at(k) * sx.at(k));
      sumdt += d;
    }
    P[slot] = ex2_approx(sumdt * ln.Av);
    S[slot] = s;
    return;
  }
  const Stream<PT> sC = par_stream<PT>(a.Cm, ln.b, t0, ln.h, ln.q);
  const bool has_z = a.z.ptr != nullptr;
  const Stream<PT> sz = has_z ? par_stream<PT>(a.z, ln.b, t0, ln.h, ln.q) : Stream<PT>{nullptr, 0};
  T* Y = reinterpret_cast<T*>(a.Y) + ((int64_t)ln.b * a.len + t0) * ln.HP + ln.hp;
  float s;
  if (MODE == 0) s = a.initial.ptr ? bc4_load_f32(a.initial, ln.b, 0, ln.h, ln.q) : 0.f;
  else s = S[slot];
  auto step = [&](float x, float d, float bv, float cv, float zv) {
    s = fmaf(ex2_approx(d * ln.Av), s, d * bv * x);
    float y = fmaf(ln.Dv, x, s * cv);
    if (has_z) y *= silu_fast(zv);
    return y;
  };
  int k = 0;
  for (; k + kChunkUnroll <= n; k += kChunkUnroll) {
    float x[kChunkUnroll], d[kChunkUnroll], bv[kChunkUnroll], cv[kChunkUnroll], zv[kChunkUnroll];
#pragma unroll
    for (int i = 0; i < kChunkUnroll; ++i) {
      x[i] = sx.at(k + i), d[i] = sdt.at(k + i), bv[i] = sB.at(k + i), cv[i] = sC.at(k + i);
      zv[i] = has_z ? sz.at(k + i) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < kChunkUnroll; ++i) Y[(int64_t)(k + i) * ln.HP] = from_f<T>(step(x[i], d[i], bv[i], cv[i], zv[i]));
  }
  for (; k < n; ++k) Y[(int64_t)k * ln.HP] = from_f<T>(step(sx.at(k), sdt.at(k), sB.at(k), sC.at(k), has_z ? sz.at(k) : 0.f));
  for (int t = te; t < t1; ++t) Y[(int64_t)(t - t0) * ln.HP] = from_f<T>(0.f);
  if (MODE == 0 && a.final_state) a.final_state[(int64_t)ln.b * ln.HP + ln.hp] = s;
}

// 16-bit rows with the projection axis contiguous and a multiple of 8: a thread takes 8 neighbouring lanes of one head, so every
// load and store is 16 bytes (a scalar lane moves 2 bytes per instruction and the kernels above are bound by instruction issue,
// not by bytes), and the loads of kVecUnroll steps go out before the first is used.  MODE 1: local state and decay product of a
// chunk.  MODE 3: the chunk replayed from its incoming state, Y written.
constexpr int kVecUnroll = 4;
template <typename T, int MODE>
__global__ void __launch_bounds__(kChunkThreads) chunk_fwd_vec_kernel(const ssm_chunk_args a, int nchunks, int chunk_len) {
  constexpr int V = 8;
  const int HP = a.heads * a.proj;
  const int hp = (blockIdx.x * kChunkThreads + threadIdx.x) * V;
  if (hp >= HP) return;
  const int h = hp / a.proj, q = hp % a.proj;
  const int b = blockIdx.z, c = blockIdx.y;
  const int valid = chunk_valid_len(a, b);
  const int t0 = c * chunk_len, t1 = min(a.len, t0 + chunk_len);
  const int n = max(t0, min(t1, valid)) - t0;
  float Av[V], Dv[V];
#pragma unroll
  for (int e = 0; e < V; ++e) {
    Av[e] = bc4_load_f32(a.A, 0, 0, h, q + e) * kLog2e;
    Dv[e] = (MODE == 3 && a.D.ptr) ? bc4_load_f32(a.D, 0, 0, h, q + e) : 0.f;
  }
  float* P = a.scratch;                                            // [batch][nchunks][HP] decay products
  float* S = a.scratch + (int64_t)a.batch * nchunks * HP;          // local end state, then incoming state
  const int64_t slot = ((int64_t)b * nchunks + c) * HP + hp;
  const T* px = reinterpret_cast<const T*>(a.X) + ((int64_t)b * a.len + t0) * HP + hp;
  const T* pdt = reinterpret_cast<const T*>(a.dt) + ((int64_t)b * a.len + t0) * a.heads + h;
  const T* pB = reinterpret_cast<const T*>(a.Bm.ptr) + bc4_off(a.Bm, b, t0, h, q);
  auto unpack8 = [](const uint4& r, float (&f)[V]) {
    Vec16<T> v;
    v.raw = r;
    v.unpack(f);
  };
  float s[V];
  if (MODE == 1) {
#pragma unroll
    for (int e = 0; e < V; ++e) s[e] = 0.f;
    float sumdt = 0.f;
    for (int k = 0; k < n; k += kVecUnroll) {
      uint4 xr[kVecUnroll], br[kVecUnroll];
      float d[kVecUnroll];
#pragma unroll
      for (int i = 0; i < kVecUnroll; ++i) {
        const int kk = min(k + i, n - 1);  // beyond the chunk: a valid address, dropped below
        xr[i] = __ldg(reinterpret_cast<const uint4*>(px + (int64_t)kk * HP));
        br[i] = __ldg(reinterpret_cast<const uint4*>(pB + (int64_t)kk * a.Bm.st));
        d[i] = to_f<T>(__ldg(pdt + (int64_t)kk * a.heads));
      }
#pragma unroll
      for (int i = 0; i < kVecUnroll; ++i) {
        if (k + i < n) {
          float x[V], bv[V];
          unpack8(xr[i], x);
          unpack8(br[i], bv);
#pragma unroll
          for (int e = 0; e < V; ++e) s[e] = fmaf(ex2_approx(d[i] * Av[e]), s[e], d[i] * bv[e] * x[e]);
          sumdt += d[i];
        }
      }
    }
    float pr[V];
#pragma unroll
    for (int e = 0; e < V; ++e) pr[e] = ex2_approx(sumdt * Av[e]);
    reinterpret_cast<float4*>(P + slot)[0] = make_float4(pr[0], pr[1], pr[2], pr[3]);
    reinterpret_cast<float4*>(P + slot)[1] = make_float4(pr[4], pr[5], pr[6], pr[7]);
    reinterpret_cast<float4*>(S + slot)[0] = make_float4(s[0], s[1], s[2], s[3]);
    reinterpret_cast<float4*>(S + slot)[1] = make_float4(s[4], s[5], s[6], s[7]);
    return;
  }
  const T* pC = reinterpret_cast<const T*>(a.Cm.ptr) + bc4_off(a.Cm, b, t0, h, q);
  const bool has_z = a.z.ptr != nullptr;
  const T* pz = has_z ? reinterpret_cast<const T*>(a.z.ptr) + bc4_off(a.z, b, t0, h, q) : nullptr;
  T* Y = reinterpret_cast<T*>(a.Y) + ((int64_t)b * a.len + t0) * HP + hp;
  {
    const float4 s0 = reinterpret_cast<const float4*>(S + slot)[0], s1 = reinterpret_cast<const float4*>(S + slot)[1];
    s[0] = s0.x, s[1] = s0.y, s[2] = s0.z, s[3] = s0.w, s[4] = s1.x, s[5] = s1.y, s[6] = s1.z, s[7] = s1.w;
  }
  for (int k = 0; k < n; k += kVecUnroll) {
    uint4 xr[kVecUnroll], br[kVecUnroll], cr[kVecUnroll], zr[kVecUnroll];
    float d[kVecUnroll];
#pragma unroll
    for (int i = 0; i < kVecUnroll; ++i) {
      const int kk = min(k + i, n - 1);
      xr[i] = __ldg(reinterpret_cast<const uint4*>(px + (int64_t)kk * HP));
      br[i] = __ldg(reinterpret_cast<const uint4*>(pB + (int64_t)kk * a.Bm.st));
      cr[i] = __ldg(reinterpret_cast<const uint4*>(pC + (int64_t)kk * a.Cm.st));
      zr[i] = has_z ? __ldg(reinterpret_cast<const uint4*>(pz + (int64_t)kk * a.z.st)) : make_uint4(0, 0, 0, 0);
      d[i] = to_f<T>(__ldg(pdt + (int64_t)kk * a.heads));
    }
#pragma unroll
    for (int i = 0; i < kVecUnroll; ++i) {
      if (k + i < n) {
        float x[V], bv[V], cv[V], zv[V], y[V];
        unpack8(xr[i], x);
        unpack8(br[i], bv);
        unpack8(cr[i], cv);
        unpack8(zr[i], zv);
#pragma unroll
        for (int e = 0; e < V; ++e) {
          s[e] = fmaf(ex2_approx(d[i] * Av[e]), s[e], d[i] * bv[e] * x[e]);
          y[e] = fmaf(Dv[e], x[e], s[e] * cv[e]);
          if (has_z) y[e] *= silu_fast(zv[e]);
        }
        Vec16<T> o;
        o.pack(y);
        *reinterpret_cast<uint4*>(Y + (int64_t)(k + i) * HP) = o.raw;
      }
    }
  }
  for (int t = t0 + n; t < t1; ++t) *reinterpret_cast<uint4*>(Y + (int64_t)(t - t0) * HP) = make_uint4(0, 0, 0, 0);
}

// The carry over the pieces: v_{c+1} = P[c] v_c + L[c], and L[c] is replaced by v_c (what enters piece c).  One lane per hp,
// kCarryGroups threads per lane: each composes kCarryPer consecutive pieces (all their loads in flight at once), the
// composites of the groups meet in shared memory, and each group then replays its pieces from what enters it; a serial
// chain of 16 + 4 + 16 multiply-adds per 64 pieces instead of 64 dependent on 64 loads.  REVERSE walks the pieces from the
// right (the adjoint).  Returns the value that leaves the last piece.
constexpr int kCarryLanes = 128, kCarryGroups = 4, kCarryPer = 16;
template <bool REVERSE>
__device__ __forceinline__ float carry_pieces(const float* __restrict__ P, float* __restrict__ Lc, int nchunks, int64_t stride, float v_in, bool live) {
  __shared__ float sP[kCarryGroups][kCarryLanes], sS[kCarryGroups][kCarryLanes];
  const int lane = threadIdx.x % kCarryLanes, grp = threadIdx.x / kCarryLanes;
  for (int base = 0; base < nchunks; base += kCarryGroups * kCarryPer) {
    const int r0 = base + grp * kCarryPer;  // position in walking order
    float local[kCarryPer], pr[kCarryPer];
#pragma unroll
    for (int i = 0; i < kCarryPer; ++i) {
      const int r = min(r0 + i, nchunks - 1);
      const int64_t at = (int64_t)(REVERSE ? nchunks - 1 - r : r) * stride;
      local[i] = Lc[at], pr[i] = P[at];
    }
    float Pg = 1.f, Sg = 0.f;
#pragma unroll
    for (int i = 0; i < kCarryPer; ++i) {
      if (r0 + i < nchunks) Sg = fmaf(pr[i], Sg, local[i]), Pg *= pr[i];
    }
    sP[grp][lane] = Pg, sS[grp][lane] = Sg;
    __syncthreads();
    float v = v_in, v_next = v_in;
#pragma unroll
    for (int g2 = 0; g2 < kCarryGroups; ++g2) {
      if (g2 < grp) v = fmaf(sP[g2][lane], v, sS[g2][lane]);
      v_next = fmaf(sP[g2][lane], v_next, sS[g2][lane]);
    }
#pragma unroll
    for (int i = 0; i < kCarryPer; ++i) {
      const int r = r0 + i;
      if (r < nchunks) {
        if (live) Lc[(int64_t)(REVERSE ? nchunks - 1 - r : r) * stride] = v;
        v = fmaf(pr[i], v, local[i]);
      }
    }
    v_in = v_next;
    __syncthreads();
  }
  return v_in;
}

// phase 2: S[c] <- state entering piece c
__global__ void __launch_bounds__(kCarryLanes * kCarryGroups) chunk_carry_kernel(const ssm_chunk_args a, int nchunks) {
  const int HP = a.heads * a.proj;
  const int hp_raw = blockIdx.x * kCarryLanes + threadIdx.x % kCarryLanes;
  const bool live = hp_raw < HP;
  const int hp = live ? hp_raw : HP - 1;  // idle lanes of the last CTA shadow a valid lane: they meet the barriers and write nothing
  const int b = blockIdx.z;
  const int h = hp / a.proj, q = hp % a.proj;
  const float* P = a.scratch + (int64_t)b * nchunks * HP + hp;
  float* S = a.scratch + (int64_t)a.batch * nchunks * HP + (int64_t)b * nchunks * HP + hp;
  const float s0 = a.initial.ptr ? bc4_load_f32(a.initial, b, 0, h, q) : 0.f;
  const float s = carry_pieces<false>(P, S, nchunks, HP, s0, live);
  if (live && threadIdx.x < kCarryLanes && a.final_state) a.final_state[(int64_t)b * HP + hp] = s;
}

// ---------------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------------
// dy_t = dout_t * silu(z_t) (or dout_t)
__device__ __forceinline__ float gated_dy(float dout, bool has_z, float zv) { return has_z ? dout * silu_fast(zv) : dout; }

// reverse phase 1: per chunk, the adjoint that leaves the chunk on its left side when nothing enters on the right:
//   carry <- exp(dt_t A) (C_t dy_t + carry), t from the chunk's last valid step down to its first
template <typename T, typename PT>
__global__ void __launch_bounds__(kChunkThreads) chunk_bwd_local_kernel(const ssm_chunk_bwd_args g, int nchunks) {
  const ssm_chunk_args& a = g.fwd;
  Lane<T> ln;
  if (!ln.init(a)) return;
  const int c = blockIdx.y;
  const int t0 = c * a.chunk_size, t1 = min(a.len, t0 + a.chunk_size);
  const int te = max(t0, min(t1, ln.valid));
  const int n = te - t0;
  float* R = g.scratch + 2 * (int64_t)a.batch * nchunks * ln.HP;  // [batch][nchunks][HP] local adjoint, then the adjoint entering each chunk
  const int64_t slot = ((int64_t)ln.b * nchunks + c) * ln.HP + ln.hp;
  const Stream<T> sdt = ln.dt(a, t0);
  const Stream<T> sdy = {reinterpret_cast<const T*>(g.dY) + ((int64_t)ln.b * a.len + t0) * ln.HP + ln.hp, ln.HP};
  const Stream<PT> sC = par_stream<PT>(a.Cm, ln.b, t0, ln.h, ln.q);
  const bool has_z = a.z.ptr != nullptr;
  const Stream<PT> sz = has_z ? par_stream<PT>(a.z, ln.b, t0, ln.h, ln.q) : Stream<PT>{nullptr, 0};
  float carry = 0.f;
  int k = n;
  for (; k - kChunkUnroll >= 0; k -= kChunkUnroll) {
    float d[kChunkUnroll], dy[kChunkUnroll], cv[kChunkUnroll];
#pragma unroll
    for (int i = 0; i < kChunkUnroll; ++i) {
      const int kk = k - 1 - i;
      d[i] = sdt.at(kk), cv[i] = sC.at(kk);
      dy[i] = gated_dy(sdy.at(kk), has_z, has_z ? sz.at(kk) : 0.f);
    }
#pragma unroll
    for (int i = 0; i < kChunkUnroll; ++i) carry = ex2_approx(d[i] * ln.Av) * fmaf(cv[i], dy[i], carry);
  }
  for (; k > 0; --k) {
    const int kk = k - 1;
    carry = ex2_approx(sdt.at(kk) * ln.Av) * fmaf(sC.at(kk), gated_dy(sdy.at(kk), has_z, has_z ? sz.at(kk) : 0.f), carry);
  }
  R[slot] = carry;
}

// the same on 16-byte lanes (8 neighbouring projections of one head per thread; 16-bit per-token C / z, see chunk_vec_ok)
template <typename T>
__global__ void __launch_bounds__(kChunkThreads) chunk_bwd_local_vec_kernel(const ssm_chunk_bwd_args g, int nchunks) {
  constexpr int V = 8, U = 4;
  const ssm_chunk_args& a = g.fwd;
  const int HP = a.heads * a.proj;
  const int hp = (blockIdx.x * kChunkThreads + threadIdx.x) * V;
  if (hp >= HP) return;
  const int h = hp / a.proj, q = hp % a.proj;
  const int b = blockIdx.z, c = blockIdx.y;
  const int t0 = c * a.chunk_size, t1 = min(a.len, t0 + a.chunk_size);
  const int n = max(t0, min(t1, chunk_valid_len(a, b))) - t0;
  float* R = g.scratch + 2 * (int64_t)a.batch * nchunks * HP + ((int64_t)b * nchunks + c) * HP + hp;
  float Av[V], carry[V];
#pragma unroll
  for (int e = 0; e < V; ++e) Av[e] = bc4_load_f32(a.A, 0, 0, h, q + e) * kLog2e, carry[e] = 0.f;
  const T* pdy = reinterpret_cast<const T*>(g.dY) + ((int64_t)b * a.len + t0) * HP + hp;
  const T* pdt = reinterpret_cast<const T*>(a.dt) + ((int64_t)b * a.len + t0) * a.heads + h;
  const T* pC = reinterpret_cast<const T*>(a.Cm.ptr) + bc4_off(a.Cm, b, t0, h, q);
  const bool has_z = a.z.ptr != nullptr;
  const T* pz = has_z ? reinterpret_cast<const T*>(a.z.ptr) + bc4_off(a.z, b, t0, h, q) : nullptr;
  for (int k = n; k > 0; k -= U) {
    uint4 gr[U], cr[U], zr[U];
    float d[U];
#pragma unroll
    for (int i = 0; i < U; ++i) {
      const int kk = max(k - 1 - i, 0);
      gr[i] = __ldg(reinterpret_cast<const uint4*>(pdy + (int64_t)kk * HP));
      cr[i] = __ldg(reinterpret_cast<const uint4*>(pC + (int64_t)kk * a.Cm.st));
      zr[i] = has_z ? __ldg(reinterpret_cast<const uint4*>(pz + (int64_t)kk * a.z.st)) : make_uint4(0, 0, 0, 0);
      d[i] = to_f<T>(__ldg(pdt + (int64_t)kk * a.heads));
    }
#pragma unroll
    for (int i = 0; i < U; ++i) {
      if (k - 1 - i < 0) break;
      float dout[V], cv[V], zv[V];
      Vec16<T> v;
      v.raw = gr[i], v.unpack(dout);
      v.raw = cr[i], v.unpack(cv);
      v.raw = zr[i], v.unpack(zv);
#pragma unroll
      for (int e = 0; e < V; ++e) carry[e] = ex2_approx(d[i] * Av[e]) * fmaf(cv[e], gated_dy(dout[e], has_z, zv[e]), carry[e]);
    }
  }
  reinterpret_cast<float4*>(R)[0] = make_float4(carry[0], carry[1], carry[2], carry[3]);
  reinterpret_cast<float4*>(R)[1] = make_float4(carry[4], carry[5], carry[6], carry[7]);
}

// reverse phase 2: over the pieces from the right; R[c] <- adjoint entering piece c from piece c + 1
__global__ void __launch_bounds__(kCarryLanes * kCarryGroups) chunk_bwd_carry_kernel(const ssm_chunk_bwd_args g, int nchunks) {
  const ssm_chunk_args& a = g.fwd;
  const int HP = a.heads * a.proj;
  const int hp_raw = blockIdx.x * kCarryLanes + threadIdx.x % kCarryLanes;
  const bool live = hp_raw < HP;
  const int hp = live ? hp_raw : HP - 1;
  const int b = blockIdx.z;
  const float* P = g.scratch + (int64_t)b * nchunks * HP + hp;
  float* R = g.scratch + 2 * (int64_t)a.batch * nchunks * HP + (int64_t)b * nchunks * HP + hp;
  const float carry = carry_pieces<true>(P, R, nchunks, HP, 0.f, live);
  if (live && threadIdx.x < kCarryLanes && g.dinitial.ptr) {
    const int h = hp / a.proj, q = hp % a.proj;
    atomicAdd(bc4_ptr(g.dinitial, b, 0, h, q), carry);
  }
}

// sum over the lanes of a warp that share a head, then one atomic per group (proj a multiple of 32: the whole warp)
__device__ __forceinline__ void add_reduced(float* dst, float v, bool whole_warp) {
  if (whole_warp) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) atomicAdd(dst, v);
  } else {
    atomicAdd(dst, v);
  }
}

// final pass: MODE 0 = one thread walks the whole sequence (no scratch); MODE 1 = one chunk per blockIdx.y, states and
// adjoints entering the chunk taken from the scratch.
template <typename T, typename PT, int MODE>
__global__ void __launch_bounds__(kChunkThreads) chunk_bwd_kernel(const ssm_chunk_bwd_args g, int nchunks) {
  const ssm_chunk_args& a = g.fwd;
  Lane<T> ln;
  if (!ln.init(a)) return;
  const int c = MODE == 0 ? 0 : blockIdx.y;
  const int t0 = MODE == 0 ? 0 : c * a.chunk_size;
  const int t1 = MODE == 0 ? a.len : min(a.len, t0 + a.chunk_size);
  const int te = max(t0, min(t1, ln.valid));
  const int n = te - t0;
  const int64_t slot = ((int64_t)ln.b * nchunks + c) * ln.HP + ln.hp;
  float s0, carry;
  if (MODE == 0) {
    s0 = a.initial.ptr ? bc4_load_f32(a.initial, ln.b, 0, ln.h, ln.q) : 0.f;
    carry = 0.f;
  } else {
    s0 = g.scratch[(int64_t)a.batch * nchunks * ln.HP + slot];
    carry = g.scratch[2 * (int64_t)a.batch * nchunks * ln.HP + slot];
  }
  const Stream<T> sx = ln.x(a, t0), sdt = ln.dt(a, t0);
  const Stream<T> sdy = {reinterpret_cast<const T*>(g.dY) + ((int64_t)ln.b * a.len + t0) * ln.HP + ln.hp, ln.HP};
  const Stream<PT> sB = par_stream<PT>(a.Bm, ln.b, t0, ln.h, ln.q);
  const Stream<PT> sC = par_stream<PT>(a.Cm, ln.b, t0, ln.h, ln.q);
  const bool has_z = a.z.ptr != nullptr;
  const Stream<PT> sz = has_z ? par_stream<PT>(a.z, ln.b, t0, ln.h, ln.q) : Stream<PT>{nullptr, 0};
  float* hist = g.history + ((int64_t)ln.b * a.len + t0) * ln.HP + ln.hp;
  T* dX = reinterpret_cast<T*>(g.dX) + ((int64_t)ln.b * a.len + t0) * ln.HP + ln.hp;

  // ---- states of the chunk, into the history ---------------------------------------------------------------
  {
    float s = s0;
    int k = 0;
    for (; k + kChunkUnroll <= n; k += kChunkUnroll) {
      float x[kChunkUnroll], d[kChunkUnroll], bv[kChunkUnroll];
#pragma unroll
      for (int i = 0; i < kChunkUnroll; ++i) x[i] = sx.at(k + i), d[i] = sdt.at(k + i), bv[i] = sB.at(k + i);
#pragma unroll
      for (int i = 0; i < kChunkUnroll; ++i) {
        s = fmaf(ex2_approx(d[i] * ln.Av), s, d[i] * bv[i] * x[i]);
        hist[(int64_t)(k + i) * ln.HP] = s;
      }
    }
    for (; k < n; ++k) {
      const float d = sdt.at(k);
      s = fmaf(ex2_approx(d * ln.Av), s, d * sB.at(k) * sx.at(k));
      hist[(int64_t)k * ln.HP] = s;
    }
  }
  // typed gradient buffers (a.typed_grads) are written in full, the rows beyond the sequence as zeros
  const bool typed_b = a.typed_grads & 1, typed_c = a.typed_grads & 2, typed_z = has_z && (a.typed_grads & 4);
  auto put = [&](const ssm_bcast4& p, bool typed, int t, float v) {
    const int64_t off = bc4_off(p, ln.b, t, ln.h, ln.q);
    if (typed) const_cast<PT*>(reinterpret_cast<const PT*>(p.ptr))[off] = from_f<PT>(v);
    else const_cast<float*>(reinterpret_cast<const float*>(p.ptr))[off] = v;
  };
  for (int t = te; t < t1; ++t) {
    dX[(int64_t)(t - t0) * ln.HP] = from_f<T>(0.f);
    if (typed_b) put(g.dB, true, t, 0.f);
    if (typed_c) put(g.dC, true, t, 0.f);
    if (typed_z) put(g.dz, true, t, 0.f);
  }

  // ---- reverse recurrence  g_t = C_t dy_t + exp(dt_{t+1} A) g_{t+1} -------------------------------------------
  const bool dense_b = bc4_dense(g.dB), dense_c = bc4_dense(g.dC), dense_z = has_z && bc4_dense(g.dz);
  const bool warp_heads = (a.proj & 31) == 0;  // a warp's 32 lanes share their head: (b, t, h) sums reduce in the warp first
  float dA_acc = 0.f, dD_acc = 0.f;
  const float A_nat = ln.Av * kLn2;
  auto back = [&](int k, float x, float d, float bv, float cv, float zv, float dout, float st, float sp) {
    const int t = t0 + k;
    float dyv = dout;
    if (has_z) {
      const float sg = sigmoid_fast(zv);
      const float yfull = fmaf(ln.Dv, x, st * cv);
      const float dzv = dout * yfull * sg * (1.f + zv * (1.f - sg));
      if (dense_z) put(g.dz, typed_z, t, dzv);
      else if (a.z.sq == 0) add_reduced(bc4_ptr(g.dz, ln.b, t, ln.h, 0), dzv, warp_heads);
      else atomicAdd(bc4_ptr(g.dz, ln.b, t, ln.h, ln.q), dzv);
      dyv = dout * zv * sg;
    }
    const float da = ex2_approx(d * ln.Av);
    const float G = fmaf(cv, dyv, carry);
    if (dense_c) put(g.dC, typed_c, t, dyv * st);
    else atomicAdd(bc4_ptr(g.dC, ln.b, t, ln.h, ln.q), dyv * st);
    if (dense_b) put(g.dB, typed_b, t, G * d * x);
    else atomicAdd(bc4_ptr(g.dB, ln.b, t, ln.h, ln.q), G * d * x);
    dX[(int64_t)k * ln.HP] = from_f<T>(fmaf(dyv, ln.Dv, G * d * bv));
    const float gsa = G * sp * da;
    add_reduced(g.ddt + ((int64_t)ln.b * a.len + t) * a.heads + ln.h, fmaf(G, bv * x, gsa * A_nat), warp_heads);
    dA_acc = fmaf(gsa, d, dA_acc);
    dD_acc = fmaf(dyv, x, dD_acc);
    carry = G * da;
  };
  int k = n;
  for (; k - kChunkUnroll >= 0; k -= kChunkUnroll) {
    float x[kChunkUnroll], d[kChunkUnroll], bv[kChunkUnroll], cv[kChunkUnroll], zv[kChunkUnroll], dout[kChunkUnroll], st[kChunkUnroll + 1];
#pragma unroll
    for (int i = 0; i < kChunkUnroll; ++i) {
      const int kk = k - 1 - i;
      x[i] = sx.at(kk), d[i] = sdt.at(kk), bv[i] = sB.at(kk), cv[i] = sC.at(kk), dout[i] = sdy.at(kk);
      zv[i] = has_z ? sz.at(kk) : 0.f;
      st[i] = hist[(int64_t)kk * ln.HP];
    }
    st[kChunkUnroll] = k - kChunkUnroll > 0 ? hist[(int64_t)(k - kChunkUnroll - 1) * ln.HP] : s0;
#pragma unroll
    for (int i = 0; i < kChunkUnroll; ++i) back(k - 1 - i, x[i], d[i], bv[i], cv[i], zv[i], dout[i], st[i], st[i + 1]);
  }
  for (; k > 0; --k) {
    const int kk = k - 1;
    back(kk, sx.at(kk), sdt.at(kk), sB.at(kk), sC.at(kk), has_z ? sz.at(kk) : 0.f, sdy.at(kk), hist[(int64_t)kk * ln.HP],
         kk > 0 ? hist[(int64_t)(kk - 1) * ln.HP] : s0);
  }
  atomicAdd(bc4_ptr(g.dA, 0, 0, ln.h, ln.q), dA_acc);
  if (g.dD.ptr) {
    if (a.D.sq == 0) add_reduced(bc4_ptr(g.dD, 0, 0, ln.h, 0), dD_acc, warp_heads);
    else atomicAdd(bc4_ptr(g.dD, 0, 0, ln.h, ln.q), dD_acc);
  }
  if (MODE == 0 && g.dinitial.ptr) atomicAdd(bc4_ptr(g.dinitial, ln.b, 0, ln.h, ln.q), carry);
}


// Final backward pass on 16-byte lanes: a thread takes 8 neighbouring projections of one head and one chunk (states and
// adjoints entering the chunk from the scratch).  Same arithmetic as chunk_bwd_kernel<.., 1>; every stream is read and
// written as 16-byte pieces, the per-(b, t, h) sum for ddt is formed over the thread's 8 lanes and, where the threads of a
// head are neighbouring lanes of one warp, over those by shuffles before one atomic add.
template <typename T>
__global__ void __launch_bounds__(kChunkThreads) chunk_bwd_vec_kernel(const ssm_chunk_bwd_args g, int nchunks) {
  constexpr int V = 8, U = 2;
  const ssm_chunk_args& a = g.fwd;
  const int HP = a.heads * a.proj;
  const int hp_raw = (blockIdx.x * kChunkThreads + threadIdx.x) * V;
  const bool active = hp_raw < HP;
  const int hp = active ? hp_raw : HP - V;  // idle threads of the last CTA shadow a valid lane group and write nothing
  const int h = hp / a.proj, q = hp % a.proj;
  const int b = blockIdx.z, c = blockIdx.y;
  const int valid = chunk_valid_len(a, b);
  const int t0 = c * a.chunk_size, t1 = min(a.len, t0 + a.chunk_size);
  const int n = max(t0, min(t1, valid)) - t0;
  const int64_t slot = ((int64_t)b * nchunks + c) * HP + hp;
  float Av[V], Dv[V], s0[V], carry[V];
  {
    const float* ps = g.scratch + (int64_t)a.batch * nchunks * HP + slot;
    const float* pr = g.scratch + 2 * (int64_t)a.batch * nchunks * HP + slot;
    const float4 a0 = reinterpret_cast<const float4*>(ps)[0], a1 = reinterpret_cast<const float4*>(ps)[1];
    const float4 r0 = reinterpret_cast<const float4*>(pr)[0], r1 = reinterpret_cast<const float4*>(pr)[1];
    s0[0] = a0.x, s0[1] = a0.y, s0[2] = a0.z, s0[3] = a0.w, s0[4] = a1.x, s0[5] = a1.y, s0[6] = a1.z, s0[7] = a1.w;
    carry[0] = r0.x, carry[1] = r0.y, carry[2] = r0.z, carry[3] = r0.w, carry[4] = r1.x, carry[5] = r1.y, carry[6] = r1.z, carry[7] = r1.w;
  }
#pragma unroll
  for (int e = 0; e < V; ++e) {
    Av[e] = bc4_load_f32(a.A, 0, 0, h, q + e) * kLog2e;
    Dv[e] = a.D.ptr ? bc4_load_f32(a.D, 0, 0, h, q + e) : 0.f;
  }
  const int64_t row0 = ((int64_t)b * a.len + t0) * HP + hp;
  const T* px = reinterpret_cast<const T*>(a.X) + row0;
  const T* pdy = reinterpret_cast<const T*>(g.dY) + row0;
  const T* pdt = reinterpret_cast<const T*>(a.dt) + ((int64_t)b * a.len + t0) * a.heads + h;
  const T* pB = reinterpret_cast<const T*>(a.Bm.ptr) + bc4_off(a.Bm, b, t0, h, q);
  const T* pC = reinterpret_cast<const T*>(a.Cm.ptr) + bc4_off(a.Cm, b, t0, h, q);
  const bool has_z = a.z.ptr != nullptr;
  const T* pz = has_z ? reinterpret_cast<const T*>(a.z.ptr) + bc4_off(a.z, b, t0, h, q) : nullptr;
  float* hist = g.history + row0;
  T* dX = reinterpret_cast<T*>(g.dX) + row0;
  // element offsets of this thread's first step in the gradient buffers of B, C, z (fp32, or the io type: a.typed_grads)
  const int64_t oB = bc4_off(g.dB, b, t0, h, q), oC = bc4_off(g.dC, b, t0, h, q), oZ = has_z ? bc4_off(g.dz, b, t0, h, q) : 0;
  const bool typed_b = a.typed_grads & 1, typed_c = a.typed_grads & 2, typed_z = a.typed_grads & 4;
  auto unpack8 = [](const uint4& r, float (&f)[V]) {
    Vec16<T> v;
    v.raw = r;
    v.unpack(f);
  };
  auto ld8 = [](const float* p, float (&f)[V]) {
    const float4 u0 = reinterpret_cast<const float4*>(p)[0], u1 = reinterpret_cast<const float4*>(p)[1];
    f[0] = u0.x, f[1] = u0.y, f[2] = u0.z, f[3] = u0.w, f[4] = u1.x, f[5] = u1.y, f[6] = u1.z, f[7] = u1.w;
  };
  auto st8 = [](float* p, const float (&f)[V]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
  };
  auto put8 = [&](const ssm_bcast4& p, bool typed, int64_t off, const float (&f)[V]) {
    if (typed) {
      Vec16<T> o;
      o.pack(f);
      *reinterpret_cast<uint4*>(const_cast<T*>(reinterpret_cast<const T*>(p.ptr)) + off) = o.raw;
    } else {
      st8(const_cast<float*>(reinterpret_cast<const float*>(p.ptr)) + off, f);
    }
  };

  // ---- states of the chunk, into the history ---------------------------------------------------------------
  {
    constexpr int UF = 4;
    float s[V];
#pragma unroll
    for (int e = 0; e < V; ++e) s[e] = s0[e];
    for (int k = 0; k < n; k += UF) {
      uint4 xr[UF], br[UF];
      float d[UF];
#pragma unroll
      for (int i = 0; i < UF; ++i) {
        const int kk = min(k + i, n - 1);
        xr[i] = __ldg(reinterpret_cast<const uint4*>(px + (int64_t)kk * HP));
        br[i] = __ldg(reinterpret_cast<const uint4*>(pB + (int64_t)kk * a.Bm.st));
        d[i] = to_f<T>(__ldg(pdt + (int64_t)kk * a.heads));
      }
#pragma unroll
      for (int i = 0; i < UF; ++i) {
        if (k + i < n) {
          float x[V], bv[V];
          unpack8(xr[i], x);
          unpack8(br[i], bv);
#pragma unroll
          for (int e = 0; e < V; ++e) s[e] = fmaf(ex2_approx(d[i] * Av[e]), s[e], d[i] * bv[e] * x[e]);
          if (active) st8(hist + (int64_t)(k + i) * HP, s);
        }
      }
    }
  }
  if (active) {
    const float zero8[V] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int t = t0 + n; t < t1; ++t) {  // beyond the sequence: zeros in what this call writes in full
      *reinterpret_cast<uint4*>(dX + (int64_t)(t - t0) * HP) = make_uint4(0, 0, 0, 0);
      if (typed_b) put8(g.dB, true, oB + (int64_t)(t - t0) * g.dB.st, zero8);
      if (typed_c) put8(g.dC, true, oC + (int64_t)(t - t0) * g.dC.st, zero8);
      if (has_z && typed_z) put8(g.dz, true, oZ + (int64_t)(t - t0) * g.dz.st, zero8);
    }
  }

  // ---- reverse recurrence  g_t = C_t dy_t + exp(dt_{t+1} A) g_{t+1} -------------------------------------------
  // threads of one head: proj / 8 neighbouring threads; reduced by shuffles when that is a power of two within a warp
  const int group = a.proj / V;
  const bool shuffle_heads = (group & (group - 1)) == 0 && group <= 32;
  float dA_acc[V], dD_acc = 0.f;
#pragma unroll
  for (int e = 0; e < V; ++e) dA_acc[e] = 0.f;
  for (int k = n; k > 0; k -= U) {
    uint4 xr[U], br[U], cr[U], zr[U], gr[U];
    float d[U], st[U + 1][V];
#pragma unroll
    for (int i = 0; i < U; ++i) {
      const int kk = max(k - 1 - i, 0);
      xr[i] = __ldg(reinterpret_cast<const uint4*>(px + (int64_t)kk * HP));
      br[i] = __ldg(reinterpret_cast<const uint4*>(pB + (int64_t)kk * a.Bm.st));
      cr[i] = __ldg(reinterpret_cast<const uint4*>(pC + (int64_t)kk * a.Cm.st));
      zr[i] = has_z ? __ldg(reinterpret_cast<const uint4*>(pz + (int64_t)kk * a.z.st)) : make_uint4(0, 0, 0, 0);
      gr[i] = __ldg(reinterpret_cast<const uint4*>(pdy + (int64_t)kk * HP));
      d[i] = to_f<T>(__ldg(pdt + (int64_t)kk * a.heads));
    }
#pragma unroll
    for (int i = 0; i <= U; ++i) {
      const int kk = k - 1 - i;  // the state after step kk; before the chunk's first step: the incoming state
      if (kk >= 0) {
        ld8(hist + (int64_t)kk * HP, st[i]);
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e) st[i][e] = s0[e];
      }
    }
#pragma unroll
    for (int i = 0; i < U; ++i) {
      const int kk = k - 1 - i;
      if (kk < 0) break;
      float x[V], bv[V], cv[V], zv[V], dout[V], dxo[V], dbo[V], dco[V], dzo[V];
      unpack8(xr[i], x);
      unpack8(br[i], bv);
      unpack8(cr[i], cv);
      unpack8(zr[i], zv);
      unpack8(gr[i], dout);
      float ddt_sum = 0.f;
#pragma unroll
      for (int e = 0; e < V; ++e) {
        float dyv = dout[e];
        if (has_z) {
          const float sg = sigmoid_fast(zv[e]);
          const float yfull = fmaf(Dv[e], x[e], st[i][e] * cv[e]);
          dzo[e] = dout[e] * yfull * sg * (1.f + zv[e] * (1.f - sg));
          dyv = dout[e] * zv[e] * sg;
        }
        const float da = ex2_approx(d[i] * Av[e]);
        const float G = fmaf(cv[e], dyv, carry[e]);
        dco[e] = dyv * st[i][e];
        dbo[e] = G * d[i] * x[e];
        dxo[e] = fmaf(dyv, Dv[e], G * d[i] * bv[e]);
        const float gsa = G * st[i + 1][e] * da;
        ddt_sum += fmaf(G, bv[e] * x[e], gsa * (Av[e] * kLn2));
        dA_acc[e] = fmaf(gsa, d[i], dA_acc[e]);
        dD_acc = fmaf(dyv, x[e], dD_acc);
        carry[e] = G * da;
      }
      if (!active) ddt_sum = 0.f;
      if (shuffle_heads) {
        for (int m = 1; m < group; m <<= 1) ddt_sum += __shfl_xor_sync(0xffffffffu, ddt_sum, m);
        if (active && (threadIdx.x & (group - 1)) == 0) atomicAdd(g.ddt + ((int64_t)b * a.len + t0 + kk) * a.heads + h, ddt_sum);
      } else if (active) {
        atomicAdd(g.ddt + ((int64_t)b * a.len + t0 + kk) * a.heads + h, ddt_sum);
      }
      if (active) {
        put8(g.dC, typed_c, oC + (int64_t)kk * g.dC.st, dco);
        put8(g.dB, typed_b, oB + (int64_t)kk * g.dB.st, dbo);
        if (has_z) put8(g.dz, typed_z, oZ + (int64_t)kk * g.dz.st, dzo);
        Vec16<T> o;
        o.pack(dxo);
        *reinterpret_cast<uint4*>(dX + (int64_t)kk * HP) = o.raw;
      }
    }
  }
  if (!active) return;
#pragma unroll
  for (int e = 0; e < V; ++e) atomicAdd(bc4_ptr(g.dA, 0, 0, h, q + e), dA_acc[e]);
  if (g.dD.ptr) atomicAdd(bc4_ptr(g.dD, 0, 0, h, 0), dD_acc);  // one skip weight per head (the launcher checks)
}

static bool bc4_dense_host(const ssm_bcast4& p) { return p.ptr && p.sb != 0 && p.st != 0 && p.sh != 0 && p.sq != 0; }

static int chunk_validate(const ssm_chunk_args* a) {
  SSM_REQUIRE(a != nullptr, SSM_ERR_NULL, "ssd_chunk_scan: args is NULL");
  SSM_REQUIRE(a->batch >= 0 && a->len >= 0 && a->heads >= 0 && a->proj >= 0, SSM_ERR_SHAPE, "ssd_chunk_scan: negative size");
  SSM_REQUIRE(a->chunk_size >= 1, SSM_ERR_SHAPE, "chunk_size must be positive.");
  SSM_REQUIRE(valid_dtype(a->io_dtype) && valid_dtype(a->par_dtype), SSM_ERR_DTYPE, "ssd_chunk_scan: unknown dtype");
  SSM_REQUIRE(a->batch <= 65535, SSM_ERR_TOO_LARGE, "ssd_chunk_scan: batch exceeds 65535");
  return SSM_OK;
}

// The recurrence does not depend on where the sequence is cut, so the forward cuts it where it suits the machine: pieces of
// at most kFwdChunkMax steps (more pieces in flight than the caller's chunk size gives at short sequences).  The scratch size
// function uses the same length.
constexpr int kFwdChunkMax = 32;
static int chunk_fwd_len(int chunk_size, int len) {
  int piece = chunk_size < kFwdChunkMax ? chunk_size : kFwdChunkMax;
  while (piece < chunk_size && ((int64_t)len + piece - 1) / piece > 65535) piece *= 2;  // the pieces are a grid axis
  return piece < chunk_size ? piece : chunk_size;
}

// 16-byte rows for the vector kernels: the projection axis contiguous and a multiple of 8, every other stride a multiple of 8
template <typename T>
static bool chunk_vec_ok(const ssm_chunk_args& a) {
  if (sizeof(T) != 2 || a.proj % 8 != 0 || a.scratch == nullptr) return false;
  auto dense8 = [](const ssm_bcast4& p) { return p.sq == 1 && p.sb % 8 == 0 && p.st % 8 == 0 && p.sh % 8 == 0 && aligned_to(p.ptr, 16); };
  if (!dense8(a.Bm) || !dense8(a.Cm) || (a.z.ptr && !dense8(a.z))) return false;
  return aligned_to(a.X, 16) && aligned_to(a.Y, 16) && aligned_to(a.scratch, 16);
}

// chunk_len: steps per piece (the backward passes the caller's chunk size, which its own scratch and history are sized by)
template <typename T, typename PT>
static int chunk_fwd_t(const ssm_chunk_args& a, cudaStream_t st, int chunk_len, bool through_phase2_only = false) {
  const int HP = a.heads * a.proj;
  const unsigned gx = (HP + kChunkThreads - 1) / kChunkThreads;
  const int nchunks = (a.len + chunk_len - 1) / chunk_len;
  if (!a.scratch || nchunks <= 1) {
    chunk_fwd_kernel<T, PT, 0><<<dim3(gx, 1, a.batch), kChunkThreads, 0, st>>>(a, 1, chunk_len);
    return launch_status("chunk_fwd_kernel<serial>");
  }
  SSM_REQUIRE(nchunks <= 65535, SSM_ERR_TOO_LARGE, "ssd_chunk_scan: more than 65535 chunks");
  const bool vec = std::is_same<T, PT>::value && chunk_vec_ok<T>(a);
  const unsigned gv = (HP / 8 + kChunkThreads - 1) / kChunkThreads;
  if constexpr (sizeof(T) == 2) {
    if (vec) chunk_fwd_vec_kernel<T, 1><<<dim3(gv, nchunks, a.batch), kChunkThreads, 0, st>>>(a, nchunks, chunk_len);
  }
  if (!vec) chunk_fwd_kernel<T, PT, 1><<<dim3(gx, nchunks, a.batch), kChunkThreads, 0, st>>>(a, nchunks, chunk_len);
  if (int rc = launch_status("chunk_fwd_kernel<local>")) return rc;
  chunk_carry_kernel<<<dim3((HP + kCarryLanes - 1) / kCarryLanes, 1, a.batch), kCarryLanes * kCarryGroups, 0, st>>>(a, nchunks);
  if (int rc = launch_status("chunk_carry_kernel")) return rc;
  if (through_phase2_only) return SSM_OK;
  if constexpr (sizeof(T) == 2) {
    if (vec) chunk_fwd_vec_kernel<T, 3><<<dim3(gv, nchunks, a.batch), kChunkThreads, 0, st>>>(a, nchunks, chunk_len);
  }
  if (!vec) chunk_fwd_kernel<T, PT, 3><<<dim3(gx, nchunks, a.batch), kChunkThreads, 0, st>>>(a, nchunks, chunk_len);
  return launch_status("chunk_fwd_kernel<apply>");
}

// The backward cuts the sequence into pieces of at most kBwdChunkMax steps, whatever the caller's chunk size: each piece is one
// serial walk per thread (replay, then the walk back), and short pieces are what puts enough of them in flight.
constexpr int kBwdChunkMax = 32;
static int chunk_bwd_len(int chunk_size, int len) {
  int piece = chunk_size < kBwdChunkMax ? chunk_size : kBwdChunkMax;
  while (piece < chunk_size && ((int64_t)len + piece - 1) / piece > 65535) piece *= 2;  // the pieces are a grid axis
  return piece < chunk_size ? piece : chunk_size;
}

template <typename T, typename PT>
static int chunk_bwd_t(const ssm_chunk_bwd_args& g_in, cudaStream_t st) {
  ssm_chunk_bwd_args g = g_in;
  g.fwd.chunk_size = chunk_bwd_len(g_in.fwd.chunk_size, g_in.fwd.len);  // the kernels cut the sequence by this field
  const ssm_chunk_args& a = g.fwd;
  const int HP = a.heads * a.proj;
  const unsigned gx = (HP + kChunkThreads - 1) / kChunkThreads;
  const int nchunks = (a.len + a.chunk_size - 1) / a.chunk_size;
  if (!g.scratch || nchunks <= 1 || nchunks > 65535) {
    chunk_bwd_kernel<T, PT, 0><<<dim3(gx, 1, a.batch), kChunkThreads, 0, st>>>(g, 1);
    return launch_status("chunk_bwd_kernel<serial>");
  }
  // states entering every chunk (forward phases 1 and 2 on the backward call's scratch; no final state, no Y)
  ssm_chunk_args f = a;
  f.scratch = g.scratch, f.final_state = nullptr;
  if (int rc = chunk_fwd_t<T, PT>(f, st, a.chunk_size, true)) return rc;
  bool local_vec = false;
  if constexpr (sizeof(T) == 2 && std::is_same<T, PT>::value) {
    ssm_chunk_args f2 = a;
    f2.scratch = g.scratch;
    f2.Y = g.dX;  // only its alignment is looked at
    local_vec = chunk_vec_ok<T>(f2) && aligned_to(g.dY, 16);
    if (local_vec) {
      const unsigned gv = (HP / 8 + kChunkThreads - 1) / kChunkThreads;
      chunk_bwd_local_vec_kernel<T><<<dim3(gv, nchunks, a.batch), kChunkThreads, 0, st>>>(g, nchunks);
    }
  }
  if (!local_vec) chunk_bwd_local_kernel<T, PT><<<dim3(gx, nchunks, a.batch), kChunkThreads, 0, st>>>(g, nchunks);
  if (int rc = launch_status("chunk_bwd_local_kernel")) return rc;
  chunk_bwd_carry_kernel<<<dim3((HP + kCarryLanes - 1) / kCarryLanes, 1, a.batch), kCarryLanes * kCarryGroups, 0, st>>>(g, nchunks);
  if (int rc = launch_status("chunk_bwd_carry_kernel")) return rc;
  if constexpr (sizeof(T) == 2 && std::is_same<T, PT>::value) {
    // 16-byte lanes: dense 16-bit B, C, z (see chunk_vec_ok), dense fp32 gradient buffers for them with 16-byte rows, and a
    // skip weight per head (or none), whose gradient is then one sum per thread
    // (a broadcast axis, stride 0, would make several steps write one element: those buffers keep the atomic path)
    auto dense4 = [](const ssm_bcast4& p) {  // multiples of 8 elements: 16-byte rows whether the buffer is fp32 or 16-bit
      return p.ptr && p.sq == 1 && p.sb != 0 && p.st != 0 && p.sh != 0 && p.sb % 8 == 0 && p.st % 8 == 0 && p.sh % 8 == 0 && aligned_to(p.ptr, 16);
    };
    ssm_chunk_args f2 = a;
    f2.scratch = g.scratch;
    f2.Y = g.dX;  // only its alignment is looked at
    const bool vec = chunk_vec_ok<T>(f2) && dense4(g.dB) && dense4(g.dC) && (!a.z.ptr || dense4(g.dz)) && (!a.D.ptr || !g.dD.ptr || a.D.sq == 0) &&
                     aligned_to(g.dY, 16) && aligned_to(g.history, 16) && (a.heads * a.proj) % 8 == 0;
    if (vec) {
      const unsigned gv = (a.heads * a.proj / 8 + kChunkThreads - 1) / kChunkThreads;
      chunk_bwd_vec_kernel<T><<<dim3(gv, nchunks, a.batch), kChunkThreads, 0, st>>>(g, nchunks);
      return launch_status("chunk_bwd_vec_kernel");
    }
  }
  chunk_bwd_kernel<T, PT, 1><<<dim3(gx, nchunks, a.batch), kChunkThreads, 0, st>>>(g, nchunks);
  return launch_status("chunk_bwd_kernel");
}

}  // namespace ssmb

using namespace ssmb;

extern "C" int64_t ssm_chunk_scan_scratch_floats(int32_t batch, int32_t len, int32_t heads, int32_t proj, int32_t chunk_size) {
  if (chunk_size < 1) return 0;
  const int64_t piece = chunk_fwd_len(chunk_size, len);
  const int64_t nchunks = (len + piece - 1) / piece;
  return 2 * (int64_t)batch * nchunks * heads * proj;
}

extern "C" int64_t ssm_chunk_scan_bwd_scratch_floats(int32_t batch, int32_t len, int32_t heads, int32_t proj, int32_t chunk_size) {
  if (chunk_size < 1) return 0;
  const int64_t piece = chunk_bwd_len(chunk_size, len);
  const int64_t nchunks = (len + piece - 1) / piece;
  return 3 * (int64_t)batch * nchunks * heads * proj;  // decay products, states entering, adjoints entering every chunk
}

extern "C" int ssm_chunk_scan_fwd(const ssm_chunk_args* a, ssm_stream_t stream) {
  if (a && a->io_dtype == SSM_F64) {
    ssm_chunk_bwd_args g{};
    g.fwd = *a;
    return f64_chunk(g, false, reinterpret_cast<cudaStream_t>(stream));
  }
  if (int rc = chunk_validate(a)) return rc;
  if (a->batch == 0 || a->heads == 0 || a->proj == 0) return SSM_OK;
  SSM_REQUIRE(a->A.ptr && a->Bm.ptr && a->Cm.ptr, SSM_ERR_NULL, "ssd_chunk_scan: A, B and C are required");
  SSM_REQUIRE(a->len == 0 || (a->X && a->dt && a->Y), SSM_ERR_NULL, "ssd_chunk_scan: X, dt and Y are required");
  SSM_REQUIRE(a->par_dtype == a->io_dtype || a->par_dtype == SSM_F32, SSM_ERR_UNSUPPORTED,
              "ssd_chunk_scan: B, C and z must have the element type of X, or float32");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool same = a->par_dtype == a->io_dtype;
  const int cl = chunk_fwd_len(a->chunk_size, a->len);
  switch (a->io_dtype) {
    case SSM_F32: return chunk_fwd_t<float, float>(*a, st, cl);
    case SSM_BF16: return same ? chunk_fwd_t<__nv_bfloat16, __nv_bfloat16>(*a, st, cl) : chunk_fwd_t<__nv_bfloat16, float>(*a, st, cl);
    default: return same ? chunk_fwd_t<__half, __half>(*a, st, cl) : chunk_fwd_t<__half, float>(*a, st, cl);
  }
}

extern "C" int ssm_chunk_scan_bwd(const ssm_chunk_bwd_args* g, ssm_stream_t stream) {
  SSM_REQUIRE(g != nullptr, SSM_ERR_NULL, "ssd_chunk_scan_backward: args is NULL");
  const ssm_chunk_args* a = &g->fwd;
  if (a->io_dtype == SSM_F64) return f64_chunk(*g, true, reinterpret_cast<cudaStream_t>(stream));
  if (int rc = chunk_validate(a)) return rc;
  if (a->batch == 0 || a->heads == 0 || a->proj == 0 || a->len == 0) return SSM_OK;
  SSM_REQUIRE(a->A.ptr && a->Bm.ptr && a->Cm.ptr && a->X && a->dt, SSM_ERR_NULL, "ssd_chunk_scan_backward: missing input");
  SSM_REQUIRE(g->dY && g->dX && g->ddt && g->dA.ptr && g->dB.ptr && g->dC.ptr && g->history, SSM_ERR_NULL,
              "ssd_chunk_scan_backward: missing gradient buffer");
  SSM_REQUIRE(!a->z.ptr || g->dz.ptr, SSM_ERR_NULL, "ssd_chunk_scan_backward: dz is required when z is given");
  SSM_REQUIRE((a->typed_grads & ~7) == 0 && (!(a->typed_grads & 1) || bc4_dense_host(g->dB)) && (!(a->typed_grads & 2) || bc4_dense_host(g->dC)) &&
                  (!(a->typed_grads & 4) || (a->z.ptr && bc4_dense_host(g->dz))),
              SSM_ERR_SHAPE, "ssd_chunk_scan_backward: a typed gradient buffer must have no broadcast axis");
  SSM_REQUIRE(a->par_dtype == a->io_dtype || a->par_dtype == SSM_F32, SSM_ERR_UNSUPPORTED,
              "ssd_chunk_scan_backward: B, C and z must have the element type of X, or float32");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool same = a->par_dtype == a->io_dtype;
  switch (a->io_dtype) {
    case SSM_F32: return chunk_bwd_t<float, float>(*g, st);
    case SSM_BF16: return same ? chunk_bwd_t<__nv_bfloat16, __nv_bfloat16>(*g, st) : chunk_bwd_t<__nv_bfloat16, float>(*g, st);
    default: return same ? chunk_bwd_t<__half, __half>(*g, st) : chunk_bwd_t<__half, float>(*g, st);
  }
}
