// Mamba-1 selective scan, forward: the fast path for vectorisable inputs whose rows share B / C
// (one B / C group per CTA, 16-byte aligned rows, d_state <= 32).
//
// A CTA owns 32 channel rows of one batch element.  LANE = ROW and WARP = STATE GROUP: warp g
// keeps states 4g .. 4g+3 of all 32 rows in registers, time is walked sequentially in tiles of
// 32 steps.  What this mapping buys over "lanes = rows x state groups":
//   * B_t and C_t of a warp's four states are the same for all of its lanes, so each is ONE
//     16-byte shared-memory load with a single, fully broadcast wavefront (the kernel is bound by
//     shared-memory wavefronts and the special-function unit, not by HBM);
//   * the per-row operands (delta, delta*u) are staged as (dl, dl, du, du) in a swizzled array:
//     one conflict-free 16-byte load per step hands the packed-fp32 (f32x2) multiplies both of
//     their operand pairs without register moves;
//   * the contraction <C, h> over the state groups is a sum over warps: every warp stores its
//     partial sums (16 bytes per 4 steps and lane) and the epilogue adds them while it forms the
//     output, so the recurrence contains no shuffle and no reduction at all.
// The operands of step group g+1 (loads, decay exponent, ex2, delta*u*B) are issued before the
// dependent multiply-adds of group g, which software-pipelines the one serial chain (the state).
// Global -> shared copies of u / delta / z (cp.async, 16 bytes) run a tile ahead into double-buffered raw tiles; the
// raw u / z of a tile stay valid until its epilogue, where the skip term D*u and the gate silu(z) are applied.  The
// small B / C tiles travel through registers (one 16-byte chunk per thread, fetched a tile ahead).  Per (row, state, step): one ex2.approx and four packed-fp32 issue slots.
#pragma once

#include "scan_common.cuh"

namespace ssmb {

constexpr int kTileRows = 32;  // rows per CTA (one per lane)

template <typename T, int NG>
struct FwdTiles {
  static constexpr int NP = 4 * NG;     // padded state count
  static constexpr int TL = kScanCkpt;  // one tile = one checkpoint interval
  static constexpr int TLP = TL + 4;
  static constexpr int V = 16 / (int)sizeof(T);
  static constexpr int NT = NG * 32;
  // bytes
  static constexpr int RAW_ROWS = 3 * kTileRows * TL * (int)sizeof(T);  // u, delta, z of one tile
  static constexpr int DD = kTileRows * TL * 16;                        // (dl, dl, du, du) per (row, step)
  static constexpr int PART = NG * kTileRows * TLP * 4;                 // partial sums [group][row][TLP]
  static constexpr int BC_F32 = 2 * TL * NP * 4;                        // B and C as fp32 [TL][NP]
  static constexpr size_t kBytes = BC_F32 + 2 * RAW_ROWS + DD + PART;
  static_assert(kBytes <= 227 * 1024, "shared memory budget");
};

// Slot of (row, step) in the (dl, dl, du, du) array.  The low three bits of the step are XOR-ed with bits of the chunk
// index and of the row so that both the threads that write a tile (8 or 4 consecutive steps each, 128 bytes apart) and
// the lanes that read one step of 32 different rows (512 bytes apart) spread over all eight 16-byte bank groups.
__device__ __forceinline__ int dd_slot(int rr, int tt) {
  return rr * kScanCkpt + ((tt & ~7) | ((tt & 7) ^ ((tt >> 3) & 3) ^ ((rr & 1) << 2) ^ ((rr >> 1) & 3)));
}

struct FwdStepOps {  // everything of one step that does not depend on the state
  float2 da0, da1, db0, db1, c0, c1;
};

// MODE 0: the whole sequence per CTA.  MODE 1 / 2: the sequence is cut into gridDim.z segments of `seg_tiles` tiles that run in
// parallel (for calls whose rows alone cannot fill the machine): pass 1 integrates every segment from a zero state (segment 0:
// from the initial state) and leaves its end state and decay product exp(A sum delta) in `split`; after the serial combine
// (scan_split_combine_kernel) pass 2 replays every segment from its true incoming state and produces the outputs.
template <typename T, int NG, int MODE>
__global__ void __launch_bounds__(NG * 32, NG <= 4 ? 3 : 1) scan_fwd_tiles_kernel(const ssm_scan_fwd_args a, const ScanFlags fl, int seg_tiles) {
  using M = FwdTiles<T, NG>;
  constexpr int NP = M::NP, TL = M::TL, TLP = M::TLP, V = M::V, NT = M::NT;
  constexpr int CH = TL / V;  // 16-byte chunks per row and tile
  constexpr int ROWS = kTileRows;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, grp = tid >> 5;
  float* sB = reinterpret_cast<float*>(smem_raw);  // [TL][NP]
  float* sC = sB + TL * NP;
  unsigned char* rbase = smem_raw + M::BC_F32;
  T* rawrows = reinterpret_cast<T*>(rbase);                                     // [2 buffers][u | delta | z][ROWS][TL]
  float4* sDD = reinterpret_cast<float4*>(rbase + 2 * M::RAW_ROWS);             // [ROWS][TL], swizzled
  float* sP = reinterpret_cast<float*>(rbase + 2 * M::RAW_ROWS + M::DD);        // [NG][ROWS][TLP]

  const int b = blockIdx.y;
  const int d0 = blockIdx.x * ROWS;
  const int N = a.nstate, L = a.len, D = a.dim;
  const bool row_ok = d0 + lane < D;
  const int d = row_ok ? d0 + lane : D - 1;
  const int64_t row = (int64_t)b * D + d;

  const T* __restrict__ gu = reinterpret_cast<const T*>(a.u);
  const T* __restrict__ gdl = reinterpret_cast<const T*>(a.delta);
  const T* __restrict__ gz = reinterpret_cast<const T*>(a.z);
  T* __restrict__ gout = reinterpret_cast<T*>(a.out);
  const bool has_z = gz != nullptr;

  float2 A2[2], h[2];
#pragma unroll
  for (int j = 0; j < 4; j += 2) {
    const int n = grp * 4 + j;
    A2[j / 2].x = n < N ? __ldg(a.A + (int64_t)d * N + n) * kLog2e : 0.f;
    A2[j / 2].y = n + 1 < N ? __ldg(a.A + (int64_t)d * N + n + 1) * kLog2e : 0.f;
    h[j / 2].x = (n < N && a.initial_state) ? __ldg(a.initial_state + row * N + n) : 0.f;
    h[j / 2].y = (n + 1 < N && a.initial_state) ? __ldg(a.initial_state + row * N + n + 1) : 0.f;
  }
  const int seg = MODE == 0 ? 0 : blockIdx.z, nseg = MODE == 0 ? 1 : gridDim.z;
  // split scratch: [2][batch][dim][nseg][N]: end state / incoming state, then decay product
  float* split_h = MODE == 0 ? nullptr : a.split_scratch + ((row * nseg + seg) * (int64_t)N);
  float* split_p = MODE == 0 ? nullptr : split_h + (int64_t)a.batch * D * nseg * N;
  if (MODE == 1 && seg > 0) h[0] = h[1] = make_float2(0.f, 0.f);
  if (MODE == 2 && seg > 0) {  // segment 0 starts from the call's initial state, loaded above
#pragma unroll
    for (int j = 0; j < 4; j += 2) {
      const int n = grp * 4 + j;
      h[j / 2].x = n < N ? split_h[n] : 0.f;
      h[j / 2].y = n + 1 < N ? split_h[n + 1] : 0.f;
    }
  }
  float sumdl = 0.f;  // MODE 1: sum of this row's delta over the segment

  const int64_t boff = bc_row_offset(b, min(d0, D - 1), fl.rows_per_group, a.b_sb, a.b_sg);
  const int64_t coff = bc_row_offset(b, min(d0, D - 1), fl.rows_per_group, a.c_sb, a.c_sg);

  const int ntiles = (L + TL - 1) / TL;
  const int k_begin = MODE == 0 ? 0 : seg * seg_tiles;
  const int k_end = MODE == 0 ? ntiles : min(ntiles, k_begin + seg_tiles);

  // ---- B / C tiles travel through registers: one 16-byte chunk (8 or 4 steps of one state) per thread and slot, fetched a
  // ---- tile ahead with a plain vector load and written to the fp32 [step][state] tiles when its tile starts
  const int bc_esz = a.bc_dtype == SSM_F32 ? 4 : 2;
  const int bc_per = 16 / bc_esz;                                 // steps per chunk
  constexpr int kBcSlots = (2 * NP * (TL / 4) + NT - 1) / NT;     // enough for fp32 coefficients
  uint4 bcreg[kBcSlots];
  const char* bc_src[kBcSlots];  // this thread's chunk of tile 0 (NULL: no chunk in this slot)
  float* bc_dst[kBcSlots];
  int bc_tt[kBcSlots];
#pragma unroll
  for (int s_ = 0; s_ < kBcSlots; ++s_) {
    const int c = tid + s_ * NT;
    const int per_op = N * (TL / bc_per);  // chunks of B (then the same number for C); within each: state fastest
    bc_src[s_] = nullptr, bc_dst[s_] = sB, bc_tt[s_] = 0;
    if (c < 2 * per_op) {
      const int which = c / per_op, rem = c % per_op;
      const int n = rem % N, tt = (rem / N) * bc_per;
      bc_tt[s_] = tt;
      bc_dst[s_] = (which ? sC : sB) + tt * NP + n;
      bc_src[s_] = which ? reinterpret_cast<const char*>(a.Cm) + (coff + (int64_t)n * a.c_sn + tt) * bc_esz
                         : reinterpret_cast<const char*>(a.Bm) + (boff + (int64_t)n * a.b_sn + tt) * bc_esz;
    }
  }
  auto bc_fetch = [&](int k) {
#pragma unroll
    for (int s_ = 0; s_ < kBcSlots; ++s_) {
      bcreg[s_] = make_uint4(0u, 0u, 0u, 0u);
      if (bc_src[s_] && k * TL + bc_tt[s_] < L) bcreg[s_] = __ldg(reinterpret_cast<const uint4*>(bc_src[s_] + (int64_t)k * TL * bc_esz));
    }
  };
  auto bc_store = [&]() {
#pragma unroll
    for (int s_ = 0; s_ < kBcSlots; ++s_) {
      if (bc_src[s_]) {
        float* dst = bc_dst[s_];
        if (a.bc_dtype == SSM_F32) {
          const float* f = reinterpret_cast<const float*>(&bcreg[s_]);
#pragma unroll
          for (int i = 0; i < 4; ++i) dst[i * NP] = f[i];
        } else if (a.bc_dtype == SSM_BF16) {
          const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&bcreg[s_]);
#pragma unroll
          for (int i = 0; i < 8; ++i) dst[i * NP] = __bfloat162float(e[i]);
        } else {
          const __half* e = reinterpret_cast<const __half*>(&bcreg[s_]);
#pragma unroll
          for (int i = 0; i < 8; ++i) dst[i * NP] = __half2float(e[i]);
        }
      }
    }
  };
  if (N < NP) {  // padded states read as zero for the whole launch
    for (int i = tid; i < 2 * TL * NP; i += NT) sB[i] = 0.f;
  }

  // one 16-byte chunk of u / delta / z per (row, chunk) and thread; out-of-range steps are zero-filled
  auto fill_raw = [&](int k) {
    const int t0 = k * TL;
    T* rr = rawrows + (k & 1) * (3 * ROWS * TL);
    for (int c = tid; c < ROWS * CH; c += NT) {
      const int r_ = c / CH, ch = c % CH;
      const int dd = min(d0 + r_, D - 1);
      const int t = t0 + ch * V;
      const bool ok = t < L;
      const int64_t off = (int64_t)b * a.row_sb + (int64_t)dd * a.row_sd + (ok ? t : 0);
      cp_async16(rr + r_ * TL + ch * V, gu + off, ok);
      cp_async16(rr + ROWS * TL + r_ * TL + ch * V, gdl + off, ok);
      if (has_z) cp_async16(rr + 2 * ROWS * TL + r_ * TL + ch * V, gz + off, ok);
    }
    cp_async_commit();
  };

  if (k_begin < k_end) {
    fill_raw(k_begin);
    bc_fetch(k_begin);
  }

  for (int k = k_begin; k < k_end; ++k) {
    const int t0 = k * TL;
    cp_async_wait_all();
    __syncthreads();  // raw tile k has landed for every thread; the other raw buffer, the fp32 tiles and the partials are free
    if (k + 1 < k_end) fill_raw(k + 1);

    const T* rawU = rawrows + (k & 1) * (3 * ROWS * TL);
    const T* rawD = rawU + ROWS * TL;
    const T* rawZ = rawD + ROWS * TL;

    // ---- delta (bias, softplus) and delta*u as fp32 operand pairs ---------------------------
    {
      const bool tail = t0 + TL > L;
      for (int c = tid; c < ROWS * CH; c += NT) {
        const int rr = c / CH, ch = c % CH;
        const int dd = min(d0 + rr, D - 1);
        float fu[V], fd[V];
        Vec16<T> v;
        v.raw = *reinterpret_cast<const uint4*>(rawU + rr * TL + ch * V);
        v.unpack(fu);
        v.raw = *reinterpret_cast<const uint4*>(rawD + rr * TL + ch * V);
        v.unpack(fd);
        const float bias = a.dt_bias ? __ldg(a.dt_bias + dd) : 0.f;
        if (a.delta_softplus) {
#pragma unroll
          for (int i = 0; i < V; ++i) fd[i] = sizeof(T) == 2 ? softplus_half_io(fd[i] + bias) : softplus_fast(fd[i] + bias);
        } else {
#pragma unroll
          for (int i = 0; i < V; ++i) fd[i] += bias;
        }
        if (tail) {  // steps beyond the sequence leave the state untouched
#pragma unroll
          for (int i = 0; i < V; ++i)
            if (t0 + ch * V + i >= L) fd[i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const float xu = fd[i] * fu[i];
          sDD[dd_slot(rr, ch * V + i)] = make_float4(fd[i], fd[i], xu, xu);
        }
      }
    }
    bc_store();
    if (k + 1 < k_end) bc_fetch(k + 1);  // lands while this tile is being processed
    __syncthreads();  // fp32 tiles ready

    // ---- recurrence over the tile ----------------------------------------------------------
    if (MODE != 1 && a.checkpoints && row_ok) {
      float* ck = a.checkpoints + (row * ntiles + k) * N + grp * 4;
      if (grp * 4 + 3 < N && (N & 3) == 0) {
        *reinterpret_cast<float4*>(ck) = make_float4(h[0].x, h[0].y, h[1].x, h[1].y);
      } else {
        if (grp * 4 < N) ck[0] = h[0].x;
        if (grp * 4 + 1 < N) ck[1] = h[0].y;
        if (grp * 4 + 2 < N) ck[2] = h[1].x;
        if (grp * 4 + 3 < N) ck[3] = h[1].y;
      }
    }
    {
      const float* pB = sB + grp * 4;
      const float* pC = sC + grp * 4;
      float* pP = sP + (grp * ROWS + lane) * TLP;
      auto prepare = [&](int tt) {
        FwdStepOps o;
        const float4 dd4 = sDD[dd_slot(lane, tt)];
        const float4 b4 = *reinterpret_cast<const float4*>(pB + tt * NP);
        const float4 c4 = *reinterpret_cast<const float4*>(pC + tt * NP);
        const float2 dl2 = make_float2(dd4.x, dd4.y), du2 = make_float2(dd4.z, dd4.w);
        const float2 e0 = __fmul2_rn(dl2, A2[0]), e1 = __fmul2_rn(dl2, A2[1]);
        o.da0 = make_float2(ex2_approx(e0.x), ex2_approx(e0.y));
        o.da1 = make_float2(ex2_approx(e1.x), ex2_approx(e1.y));
        o.db0 = __fmul2_rn(du2, make_float2(b4.x, b4.y));
        o.db1 = __fmul2_rn(du2, make_float2(b4.z, b4.w));
        o.c0 = make_float2(c4.x, c4.y), o.c1 = make_float2(c4.z, c4.w);
        if (MODE == 1) sumdl += dd4.x;
        return o;
      };
      FwdStepOps cur[4], nxt[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) cur[i] = prepare(i);
#pragma unroll
      for (int q = 0; q < TL; q += 4) {
        if (q + 4 < TL) {
#pragma unroll
          for (int i = 0; i < 4; ++i) nxt[i] = prepare(q + 4 + i);
        }
        float p[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          h[0] = __ffma2_rn(cur[i].da0, h[0], cur[i].db0);
          h[1] = __ffma2_rn(cur[i].da1, h[1], cur[i].db1);
          if (MODE != 1) {
            const float2 acc = __ffma2_rn(cur[i].c1, h[1], __fmul2_rn(cur[i].c0, h[0]));
            p[i] = acc.x + acc.y;
          }
        }
        if (MODE != 1) *reinterpret_cast<float4*>(pP + q) = make_float4(p[0], p[1], p[2], p[3]);
#pragma unroll
        for (int i = 0; i < 4; ++i) cur[i] = nxt[i];
      }
    }
    __syncthreads();  // every state group's partial sums are in place
    if (MODE == 1) continue;  // pass 1 of a split call produces no output

    // ---- epilogue: add the state groups' partial sums, skip term, gate, store ---------------------
    for (int c = tid; c < ROWS * CH; c += NT) {
      const int rr = c / CH, ch = c % CH;
      const int dd = d0 + rr;
      const int t = t0 + ch * V;
      if (dd < D && t < L) {
        float y[V], fu[V], fz[V];
#pragma unroll
        for (int i = 0; i < V; ++i) y[i] = 0.f;
#pragma unroll
        for (int s = 0; s < NG; ++s) {
          const float* src = sP + (s * ROWS + rr) * TLP + ch * V;
#pragma unroll
          for (int i = 0; i < V; i += 4) {
            const float4 q4 = *reinterpret_cast<const float4*>(src + i);
            y[i] += q4.x, y[i + 1] += q4.y, y[i + 2] += q4.z, y[i + 3] += q4.w;
          }
        }
        Vec16<T> v;
        v.raw = *reinterpret_cast<const uint4*>(rawU + rr * TL + ch * V);
        v.unpack(fu);
        const float Dv = a.D ? __ldg(a.D + dd) : 0.f;
        if (has_z) {
          v.raw = *reinterpret_cast<const uint4*>(rawZ + rr * TL + ch * V);
          v.unpack(fz);
#pragma unroll
          for (int i = 0; i < V; ++i) y[i] = fmaf(Dv, fu[i], y[i]) * silu_fast(fz[i]);
        } else {
#pragma unroll
          for (int i = 0; i < V; ++i) y[i] = fmaf(Dv, fu[i], y[i]);
        }
        v.pack(y);
        v.store_stream(gout + (int64_t)b * a.row_sb + (int64_t)dd * a.row_sd + t);
      }
    }
  }

  if (MODE == 1) {
    if (row_ok) {
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const int n = grp * 4 + j;
        if (n < N) split_h[n] = h[j / 2].x, split_p[n] = ex2_approx(sumdl * A2[j / 2].x);
        if (n + 1 < N) split_h[n + 1] = h[j / 2].y, split_p[n + 1] = ex2_approx(sumdl * A2[j / 2].y);
      }
    }
    return;
  }
  if (a.last_state && row_ok && seg == nseg - 1) {
#pragma unroll
    for (int j = 0; j < 4; j += 2) {
      const int n = grp * 4 + j;
      if (n < N) store_dyn(a.last_state, row * N + n, a.last_dtype, h[j / 2].x);
      if (n + 1 < N) store_dyn(a.last_state, row * N + n + 1, a.last_dtype, h[j / 2].y);
    }
  }
}

// Serial pass over the segments of a split call: split_h[s] <- state entering segment s.  One thread per (row, state).
static __global__ void __launch_bounds__(128) scan_split_combine_kernel(float* __restrict__ split, int64_t rows_states, int nstate, int nseg) {
  const int64_t i = (int64_t)blockIdx.x * 128 + threadIdx.x;
  if (i >= rows_states) return;
  const int64_t row = i / nstate;
  const int n = (int)(i % nstate);
  float* hs = split + row * nseg * nstate + n;
  const float* ps = hs + rows_states * nseg;
  float h = 0.f;  // segment 0 was integrated from the call's initial state already
  for (int s_ = 0; s_ < nseg; ++s_) {
    const float local = hs[(int64_t)s_ * nstate];
    hs[(int64_t)s_ * nstate] = h;
    h = s_ == 0 ? local : fmaf(ps[(int64_t)s_ * nstate], h, local);
  }
}

// Segments of a split call: enough to offer every SM about two CTAs, every segment at least four tiles long; 1 = no split.
static inline int fwd_split_segments(int batch, int dim, int len) {
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t ctas = (int64_t)batch * ((dim + kTileRows - 1) / kTileRows);
  const int tiles = (len + kScanCkpt - 1) / kScanCkpt;
  if (ctas >= sms || tiles < 8) return 1;
  int64_t want = (2 * sms + ctas - 1) / ctas;
  const int most = tiles / 4;
  if (want > most) want = most;
  return want < 2 ? 1 : (int)want;
}

template <typename T, int NG>
static int launch_fwd_tiles(const ssm_scan_fwd_args& a, const ScanFlags& fl, cudaStream_t st) {
  using M = FwdTiles<T, NG>;
  const int ntiles = (a.len + kScanCkpt - 1) / kScanCkpt;
  const int nseg = a.split_scratch && a.split_segments > 1 ? a.split_segments : 1;
  const unsigned gx = (a.dim + kTileRows - 1) / kTileRows;
  if (nseg <= 1) {
    auto kern = scan_fwd_tiles_kernel<T, NG, 0>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)M::kBytes);
    kern<<<dim3(gx, a.batch), NG * 32, M::kBytes, st>>>(a, fl, ntiles);
    return launch_status("scan_fwd_tiles_kernel");
  }
  const int seg_tiles = (ntiles + nseg - 1) / nseg;
  const int used = (ntiles + seg_tiles - 1) / seg_tiles;  // segments that hold at least one tile
  auto k1 = scan_fwd_tiles_kernel<T, NG, 1>;
  auto k2 = scan_fwd_tiles_kernel<T, NG, 2>;
  cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)M::kBytes);
  cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)M::kBytes);
  k1<<<dim3(gx, a.batch, used), NG * 32, M::kBytes, st>>>(a, fl, seg_tiles);
  if (int rc = launch_status("scan_fwd_tiles_kernel<local>")) return rc;
  const int64_t rs = (int64_t)a.batch * a.dim * a.nstate;
  scan_split_combine_kernel<<<(unsigned)((rs + 127) / 128), 128, 0, st>>>(a.split_scratch, rs, a.nstate, used);
  if (int rc = launch_status("scan_split_combine_kernel")) return rc;
  k2<<<dim3(gx, a.batch, used), NG * 32, M::kBytes, st>>>(a, fl, seg_tiles);
  return launch_status("scan_fwd_tiles_kernel<final>");
}

// True when the tile kernel covers this call: vectorisable rows and coefficients and a CTA's 32 rows inside one
// B / C group.
static inline bool fwd_tiles_ok(const ssm_scan_fwd_args& a, const ScanFlags& fl) {
  return fl.io_vec && fl.bc_vec && a.b_st == 1 && a.c_st == 1 && (fl.rows_per_group % kTileRows == 0) && a.len > 0 && a.nstate <= 32;
}

template <typename T>
static int dispatch_fwd_tiles(const ssm_scan_fwd_args& a, const ScanFlags& fl, cudaStream_t st) {
  const int ng = (a.nstate + 3) / 4;
  if (ng <= 1) return launch_fwd_tiles<T, 1>(a, fl, st);
  if (ng <= 2) return launch_fwd_tiles<T, 2>(a, fl, st);
  if (ng <= 4) return launch_fwd_tiles<T, 4>(a, fl, st);
  return launch_fwd_tiles<T, 8>(a, fl, st);
}

}  // namespace ssmb
