// Mamba-1 selective scan, forward, for sm_100a.
//
// Work decomposition (see scan_common.cuh): lanes = rows x state groups, time sequential.
// Per (row, state, step) the kernel spends one ex2.approx plus packed-fp32 (f32x2) multiply
// and fused multiply-adds on pairs of states: the decay exponent, the state update and the
// output contribution.  The <C, h> contraction over states is a register reduce-scatter
// across the LPR lanes of the row, amortised over TB steps.  B and C tiles are read from
// global memory once per CTA (ROWS channel rows share them), u / delta / z once, out
// written once; the next tile's loads (cp.async) overlap the current tile's recurrence.
#pragma once

#include "scan_common.cuh"
#include "selective_scan_fwd_tiles.cuh"

namespace ssmb {

template <typename T, int NS, int LPR, bool SHARED>
struct FwdSmem {
  using S = ScanShape<NS, LPR>;
  static constexpr int TL = (S::NP <= 32 && S::RPW <= 8) ? 64 : 32;
  static constexpr int TLP = TL + 4;
  // floats
  static constexpr int BC_WORK = SHARED ? 2 * TL * S::NP : 0;
  static constexpr int WARP_WORK = 4 * S::RPW * TLP;
  // bytes
  static constexpr int BC_RAW_BYTES = SHARED ? 2 * S::NP * TL * 4 : 0;
  static constexpr int WARP_RAW_BYTES = 3 * S::RPW * TL * (int)sizeof(T);
  static constexpr size_t kBytes = sizeof(float) * (BC_WORK + kScanWarps * WARP_WORK) + BC_RAW_BYTES + kScanWarps * WARP_RAW_BYTES;
  static_assert(kBytes <= 227 * 1024, "shared memory budget");
  static constexpr size_t bytes() { return kBytes; }
};

template <typename T, int NS, int LPR, bool SHARED, int UNROLL = 2>
__global__ void __launch_bounds__(kScanWarps * 32) scan_fwd_kernel(const ssm_scan_fwd_args a, const ScanFlags fl) {
  using S = ScanShape<NS, LPR>;
  using M = FwdSmem<T, NS, LPR, SHARED>;
  constexpr int NP = S::NP, RPW = S::RPW, ROWS = S::ROWS, TB = S::TB;
  constexpr int TL = M::TL, TLP = M::TLP;
  constexpr int V = 16 / sizeof(T);
  constexpr int NT = kScanWarps * 32;
  static_assert(TL % TB == 0 && TL % kScanCkpt == 0, "tile must hold whole batches and checkpoints");
  static_assert(NS % 2 == 0, "states are processed in pairs");

  extern __shared__ __align__(16) float smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* sB = smem;                                          // [TL][NP]
  float* sC = sB + M::BC_WORK / 2;                           // [TL][NP]
  float* sDl = smem + M::BC_WORK + warp * M::WARP_WORK;      // per warp: [RPW][TLP] x 4
  float* sDu = sDl + RPW * TLP;
  float* sY = sDu + RPW * TLP;
  float* sG = sY + RPW * TLP;
  char* rawbase = reinterpret_cast<char*>(smem + M::BC_WORK + kScanWarps * M::WARP_WORK);
  char* rawB = rawbase;                                      // [NP][TL] source dtype (or fp32)
  char* rawC = rawbase + M::BC_RAW_BYTES / 2;
  T* rawU = reinterpret_cast<T*>(rawbase + M::BC_RAW_BYTES + warp * M::WARP_RAW_BYTES);  // [RPW][TL]
  T* rawD = rawU + RPW * TL;
  T* rawZ = rawD + RPW * TL;

  const int b = blockIdx.y;
  const int d0 = blockIdx.x * ROWS;
  const int N = a.nstate, L = a.len, D = a.dim;
  const int r = lane / LPR, sg = lane % LPR;
  const int drow0 = d0 + warp * RPW;
  const int d_raw = drow0 + r;
  const bool row_ok = d_raw < D;
  const int d = row_ok ? d_raw : D - 1;
  const int64_t row = (int64_t)b * D + d;

  const T* __restrict__ gu = reinterpret_cast<const T*>(a.u);
  const T* __restrict__ gdl = reinterpret_cast<const T*>(a.delta);
  const T* __restrict__ gz = reinterpret_cast<const T*>(a.z);
  T* __restrict__ gout = reinterpret_cast<T*>(a.out);

  // per-lane state, held as pairs for the packed-fp32 pipe
  float2 A2[NS / 2], h[NS / 2];
#pragma unroll
  for (int j = 0; j < NS; j += 2) {
    const int n = sg * NS + j;
    A2[j / 2].x = n < N ? __ldg(a.A + (int64_t)d * N + n) * kLog2e : 0.f;
    A2[j / 2].y = n + 1 < N ? __ldg(a.A + (int64_t)d * N + n + 1) * kLog2e : 0.f;
    h[j / 2].x = (n < N && a.initial_state) ? __ldg(a.initial_state + row * N + n) : 0.f;
    h[j / 2].y = (n + 1 < N && a.initial_state) ? __ldg(a.initial_state + row * N + n + 1) : 0.f;
  }

  const int64_t boff = bc_row_offset(b, SHARED ? min(d0, D - 1) : d, fl.rows_per_group, a.b_sb, a.b_sg);
  const int64_t coff = bc_row_offset(b, SHARED ? min(d0, D - 1) : d, fl.rows_per_group, a.c_sb, a.c_sg);
  const int bcsz = a.bc_dtype == SSM_F32 ? 4 : 2;
  const char* Bbase = reinterpret_cast<const char*>(a.Bm) + boff * bcsz;
  const char* Cbase = reinterpret_cast<const char*>(a.Cm) + coff * bcsz;
  const bool io_vec = fl.io_vec != 0, bc_vec = fl.bc_vec != 0;
  const int raw_bc_dtype = bc_vec ? a.bc_dtype : SSM_F32;

  const int ntiles = (L + TL - 1) / TL;
  const int nck = (L + kScanCkpt - 1) / kScanCkpt;

  auto fill_raw = [&](int t0) {
    fill_rows_raw<T, RPW, TL>(rawU, gu, b, D, L, drow0, t0, io_vec, lane, a.row_sb, a.row_sd);
    fill_rows_raw<T, RPW, TL>(rawD, gdl, b, D, L, drow0, t0, io_vec, lane, a.row_sb, a.row_sd);
    if (gz) fill_rows_raw<T, RPW, TL>(rawZ, gz, b, D, L, drow0, t0, io_vec, lane, a.row_sb, a.row_sd);
    if (SHARED) {
      fill_bc_raw<TL>(rawB, Bbase, a.bc_dtype, a.b_sn, a.b_st, N, t0, L, bc_vec, tid, NT);
      fill_bc_raw<TL>(rawC, Cbase, a.bc_dtype, a.c_sn, a.c_st, N, t0, L, bc_vec, tid, NT);
    }
    cp_async_commit();
  };

  if (ntiles > 0) fill_raw(0);

  for (int k = 0; k < ntiles; ++k) {
    const int t0 = k * TL;
    cp_async_wait_all();
    __syncthreads();  // raw tile k complete for every thread; previous tile's working arrays free

    // ---- raw -> fp32 working arrays: dl, dl*u, D*u, silu(z) --------------------------------
    {
      constexpr int CH = TL / V;
      for (int c = lane; c < RPW * CH; c += 32) {
        const int rr = c / CH, ch = c % CH;
        const int dd = min(drow0 + rr, D - 1);
        const int t = t0 + ch * V;
        float fu[V], fd[V], fz[V], fy[V];
        Vec16<T> v;
        v.raw = *reinterpret_cast<const uint4*>(rawU + rr * TL + ch * V);
        v.unpack(fu);
        v.raw = *reinterpret_cast<const uint4*>(rawD + rr * TL + ch * V);
        v.unpack(fd);
        if (gz) {
          v.raw = *reinterpret_cast<const uint4*>(rawZ + rr * TL + ch * V);
          v.unpack(fz);
        }
        const float bias = a.dt_bias ? __ldg(a.dt_bias + dd) : 0.f;
        const float Dv = a.D ? __ldg(a.D + dd) : 0.f;
#pragma unroll
        for (int i = 0; i < V; ++i) {
          float x = fd[i] + bias;
          if (a.delta_softplus) x = softplus_fast(x);
          if (t + i >= L) x = 0.f;  // steps beyond the sequence leave the state untouched
          fd[i] = x;
          fy[i] = Dv * fu[i];
          fu[i] = x * fu[i];
          fz[i] = gz ? silu_fast(fz[i]) : 1.f;
        }
        const int o = rr * TLP + ch * V;
#pragma unroll
        for (int i = 0; i < V; i += 4) {
          *reinterpret_cast<float4*>(sDl + o + i) = make_float4(fd[i], fd[i + 1], fd[i + 2], fd[i + 3]);
          *reinterpret_cast<float4*>(sDu + o + i) = make_float4(fu[i], fu[i + 1], fu[i + 2], fu[i + 3]);
          *reinterpret_cast<float4*>(sY + o + i) = make_float4(fy[i], fy[i + 1], fy[i + 2], fy[i + 3]);
          *reinterpret_cast<float4*>(sG + o + i) = make_float4(fz[i], fz[i + 1], fz[i + 2], fz[i + 3]);
        }
      }
    }
    if (SHARED) {
      convert_bc<TL, NP>(sB, rawB, raw_bc_dtype, N, tid, NT);
      convert_bc<TL, NP>(sC, rawC, raw_bc_dtype, N, tid, NT);
    }
    __syncthreads();  // working arrays ready; raw buffers free
    if (k + 1 < ntiles) fill_raw(t0 + TL);  // overlaps the recurrence below

    // ---- recurrence over the tile ----------------------------------------------------------
    const float* rDl = sDl + r * TLP;
    const float* rDu = sDu + r * TLP;
    float* rY = sY + r * TLP;
#pragma unroll UNROLL
    for (int tb0 = 0; tb0 < TL; tb0 += TB) {
      if (a.checkpoints && ((t0 + tb0) % kScanCkpt) == 0 && (t0 + tb0) < L && row_ok) {
        float* ck = a.checkpoints + (row * nck + (t0 + tb0) / kScanCkpt) * N;
#pragma unroll
        for (int j = 0; j < NS; j += 2) {
          if (sg * NS + j < N) ck[sg * NS + j] = h[j / 2].x;
          if (sg * NS + j + 1 < N) ck[sg * NS + j + 1] = h[j / 2].y;
        }
      }
      float p[TB];
#pragma unroll
      for (int q = 0; q < TB; q += 4) {
        const int tt = tb0 + q;
        const float4 dl4 = *reinterpret_cast<const float4*>(rDl + tt);
        const float4 du4 = *reinterpret_cast<const float4*>(rDu + tt);
        const float dl[4] = {dl4.x, dl4.y, dl4.z, dl4.w};
        const float du[4] = {du4.x, du4.y, du4.z, du4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float bv[NS], cv[NS];
          if (SHARED) {
            load_states<NS, NP>(sB, tt + i, sg, bv);
            load_states<NS, NP>(sC, tt + i, sg, cv);
          } else {
            const int t = t0 + tt + i;
#pragma unroll
            for (int j = 0; j < NS; ++j) {
              const int n = sg * NS + j;
              const bool ok = n < N && t < L;
              bv[j] = ok ? load_dyn(Bbase, (int64_t)n * a.b_sn + (int64_t)t * a.b_st, a.bc_dtype) : 0.f;
              cv[j] = ok ? load_dyn(Cbase, (int64_t)n * a.c_sn + (int64_t)t * a.c_st, a.bc_dtype) : 0.f;
            }
          }
          const float2 dl2 = make_float2(dl[i], dl[i]);
          const float2 du2 = make_float2(du[i], du[i]);
          float2 acc = make_float2(0.f, 0.f);
#pragma unroll
          for (int j = 0; j < NS; j += 2) {
            const float2 e = __fmul2_rn(dl2, A2[j / 2]);
            const float2 da = make_float2(ex2_approx(e.x), ex2_approx(e.y));
            h[j / 2] = __ffma2_rn(da, h[j / 2], __fmul2_rn(du2, make_float2(bv[j], bv[j + 1])));
            acc = __ffma2_rn(make_float2(cv[j], cv[j + 1]), h[j / 2], acc);
          }
          p[q + i] = acc.x + acc.y;
        }
      }
      reduce_scatter<LPR, 1, TB>(p, lane);
      constexpr int PER = TB / LPR;
#pragma unroll
      for (int i = 0; i < PER; ++i) rY[tb0 + sg * PER + i] += p[i];
    }
    __syncwarp();

    // ---- epilogue: gate, convert, store ------------------------------------------------------
    if (io_vec) {
      constexpr int CH = TL / V;
      for (int c = lane; c < RPW * CH; c += 32) {
        const int rr = c / CH, ch = c % CH;
        const int dd = drow0 + rr;
        const int t = t0 + ch * V;
        if (dd < D && t < L) {
          const int o = rr * TLP + ch * V;
          float f[V];
#pragma unroll
          for (int i = 0; i < V; i += 4) {
            const float4 y4 = *reinterpret_cast<const float4*>(sY + o + i);
            const float4 g4 = *reinterpret_cast<const float4*>(sG + o + i);
            f[i] = y4.x * g4.x, f[i + 1] = y4.y * g4.y, f[i + 2] = y4.z * g4.z, f[i + 3] = y4.w * g4.w;
          }
          Vec16<T> v;
          v.pack(f);
          v.store_stream(gout + (int64_t)b * a.row_sb + (int64_t)dd * a.row_sd + t);
        }
      }
    } else {
      for (int i = lane; i < RPW * TL; i += 32) {
        const int rr = i / TL, tt = i % TL;
        const int dd = drow0 + rr;
        const int t = t0 + tt;
        if (dd < D && t < L) gout[(int64_t)b * a.row_sb + (int64_t)dd * a.row_sd + t] = from_f<T>(sY[rr * TLP + tt] * sG[rr * TLP + tt]);
      }
    }
  }

  if (a.last_state && row_ok) {
#pragma unroll
    for (int j = 0; j < NS; j += 2) {
      const int n = sg * NS + j;
      if (n < N) store_dyn(a.last_state, row * N + n, a.last_dtype, h[j / 2].x);
      if (n + 1 < N) store_dyn(a.last_state, row * N + n + 1, a.last_dtype, h[j / 2].y);
    }
  }
}

template <typename T, int NS, int LPR, int UNROLL = 2>
static int launch_fwd(const ssm_scan_fwd_args& a, ScanFlags fl, cudaStream_t st) {
  using S = ScanShape<NS, LPR>;
  fl.shared_bc = (fl.rows_per_group % S::ROWS == 0);
  dim3 grid((a.dim + S::ROWS - 1) / S::ROWS, a.batch);
  if (fl.shared_bc) {
    const size_t smem = FwdSmem<T, NS, LPR, true>::bytes();
    auto kern = scan_fwd_kernel<T, NS, LPR, true, UNROLL>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<grid, kScanWarps * 32, smem, st>>>(a, fl);
  } else {
    const size_t smem = FwdSmem<T, NS, LPR, false>::bytes();
    auto kern = scan_fwd_kernel<T, NS, LPR, false, UNROLL>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<grid, kScanWarps * 32, smem, st>>>(a, fl);
  }
  return launch_status("scan_fwd_kernel");
}

// nstate -> lanes per row (states per lane is 4, or 8 above 128 states)
static int fwd_lpr(int n) { return n <= 4 ? 1 : n <= 8 ? 2 : n <= 16 ? 4 : n <= 32 ? 8 : n <= 64 ? 16 : 32; }

template <typename T>
int dispatch_fwd(const ssm_scan_fwd_args& a, const ScanFlags& fl, cudaStream_t st) {
  const int n = a.nstate;
  if (fwd_tiles_ok(a, fl)) return dispatch_fwd_tiles<T>(a, fl, st);  // selective_scan_fwd_tiles.cuh; the general kernel below otherwise
  switch (fwd_lpr(n)) {
    case 1: return launch_fwd<T, 4, 1>(a, fl, st);
    case 2: return launch_fwd<T, 4, 2>(a, fl, st);
    case 4: return launch_fwd<T, 4, 4>(a, fl, st);
    case 8: return launch_fwd<T, 4, 8>(a, fl, st);
    case 16: return launch_fwd<T, 4, 16>(a, fl, st);
    default: return n <= 128 ? launch_fwd<T, 4, 32>(a, fl, st) : launch_fwd<T, 8, 32>(a, fl, st);
  }
}

int scan_validate(const ssm_scan_fwd_args* a, ScanFlags* fl, int rows_per_cta_hint);

}  // namespace ssmb

