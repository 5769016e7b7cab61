// Mamba-1 selective scan, backward, for sm_100a.
//
// Same lane layout as the forward kernel (scan_common.cuh).  Time is walked in reverse in
// tiles of one checkpoint interval: the tile's states are rebuilt from the checkpoint the
// forward pass stored (kept in shared memory, one float4 per lane and step), then the
// adjoint recurrence  G_t = C_t dy_t + a_{t+1} G_{t+1}  runs backwards with G carried in
// registers across tiles; grad_last_state seeds it.  Contractions over states (du, ddelta,
// y for dz) are register reduce-scatters across the lanes of a row; contractions over the
// rows that share a B / C group (dB, dC) are reduce-scatters across the rows of a warp,
// then shared-memory accumulation across the CTA's warps and one global atomic per CTA,
// state and step.
#include "scan_common.cuh"

namespace ssmb {

template <int NS, int LPR>
struct BwdShape : ScanShape<NS, LPR> {
  using S = ScanShape<NS, LPR>;
  static constexpr int NW = S::NP > 128 ? 2 : kScanWarps;  // warps per CTA
  static constexpr int ROWS = NW * S::RPW;
  static constexpr int TL = kScanCkpt;
  static constexpr int TLP = TL + 4;
  static constexpr int CNT4 = NS * 4 > S::RPW ? NS * 4 : S::RPW;  // entries per 4-step row reduction
  static constexpr int WARP_ROWS_F = 6 * S::RPW * TLP;            // 6 row arrays
  static constexpr int WARP_HIST_F = (TL + 1) * 32 * NS;
  static constexpr int WARP_F = WARP_ROWS_F + WARP_HIST_F + 2 * 32;  // + per-row dD / dbias sums
  static constexpr size_t smem_bytes(bool shared) { return sizeof(float) * ((shared ? 4 * S::NP * TLP : 0) + NW * WARP_F); }
};

template <typename T, int NS, int LPR, bool SHARED>
__global__ void __launch_bounds__(BwdShape<NS, LPR>::NW * 32) scan_bwd_kernel(const ssm_scan_bwd_args g, const ScanFlags fl) {
  using S = BwdShape<NS, LPR>;
  constexpr int NP = S::NP, RPW = S::RPW, ROWS = S::ROWS, TB = S::TB, TL = S::TL, TLP = S::TLP, NW = S::NW, CNT4 = S::CNT4;
  constexpr int V = 16 / sizeof(T);
  constexpr int NT = NW * 32;
  const ssm_scan_fwd_args& a = g.fwd;

  extern __shared__ __align__(16) float smem[];
  float* sB = smem;
  float* sC = sB + (SHARED ? NP * TLP : 0);
  float* sdB = sC + (SHARED ? NP * TLP : 0);
  float* sdC = sdB + (SHARED ? NP * TLP : 0);
  float* wbase = sdC + (SHARED ? NP * TLP : 0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* sDl = wbase + warp * S::WARP_F;  // delta after bias / softplus
  float* sU = sDl + RPW * TLP;            // u
  float* sDy = sU + RPW * TLP;            // dout * silu(z)
  float* sZf = sDy + RPW * TLP;           // dout * silu'(z), finished into dz once y is rebuilt
  float* sDu = sZf + RPW * TLP;           // out: sum_n G*B, finished into du
  float* sDd = sDu + RPW * TLP;           // out: ddelta (before the softplus factor)
  float* hist = sDd + RPW * TLP;          // [(TL+1)][32][NS]
  float* sRowD = hist + S::WARP_HIST_F;   // [32] per-row dD partial
  float* sRowB = sRowD + 32;              // [32] per-row ddt_bias partial

  const int b = blockIdx.y;
  const int d0 = blockIdx.x * ROWS;
  const int N = a.nstate, L = a.len, D = a.dim;
  const int r = lane / LPR, sg = lane % LPR;
  const int d_raw = d0 + warp * RPW + r;
  const bool row_ok = d_raw < D;
  const int d = row_ok ? d_raw : D - 1;
  const int64_t row = (int64_t)b * D + d;

  const T* __restrict__ gu = reinterpret_cast<const T*>(a.u);
  const T* __restrict__ gdl = reinterpret_cast<const T*>(a.delta);
  const T* __restrict__ gz = reinterpret_cast<const T*>(a.z);
  const T* __restrict__ gdo = reinterpret_cast<const T*>(g.dout);
  T* __restrict__ gdu = reinterpret_cast<T*>(g.du);
  T* __restrict__ gdd = reinterpret_cast<T*>(g.ddelta);
  T* __restrict__ gdz = reinterpret_cast<T*>(g.dz);

  float A2[NS], carry[NS], dAacc[NS];
#pragma unroll
  for (int j = 0; j < NS; ++j) {
    const int n = sg * NS + j;
    A2[j] = n < N ? __ldg(a.A + (int64_t)d * N + n) * kLog2e : 0.f;
    carry[j] = (n < N && g.dlast_state) ? __ldg(g.dlast_state + row * N + n) : 0.f;
    dAacc[j] = 0.f;
  }
  if (lane < 32) sRowD[lane] = 0.f, sRowB[lane] = 0.f;
  if (SHARED) {
    for (int i = tid; i < 4 * NP * TLP; i += NT) sB[i] = 0.f;
  }

  const int rpg = fl.rows_per_group;
  const int dref = SHARED ? min(d0, D - 1) : d;
  const int64_t boff = bc_row_offset(b, dref, rpg, a.b_sb, a.b_sg);
  const int64_t coff = bc_row_offset(b, dref, rpg, a.c_sb, a.c_sg);
  const int64_t dboff = bc_row_offset(b, dref, rpg, g.db_sb, g.db_sg);
  const int64_t dcoff = bc_row_offset(b, dref, rpg, g.dc_sb, g.dc_sg);
  const int bcsz = a.bc_dtype == SSM_F32 ? 4 : 2;
  const char* Bbase = reinterpret_cast<const char*>(a.Bm) + boff * bcsz;
  const char* Cbase = reinterpret_cast<const char*>(a.Cm) + coff * bcsz;

  const int ntiles = (L + TL - 1) / TL;

  for (int k = ntiles - 1; k >= 0; --k) {
    const int t0 = k * TL;
    if (SHARED) {
      __syncthreads();  // previous tile's B / C consumed and dB / dC flushed
      stage_bc<TL, TLP>(sB, Bbase, a.bc_dtype, a.b_sn, a.b_st, N, t0, L, fl.bc_vec != 0, tid, NT);
      stage_bc<TL, TLP>(sC, Cbase, a.bc_dtype, a.c_sn, a.c_st, N, t0, L, fl.bc_vec != 0, tid, NT);
      for (int i = tid; i < 2 * NP * TLP; i += NT) sdB[i] = 0.f;
    } else {
      __syncwarp();
    }
    // ---- stage this warp's rows -------------------------------------------------------
    if (fl.io_vec) {
      constexpr int CH = TL / V;
      for (int c = lane; c < RPW * CH; c += 32) {
        const int rr = c / CH, ch = c % CH;
        const int dd = min(d0 + warp * RPW + rr, D - 1);
        const int64_t base = ((int64_t)b * D + dd) * L;
        const int t = t0 + ch * V;
        float fu[V], fd[V], fz[V], fo[V], fdy[V], fzf[V];
        if (t < L) {
          Vec16<T> v;
          v.load_stream(gu + base + t);
          v.unpack(fu);
          v.load_stream(gdl + base + t);
          v.unpack(fd);
          v.load_stream(gdo + base + t);
          v.unpack(fo);
          if (gz) {
            v.load_stream(gz + base + t);
            v.unpack(fz);
          }
          const float bias = a.dt_bias ? __ldg(a.dt_bias + dd) : 0.f;
#pragma unroll
          for (int i = 0; i < V; ++i) {
            float x = fd[i] + bias;
            if (a.delta_softplus) x = softplus_f(x);
            fd[i] = x;
            if (gz) {
              const float zv = fz[i];
              const float s = sigmoid_fast(zv);
              fdy[i] = fo[i] * zv * s;
              fzf[i] = fo[i] * s * (1.f + zv * (1.f - s));
            } else {
              fdy[i] = fo[i], fzf[i] = 0.f;
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < V; ++i) fu[i] = fd[i] = fdy[i] = fzf[i] = 0.f;
        }
        const int o = rr * TLP + ch * V;
#pragma unroll
        for (int i = 0; i < V; i += 4) {
          *reinterpret_cast<float4*>(sDl + o + i) = make_float4(fd[i], fd[i + 1], fd[i + 2], fd[i + 3]);
          *reinterpret_cast<float4*>(sU + o + i) = make_float4(fu[i], fu[i + 1], fu[i + 2], fu[i + 3]);
          *reinterpret_cast<float4*>(sDy + o + i) = make_float4(fdy[i], fdy[i + 1], fdy[i + 2], fdy[i + 3]);
          *reinterpret_cast<float4*>(sZf + o + i) = make_float4(fzf[i], fzf[i + 1], fzf[i + 2], fzf[i + 3]);
        }
      }
    } else {
      for (int i = lane; i < RPW * TL; i += 32) {
        const int rr = i / TL, tt = i % TL;
        const int dd = min(d0 + warp * RPW + rr, D - 1);
        const int64_t base = ((int64_t)b * D + dd) * L;
        const int t = t0 + tt;
        float uu = 0.f, dl = 0.f, dy = 0.f, zf = 0.f;
        if (t < L) {
          uu = to_f<T>(gu[base + t]);
          dl = to_f<T>(gdl[base + t]) + (a.dt_bias ? __ldg(a.dt_bias + dd) : 0.f);
          if (a.delta_softplus) dl = softplus_f(dl);
          const float dov = to_f<T>(gdo[base + t]);
          if (gz) {
            const float zv = to_f<T>(gz[base + t]);
            const float s = sigmoid_fast(zv);
            dy = dov * zv * s;
            zf = dov * s * (1.f + zv * (1.f - s));
          } else {
            dy = dov;
          }
        }
        const int o = rr * TLP + tt;
        sDl[o] = dl, sU[o] = uu, sDy[o] = dy, sZf[o] = zf;
      }
    }
    if (SHARED) __syncthreads();
    else __syncwarp();

    const float* rDl = sDl + r * TLP;
    const float* rU = sU + r * TLP;
    const float* rDy = sDy + r * TLP;
    float* rDu = sDu + r * TLP;
    float* rDd = sDd + r * TLP;
    float* rZf = sZf + r * TLP;
    const float Dv = a.D ? __ldg(a.D + d) : 0.f;

    // ---- rebuild the tile's states from the checkpoint -----------------------------------
    {
      float h[NS];
      const int nck = ntiles;  // TL == checkpoint interval
      const float* ck = a.checkpoints + (row * nck + k) * N;
#pragma unroll
      for (int j = 0; j < NS; ++j) {
        const int n = sg * NS + j;
        h[j] = n < N ? __ldg(ck + n) : 0.f;
        hist[(0 * 32 + lane) * NS + j] = h[j];
      }
#pragma unroll 1
      for (int tb0 = 0; tb0 < TL; tb0 += TB) {
        float p[TB];
#pragma unroll
        for (int i = 0; i < TB; ++i) p[i] = 0.f;
#pragma unroll
        for (int q = 0; q < TB; q += 4) {
          const int tt = tb0 + q;
          const float4 dl4 = *reinterpret_cast<const float4*>(rDl + tt);
          const float4 u4 = *reinterpret_cast<const float4*>(rU + tt);
          const float dl[4] = {dl4.x, dl4.y, dl4.z, dl4.w};
          const float du[4] = {dl4.x * u4.x, dl4.y * u4.y, dl4.z * u4.z, dl4.w * u4.w};
#pragma unroll
          for (int j = 0; j < NS; ++j) {
            float bv[4], cv[4];
            if (SHARED) {
              const float4 b4 = *reinterpret_cast<const float4*>(sB + (sg * NS + j) * TLP + tt);
              const float4 c4 = *reinterpret_cast<const float4*>(sC + (sg * NS + j) * TLP + tt);
              bv[0] = b4.x, bv[1] = b4.y, bv[2] = b4.z, bv[3] = b4.w;
              cv[0] = c4.x, cv[1] = c4.y, cv[2] = c4.z, cv[3] = c4.w;
            } else {
              const int n = sg * NS + j;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int t = t0 + tt + i;
                const bool ok = n < N && t < L;
                bv[i] = ok ? load_dyn(Bbase, (int64_t)n * a.b_sn + (int64_t)t * a.b_st, a.bc_dtype) : 0.f;
                cv[i] = ok ? load_dyn(Cbase, (int64_t)n * a.c_sn + (int64_t)t * a.c_st, a.bc_dtype) : 0.f;
              }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float da = ex2_approx(dl[i] * A2[j]);
              h[j] = fmaf(da, h[j], du[i] * bv[i]);
              hist[((tt + i + 1) * 32 + lane) * NS + j] = h[j];
              p[q + i] = fmaf(cv[i], h[j], p[q + i]);
            }
          }
        }
        if (gz) {
          reduce_scatter<LPR, 1, TB>(p, lane);
          constexpr int PER = TB / LPR;
#pragma unroll
          for (int i = 0; i < PER; ++i) {  // dz = dout * silu'(z) * (sum_n C h + D u)
            const int tt = tb0 + sg * PER + i;
            rZf[tt] *= fmaf(Dv, rU[tt], p[i]);
          }
        }
      }
    }
    __syncwarp();

    // ---- adjoint recurrence, last step of the tile first ----------------------------------
#pragma unroll 1
    for (int tb0 = TL - TB; tb0 >= 0; tb0 -= TB) {
      float s1[TB], s2[TB];
#pragma unroll
      for (int i = 0; i < TB; ++i) s1[i] = 0.f, s2[i] = 0.f;
#pragma unroll
      for (int q = TB - 4; q >= 0; q -= 4) {
        const int tt = tb0 + q;
        const float4 dl4 = *reinterpret_cast<const float4*>(rDl + tt);
        const float4 u4 = *reinterpret_cast<const float4*>(rU + tt);
        const float4 dy4 = *reinterpret_cast<const float4*>(rDy + tt);
        const float dl[4] = {dl4.x, dl4.y, dl4.z, dl4.w};
        const float du[4] = {dl4.x * u4.x, dl4.y * u4.y, dl4.z * u4.z, dl4.w * u4.w};
        const float dy[4] = {dy4.x, dy4.y, dy4.z, dy4.w};
        float vB[CNT4], vC[CNT4];
#pragma unroll
        for (int i = 0; i < CNT4; ++i) vB[i] = 0.f, vC[i] = 0.f;
#pragma unroll
        for (int j = 0; j < NS; ++j) {
          float bv[4], cv[4];
          if (SHARED) {
            const float4 b4 = *reinterpret_cast<const float4*>(sB + (sg * NS + j) * TLP + tt);
            const float4 c4 = *reinterpret_cast<const float4*>(sC + (sg * NS + j) * TLP + tt);
            bv[0] = b4.x, bv[1] = b4.y, bv[2] = b4.z, bv[3] = b4.w;
            cv[0] = c4.x, cv[1] = c4.y, cv[2] = c4.z, cv[3] = c4.w;
          } else {
            const int n = sg * NS + j;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int t = t0 + tt + i;
              const bool ok = n < N && t < L;
              bv[i] = ok ? load_dyn(Bbase, (int64_t)n * a.b_sn + (int64_t)t * a.b_st, a.bc_dtype) : 0.f;
              cv[i] = ok ? load_dyn(Cbase, (int64_t)n * a.c_sn + (int64_t)t * a.c_st, a.bc_dtype) : 0.f;
            }
          }
#pragma unroll
          for (int i = 3; i >= 0; --i) {
            const float hc = hist[((tt + i + 1) * 32 + lane) * NS + j];
            const float hp = hist[((tt + i) * 32 + lane) * NS + j];
            const float da = ex2_approx(dl[i] * A2[j]);
            const float G = fmaf(cv[i], dy[i], carry[j]);
            vC[j * 4 + i] = dy[i] * hc;
            vB[j * 4 + i] = G * du[i];
            s1[q + i] = fmaf(G, bv[i], s1[q + i]);
            const float gha = G * hp * da;
            s2[q + i] = fmaf(gha, A2[j], s2[q + i]);
            dAacc[j] = fmaf(gha, dl[i], dAacc[j]);
            carry[j] = da * G;
          }
        }
        if (SHARED) {
          reduce_scatter<RPW, LPR, CNT4>(vB, lane);
          reduce_scatter<RPW, LPR, CNT4>(vC, lane);
          constexpr int PERR = CNT4 / RPW;
#pragma unroll
          for (int i = 0; i < PERR; ++i) {
            const int e = r * PERR + i;
            if (e < NS * 4) {
              const int o = (sg * NS + e / 4) * TLP + tt + (e % 4);
              atomicAdd(sdB + o, vB[i]);
              atomicAdd(sdC + o, vC[i]);
            }
          }
        } else if (row_ok) {
#pragma unroll
          for (int j = 0; j < NS; ++j) {
            const int n = sg * NS + j;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int t = t0 + tt + i;
              if (n < N && t < L) {
                atomicAdd(g.dB + dboff + (int64_t)n * g.db_sn + (int64_t)t * g.db_st, vB[j * 4 + i]);
                atomicAdd(g.dC + dcoff + (int64_t)n * g.dc_sn + (int64_t)t * g.dc_st, vC[j * 4 + i]);
              }
            }
          }
        }
      }
      reduce_scatter<LPR, 1, TB>(s1, lane);
      reduce_scatter<LPR, 1, TB>(s2, lane);
      constexpr int PER = TB / LPR;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int tt = tb0 + sg * PER + i;
        rDu[tt] = fmaf(s1[i], rDl[tt], rDy[tt] * Dv);
        rDd[tt] = fmaf(s1[i], rU[tt], s2[i] * kLn2);
      }
    }
    if (SHARED) __syncthreads();
    else __syncwarp();

    // ---- flush the tile's dB / dC, write du / ddelta / dz ---------------------------------
    if (SHARED) {
      for (int i = tid; i < N * TL; i += NT) {
        const int n = i / TL, tt = i % TL;
        const int t = t0 + tt;
        if (t < L) {
          atomicAdd(g.dB + dboff + (int64_t)n * g.db_sn + (int64_t)t * g.db_st, sdB[n * TLP + tt]);
          atomicAdd(g.dC + dcoff + (int64_t)n * g.dc_sn + (int64_t)t * g.dc_st, sdC[n * TLP + tt]);
        }
      }
    }
    if (fl.io_vec) {
      constexpr int CH = TL / V;
      for (int c = lane; c < RPW * CH; c += 32) {
        const int rr = c / CH, ch = c % CH;
        const int dd = d0 + warp * RPW + rr;
        const int t = t0 + ch * V;
        if (dd < D && t < L) {
          const int o = rr * TLP + ch * V;
          const int64_t base = ((int64_t)b * D + dd) * L + t;
          float f[V], sumD = 0.f, sumB = 0.f;
#pragma unroll
          for (int i = 0; i < V; ++i) f[i] = sDu[o + i], sumD = fmaf(sDy[o + i], sU[o + i], sumD);
          Vec16<T> v;
          v.pack(f);
          v.store_stream(gdu + base);
#pragma unroll
          for (int i = 0; i < V; ++i) {
            // d softplus(pre) / d pre = sigmoid(pre) = 1 - exp(-softplus(pre))
            f[i] = a.delta_softplus ? sDd[o + i] * -expm1f(-sDl[o + i]) : sDd[o + i];
            sumB += f[i];
          }
          v.pack(f);
          v.store_stream(gdd + base);
          if (gdz) {
#pragma unroll
            for (int i = 0; i < V; ++i) f[i] = sZf[o + i];
            v.pack(f);
            v.store_stream(gdz + base);
          }
          atomicAdd(sRowD + rr, sumD);
          atomicAdd(sRowB + rr, sumB);
        }
      }
    } else {
      for (int i = lane; i < RPW * TL; i += 32) {
        const int rr = i / TL, tt = i % TL;
        const int dd = d0 + warp * RPW + rr;
        const int t = t0 + tt;
        if (dd < D && t < L) {
          const int o = rr * TLP + tt;
          const int64_t base = ((int64_t)b * D + dd) * L + t;
          gdu[base] = from_f<T>(sDu[o]);
          const float dd_raw = a.delta_softplus ? sDd[o] * -expm1f(-sDl[o]) : sDd[o];
          gdd[base] = from_f<T>(dd_raw);
          if (gdz) gdz[base] = from_f<T>(sZf[o]);
          atomicAdd(sRowD + rr, sDy[o] * sU[o]);
          atomicAdd(sRowB + rr, dd_raw);
        }
      }
    }
  }

  __syncwarp();
  if (row_ok) {
#pragma unroll
    for (int j = 0; j < NS; ++j) {
      const int n = sg * NS + j;
      if (n < N) atomicAdd(g.dA + (int64_t)d * N + n, dAacc[j]);
    }
    if (sg == 0) {
      if (g.dD) atomicAdd(g.dD + d, sRowD[r]);
      if (g.ddt_bias) atomicAdd(g.ddt_bias + d, sRowB[r]);
    }
  }
}

template <typename T, int NS, int LPR>
static int launch_bwd(const ssm_scan_bwd_args& g, const ScanFlags& fl, cudaStream_t st) {
  using S = BwdShape<NS, LPR>;
  const ssm_scan_fwd_args& a = g.fwd;
  dim3 grid((a.dim + S::ROWS - 1) / S::ROWS, a.batch);
  if (fl.shared_bc) {
    const size_t smem = S::smem_bytes(true);
    auto kern = scan_bwd_kernel<T, NS, LPR, true>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<grid, S::NW * 32, smem, st>>>(g, fl);
  } else {
    const size_t smem = S::smem_bytes(false);
    auto kern = scan_bwd_kernel<T, NS, LPR, false>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<grid, S::NW * 32, smem, st>>>(g, fl);
  }
  return launch_status("scan_bwd_kernel");
}

template <typename T>
static int dispatch_bwd(const ssm_scan_bwd_args& g, ScanFlags& fl, cudaStream_t st) {
  const int n = g.fwd.nstate;
  auto shared = [&](int rows) { fl.shared_bc = (fl.rows_per_group % rows == 0); };
  if (n <= 4) return shared(BwdShape<4, 1>::ROWS), launch_bwd<T, 4, 1>(g, fl, st);
  if (n <= 8) return shared(BwdShape<4, 2>::ROWS), launch_bwd<T, 4, 2>(g, fl, st);
  if (n <= 16) return shared(BwdShape<4, 4>::ROWS), launch_bwd<T, 4, 4>(g, fl, st);
  if (n <= 32) return shared(BwdShape<4, 8>::ROWS), launch_bwd<T, 4, 8>(g, fl, st);
  if (n <= 64) return shared(BwdShape<4, 16>::ROWS), launch_bwd<T, 4, 16>(g, fl, st);
  if (n <= 128) return shared(BwdShape<4, 32>::ROWS), launch_bwd<T, 4, 32>(g, fl, st);
  return shared(BwdShape<8, 32>::ROWS), launch_bwd<T, 8, 32>(g, fl, st);
}

int scan_validate(const ssm_scan_fwd_args* a, ScanFlags* fl, int rows_per_cta);

}  // namespace ssmb

using namespace ssmb;

extern "C" int ssm_selective_scan_bwd(const ssm_scan_bwd_args* g, ssm_stream_t stream) {
  SSM_REQUIRE(g != nullptr, SSM_ERR_NULL, "selective_scan_backward: args is NULL");
  const ssm_scan_fwd_args* a = &g->fwd;
  ScanFlags fl{};
  if (int rc = scan_validate(a, &fl, 1)) return rc;
  if (a->batch == 0 || a->dim == 0 || a->len == 0) return SSM_OK;
  SSM_REQUIRE(a->checkpoints, SSM_ERR_NULL, "selective_scan_backward: forward checkpoints are required");
  SSM_REQUIRE(g->dout && g->du && g->ddelta && g->dA && g->dB && g->dC, SSM_ERR_NULL, "selective_scan_backward: missing pointer");
  SSM_REQUIRE(!a->z == !g->dz, SSM_ERR_NULL, "selective_scan_backward: dz must be given exactly when z is");
  const int v = 16 / dtype_size(a->io_dtype);
  fl.io_vec = fl.io_vec && aligned_to(g->dout, 16) && aligned_to(g->du, 16) && aligned_to(g->ddelta, 16) && (!g->dz || aligned_to(g->dz, 16)) &&
              (a->len % v == 0);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (a->io_dtype) {
    case SSM_F32: return dispatch_bwd<float>(*g, fl, st);
    case SSM_BF16: return dispatch_bwd<__nv_bfloat16>(*g, fl, st);
    default: return dispatch_bwd<__half>(*g, fl, st);
  }
}
