// Mamba-1 selective scan, forward, for sm_100a.
//
// Work decomposition (see scan_common.cuh): lanes = rows x state groups, time sequential.
// Per (row, state, step) the kernel spends one ex2.approx, the state FMA and the output
// FMA; the <C, h> contraction over states is a register reduce-scatter across the LPR
// lanes of the row, amortised over TB steps.  B and C tiles are read from global memory
// once per CTA (ROWS channel rows share them), u/delta/z once, out written once.
#include "scan_common.cuh"

namespace ssmb {

template <typename T, int NS, int LPR, bool SHARED>
__global__ void __launch_bounds__(kScanWarps * 32) scan_fwd_kernel(const ssm_scan_fwd_args a, const ScanFlags fl) {
  using S = ScanShape<NS, LPR>;
  constexpr int NP = S::NP, RPW = S::RPW, ROWS = S::ROWS, TB = S::TB;
  constexpr int TL = NP <= 32 ? 64 : 32;
  constexpr int TLP = TL + 4;
  constexpr int V = 16 / sizeof(T);
  static_assert(TL % TB == 0 && TL % kScanCkpt == 0, "tile must hold whole batches and checkpoints");

  extern __shared__ __align__(16) float smem[];
  float* sB = smem;                                  // [NP][TLP] (SHARED only)
  float* sC = sB + (SHARED ? NP * TLP : 0);          // [NP][TLP]
  float* warp_base = sC + (SHARED ? NP * TLP : 0);   // per warp: 4 x [RPW][TLP]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* sDl = warp_base + warp * (4 * RPW * TLP);
  float* sDu = sDl + RPW * TLP;
  float* sY = sDu + RPW * TLP;
  float* sG = sY + RPW * TLP;

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
  T* __restrict__ gout = reinterpret_cast<T*>(a.out);

  // per-lane state
  float A2[NS], h[NS];
#pragma unroll
  for (int j = 0; j < NS; ++j) {
    const int n = sg * NS + j;
    A2[j] = n < N ? __ldg(a.A + (int64_t)d * N + n) * kLog2e : 0.f;
    h[j] = (n < N && a.initial_state) ? __ldg(a.initial_state + row * N + n) : 0.f;
  }

  if (SHARED) {  // padded state rows stay zero for the whole kernel
    for (int i = tid; i < 2 * NP * TLP; i += kScanWarps * 32) sB[i] = 0.f;
  }

  // B/C bases
  const int64_t boff = bc_row_offset(b, SHARED ? min(d0, D - 1) : d, fl.rows_per_group, a.b_sb, a.b_sg);
  const int64_t coff = bc_row_offset(b, SHARED ? min(d0, D - 1) : d, fl.rows_per_group, a.c_sb, a.c_sg);
  const int bcsz = a.bc_dtype == SSM_F32 ? 4 : 2;
  const char* Bbase = reinterpret_cast<const char*>(a.Bm) + boff * bcsz;
  const char* Cbase = reinterpret_cast<const char*>(a.Cm) + coff * bcsz;

  const int ntiles = (L + TL - 1) / TL;
  const int nck = (L + kScanCkpt - 1) / kScanCkpt;

  for (int k = 0; k < ntiles; ++k) {
    const int t0 = k * TL;
    if (SHARED) {
      __syncthreads();  // previous tile's B/C fully consumed
      stage_bc<TL, TLP>(sB, Bbase, a.bc_dtype, a.b_sn, a.b_st, N, t0, L, fl.bc_vec != 0, tid, kScanWarps * 32);
      stage_bc<TL, TLP>(sC, Cbase, a.bc_dtype, a.c_sn, a.c_st, N, t0, L, fl.bc_vec != 0, tid, kScanWarps * 32);
    } else {
      __syncwarp();
    }
    // ---- stage this warp's rows: dl, dl*u, D*u, silu(z) ------------------------------
    if (fl.io_vec) {
      constexpr int CH = TL / V;
      for (int c = lane; c < RPW * CH; c += 32) {
        const int rr = c / CH, ch = c % CH;
        const int dd = min(d0 + warp * RPW + rr, D - 1);
        const int64_t base = ((int64_t)b * D + dd) * L;
        const int t = t0 + ch * V;
        float fu[V], fd[V], fz[V], fy[V];
        if (t < L) {
          Vec16<T> v;
          v.load_stream(gu + base + t);
          v.unpack(fu);
          v.load_stream(gdl + base + t);
          v.unpack(fd);
          if (gz) {
            v.load_stream(gz + base + t);
            v.unpack(fz);
          }
          const float bias = a.dt_bias ? __ldg(a.dt_bias + dd) : 0.f;
          const float Dv = a.D ? __ldg(a.D + dd) : 0.f;
#pragma unroll
          for (int i = 0; i < V; ++i) {
            float x = fd[i] + bias;
            if (a.delta_softplus) x = softplus_f(x);
            fd[i] = x;
            fy[i] = Dv * fu[i];
            fu[i] = x * fu[i];
            fz[i] = gz ? silu_f(fz[i]) : 1.f;
          }
        } else {
#pragma unroll
          for (int i = 0; i < V; ++i) fu[i] = fd[i] = fy[i] = 0.f, fz[i] = 1.f;
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
    } else {
      for (int i = lane; i < RPW * TL; i += 32) {
        const int rr = i / TL, tt = i % TL;
        const int dd = min(d0 + warp * RPW + rr, D - 1);
        const int64_t base = ((int64_t)b * D + dd) * L;
        const int t = t0 + tt;
        float dl = 0.f, du = 0.f, y0 = 0.f, g = 1.f;
        if (t < L) {
          const float uu = to_f<T>(gu[base + t]);
          float x = to_f<T>(gdl[base + t]) + (a.dt_bias ? __ldg(a.dt_bias + dd) : 0.f);
          if (a.delta_softplus) x = softplus_f(x);
          dl = x;
          du = x * uu;
          y0 = a.D ? __ldg(a.D + dd) * uu : 0.f;
          g = gz ? silu_f(to_f<T>(gz[base + t])) : 1.f;
        }
        const int o = rr * TLP + tt;
        sDl[o] = dl, sDu[o] = du, sY[o] = y0, sG[o] = g;
      }
    }
    if (SHARED) __syncthreads();
    else __syncwarp();

    // ---- recurrence over the tile ----------------------------------------------------
    const float* rDl = sDl + r * TLP;
    const float* rDu = sDu + r * TLP;
    float* rY = sY + r * TLP;
#pragma unroll 1
    for (int tb0 = 0; tb0 < TL; tb0 += TB) {
      if (a.checkpoints && ((t0 + tb0) % kScanCkpt) == 0 && (t0 + tb0) < L && row_ok) {
        float* ck = a.checkpoints + (row * nck + (t0 + tb0) / kScanCkpt) * N;
#pragma unroll
        for (int j = 0; j < NS; ++j)
          if (sg * NS + j < N) ck[sg * NS + j] = h[j];
      }
      float p[TB];
#pragma unroll
      for (int i = 0; i < TB; ++i) p[i] = 0.f;
#pragma unroll
      for (int q = 0; q < TB; q += 4) {
        const int tt = tb0 + q;
        const float4 dl4 = *reinterpret_cast<const float4*>(rDl + tt);
        const float4 du4 = *reinterpret_cast<const float4*>(rDu + tt);
        const float dl[4] = {dl4.x, dl4.y, dl4.z, dl4.w};
        const float du[4] = {du4.x, du4.y, du4.z, du4.w};
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
            p[q + i] = fmaf(cv[i], h[j], p[q + i]);
          }
        }
      }
      reduce_scatter<LPR, 1, TB>(p, lane);
      constexpr int PER = TB / LPR;
#pragma unroll
      for (int i = 0; i < PER; ++i) rY[tb0 + sg * PER + i] += p[i];
    }
    __syncwarp();

    // ---- epilogue: gate, convert, store ------------------------------------------------
    if (fl.io_vec) {
      constexpr int CH = TL / V;
      for (int c = lane; c < RPW * CH; c += 32) {
        const int rr = c / CH, ch = c % CH;
        const int dd = d0 + warp * RPW + rr;
        const int t = t0 + ch * V;
        if (dd < D && t < L) {
          const int o = rr * TLP + ch * V;
          float f[V];
#pragma unroll
          for (int i = 0; i < V; ++i) f[i] = sY[o + i] * sG[o + i];
          Vec16<T> v;
          v.pack(f);
          v.store_stream(gout + ((int64_t)b * D + dd) * L + t);
        }
      }
    } else {
      for (int i = lane; i < RPW * TL; i += 32) {
        const int rr = i / TL, tt = i % TL;
        const int dd = d0 + warp * RPW + rr;
        const int t = t0 + tt;
        if (dd < D && t < L) gout[((int64_t)b * D + dd) * L + t] = from_f<T>(sY[rr * TLP + tt] * sG[rr * TLP + tt]);
      }
    }
  }

  if (a.last_state && row_ok) {
#pragma unroll
    for (int j = 0; j < NS; ++j) {
      const int n = sg * NS + j;
      if (n < N) store_dyn(a.last_state, row * N + n, a.last_dtype, h[j]);
    }
  }
}

template <typename T, int NS, int LPR>
static int launch_fwd(const ssm_scan_fwd_args& a, const ScanFlags& fl, cudaStream_t st) {
  using S = ScanShape<NS, LPR>;
  constexpr int TL = S::NP <= 32 ? 64 : 32;
  constexpr int TLP = TL + 4;
  dim3 grid((a.dim + S::ROWS - 1) / S::ROWS, a.batch);
  const size_t per_warp = 4 * S::RPW * TLP * sizeof(float);
  if (fl.shared_bc) {
    const size_t smem = 2 * S::NP * TLP * sizeof(float) + kScanWarps * per_warp;
    auto kern = scan_fwd_kernel<T, NS, LPR, true>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<grid, kScanWarps * 32, smem, st>>>(a, fl);
  } else {
    const size_t smem = kScanWarps * per_warp;
    auto kern = scan_fwd_kernel<T, NS, LPR, false>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<grid, kScanWarps * 32, smem, st>>>(a, fl);
  }
  return launch_status("scan_fwd_kernel");
}

template <typename T>
static int dispatch_fwd(const ssm_scan_fwd_args& a, const ScanFlags& fl, cudaStream_t st) {
  const int n = a.nstate;
  if (n <= 4) return launch_fwd<T, 4, 1>(a, fl, st);
  if (n <= 8) return launch_fwd<T, 4, 2>(a, fl, st);
  if (n <= 16) return launch_fwd<T, 4, 4>(a, fl, st);
  if (n <= 32) return launch_fwd<T, 4, 8>(a, fl, st);
  if (n <= 64) return launch_fwd<T, 4, 16>(a, fl, st);
  if (n <= 128) return launch_fwd<T, 4, 32>(a, fl, st);
  return launch_fwd<T, 8, 32>(a, fl, st);
}

int scan_validate(const ssm_scan_fwd_args* a, ScanFlags* fl, int rows_per_cta_hint);

}  // namespace ssmb

using namespace ssmb;

// Argument checks shared with the backward entry point.
int ssmb::scan_validate(const ssm_scan_fwd_args* a, ScanFlags* fl, int rows_per_cta) {
  SSM_REQUIRE(a != nullptr, SSM_ERR_NULL, "selective_scan: args is NULL");
  SSM_REQUIRE(a->batch >= 0 && a->dim >= 0 && a->len >= 0, SSM_ERR_SHAPE, "selective_scan: negative size");
  SSM_REQUIRE(a->nstate >= 1 && a->nstate <= 256, SSM_ERR_UNSUPPORTED, "selective_scan: nstate must be in [1, 256]");
  SSM_REQUIRE(valid_dtype(a->io_dtype) && valid_dtype(a->bc_dtype), SSM_ERR_DTYPE, "selective_scan: unknown dtype");
  SSM_REQUIRE(a->batch <= 65535, SSM_ERR_TOO_LARGE, "selective_scan: batch exceeds 65535");
  if (a->batch == 0 || a->dim == 0) return SSM_OK;
  SSM_REQUIRE(a->A && a->Bm && a->Cm, SSM_ERR_NULL, "selective_scan: A, B and C are required");
  SSM_REQUIRE(a->len == 0 || (a->u && a->delta), SSM_ERR_NULL, "selective_scan: u and delta are required");
  SSM_REQUIRE(a->bc_groups >= 1 && a->dim % a->bc_groups == 0, SSM_ERR_SHAPE, "Group dimension must divide D.");
  const int esz = dtype_size(a->io_dtype);
  const int v = 16 / esz;
  fl->io_vec = (a->len % v == 0) && aligned_to(a->u, 16) && aligned_to(a->delta, 16) && (!a->z || aligned_to(a->z, 16)) &&
               (!a->out || aligned_to(a->out, 16));
  const int bv = 16 / dtype_size(a->bc_dtype);
  auto ok = [&](const void* p, int64_t sb, int64_t sg, int64_t sn, int64_t st) {
    return st == 1 && aligned_to(p, 16) && sb % bv == 0 && sg % bv == 0 && sn % bv == 0;
  };
  fl->bc_vec = ok(a->Bm, a->b_sb, a->b_sg, a->b_sn, a->b_st) && ok(a->Cm, a->c_sb, a->c_sg, a->c_sn, a->c_st) && (a->len % bv == 0);
  fl->rows_per_group = a->dim / a->bc_groups;
  fl->shared_bc = (fl->rows_per_group % rows_per_cta == 0);
  return SSM_OK;
}

static int rows_per_cta_for(int n) {
  const int lpr = n <= 4 ? 1 : n <= 8 ? 2 : n <= 16 ? 4 : n <= 32 ? 8 : n <= 64 ? 16 : 32;
  return kScanWarps * (32 / lpr);
}

extern "C" int ssm_scan_checkpoint_interval(void) { return kScanCkpt; }

extern "C" int ssm_selective_scan_fwd(const ssm_scan_fwd_args* a, ssm_stream_t stream) {
  ScanFlags fl{};
  if (int rc = scan_validate(a, &fl, a ? rows_per_cta_for(a->nstate) : 1)) return rc;
  SSM_REQUIRE(valid_dtype(a->last_dtype) || !a->last_state, SSM_ERR_DTYPE, "selective_scan: unknown last_state dtype");
  if (a->batch == 0 || a->dim == 0) return SSM_OK;
  SSM_REQUIRE(a->len == 0 || a->out, SSM_ERR_NULL, "selective_scan: out is required");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (a->io_dtype) {
    case SSM_F32: return dispatch_fwd<float>(*a, fl, st);
    case SSM_BF16: return dispatch_fwd<__nv_bfloat16>(*a, fl, st);
    default: return dispatch_fwd<__half>(*a, fl, st);
  }
}
