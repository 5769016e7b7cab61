// Mamba-1 selective scan, backward, for sm_100a.
//
// Same lane layout and tile staging as the forward kernel (scan_common.cuh).  Time is walked
// in reverse in tiles of one checkpoint interval: the tile's states are rebuilt from the
// checkpoint the forward pass stored (kept in shared memory, one 16-byte group per lane and
// step), then the adjoint recurrence  G_t = C_t dy_t + a_{t+1} G_{t+1}  runs backwards with G
// carried in registers across tiles; grad_last_state seeds it.  Contractions over states
// (du, ddelta, y for dz) are register reduce-scatters across the lanes of a row;
// contractions over the rows that share a B / C group (dB, dC) are reduce-scatters across
// the rows of a warp, done through a per-warp shared-memory staging area: every lane writes
// its (state, 4 steps) products as 16-byte groups, then each lane sums one (state, 4 steps)
// group over the warp's rows and adds it to global memory with one vector reduction.
#pragma once

#include "scan_common.cuh"

namespace ssmb {

template <typename T, int NS, int LPR, bool SHARED>
struct BwdShape : ScanShape<NS, LPR> {
  using S = ScanShape<NS, LPR>;
  static constexpr int NW = (S::NP > 128 || S::RPW > 16) ? 2 : kScanWarps;  // warps per CTA
  static constexpr int ROWS = NW * S::RPW;
  static constexpr int TL = kScanCkpt;
  static constexpr int TLP = TL + 4;
  // floats
  static constexpr int BC_WORK = SHARED ? 2 * TL * S::NP : 0;  // B, C as [TL][NP]
  static constexpr int WARP_ROWS = 4 * S::RPW * TLP;
  static constexpr int WARP_HIST = (TL / 4 + 1) * 32 * NS;  // states after every fourth step (+ the checkpoint)
  static constexpr int WARP_STAGE = SHARED ? 2 * S::NP * S::RPW * 4 : 0;  // dB / dC products of 4 steps: [2 * NP][RPW][4]
  static constexpr int WARP_WORK = WARP_ROWS + WARP_HIST + WARP_STAGE;
  // bytes
  static constexpr int BC_RAW_BYTES = SHARED ? 2 * S::NP * TL * 4 : 0;
  static constexpr int WARP_RAW_BYTES = 4 * S::RPW * TL * (int)sizeof(T);
  static constexpr size_t kBytes = sizeof(float) * (BC_WORK + NW * WARP_WORK) + BC_RAW_BYTES + NW * WARP_RAW_BYTES;
  static_assert(kBytes <= 227 * 1024, "shared memory budget");
  static constexpr size_t bytes() { return kBytes; }
};

template <typename T, int NS, int LPR, bool SHARED>
__global__ void __launch_bounds__(BwdShape<T, NS, LPR, SHARED>::NW * 32, BwdShape<T, NS, LPR, SHARED>::NW == 4 ? 3 : 1) scan_bwd_kernel(const ssm_scan_bwd_args g, const ScanFlags fl) {
  using S = BwdShape<T, NS, LPR, SHARED>;
  constexpr int NP = S::NP, RPW = S::RPW, ROWS = S::ROWS, TB = S::TB, TL = S::TL, TLP = S::TLP, NW = S::NW;
  constexpr int V = 16 / sizeof(T);
  constexpr int NT = NW * 32;
  const ssm_scan_fwd_args& a = g.fwd;

  extern __shared__ __align__(16) float smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* sB = smem;  // [TL][NP] each
  float* sC = sB + S::BC_WORK / 2;
  float* wbase = smem + S::BC_WORK + warp * S::WARP_WORK;
  float* sDl = wbase;               // delta after bias / softplus (0 beyond the sequence)
  float* sU = sDl + RPW * TLP;      // u; overwritten step by step with ddelta once u is dead
  float* sDy = sU + RPW * TLP;      // dout * silu(z); overwritten step by step with du
  float* sZf = sDy + RPW * TLP;     // dout * silu'(z), finished into dz once y is rebuilt
  float* hist = sZf + RPW * TLP;    // [(TL/4+1)][32][NS]: slot m = state after step 4m-1 (slot 0: the checkpoint)
  float* stage = hist + S::WARP_HIST;
  char* rawbase = reinterpret_cast<char*>(smem + S::BC_WORK + NW * S::WARP_WORK);
  char* rawB = rawbase;
  char* rawC = rawbase + S::BC_RAW_BYTES / 2;
  T* rawU = reinterpret_cast<T*>(rawbase + S::BC_RAW_BYTES + warp * S::WARP_RAW_BYTES);
  T* rawD = rawU + RPW * TL;
  T* rawZ = rawD + RPW * TL;
  T* rawO = rawZ + RPW * TL;

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
  const T* __restrict__ gdo = reinterpret_cast<const T*>(g.dout);
  T* __restrict__ gdu = reinterpret_cast<T*>(g.du);
  T* __restrict__ gdd = reinterpret_cast<T*>(g.ddelta);
  T* __restrict__ gdz = reinterpret_cast<T*>(g.dz);

  // per-lane state as pairs of adjacent states for the packed-fp32 (f32x2) pipe
  float2 A2[NS / 2], carry[NS / 2], dAacc[NS / 2];
#pragma unroll
  for (int j = 0; j < NS; j += 2) {
    const int n = sg * NS + j;
    A2[j / 2].x = n < N ? __ldg(a.A + (int64_t)d * N + n) * kLog2e : 0.f;
    A2[j / 2].y = n + 1 < N ? __ldg(a.A + (int64_t)d * N + n + 1) * kLog2e : 0.f;
    carry[j / 2].x = (n < N && g.dlast_state) ? __ldg(g.dlast_state + row * N + n) : 0.f;
    carry[j / 2].y = (n + 1 < N && g.dlast_state) ? __ldg(g.dlast_state + row * N + n + 1) : 0.f;
    dAacc[j / 2] = make_float2(0.f, 0.f);
  }
  float dDacc = 0.f, dBiasAcc = 0.f;  // this lane's share of the row's dD / ddt_bias

  const int rpg = fl.rows_per_group;
  const int dref = SHARED ? min(d0, D - 1) : d;
  const int64_t boff = bc_row_offset(b, dref, rpg, a.b_sb, a.b_sg);
  const int64_t coff = bc_row_offset(b, dref, rpg, a.c_sb, a.c_sg);
  const int64_t dboff = bc_row_offset(b, dref, rpg, g.db_sb, g.db_sg);
  const int64_t dcoff = bc_row_offset(b, dref, rpg, g.dc_sb, g.dc_sg);
  const int bcsz = a.bc_dtype == SSM_F32 ? 4 : 2;
  const char* Bbase = reinterpret_cast<const char*>(a.Bm) + boff * bcsz;
  const char* Cbase = reinterpret_cast<const char*>(a.Cm) + coff * bcsz;
  const bool io_vec = fl.io_vec != 0, bc_vec = fl.bc_vec != 0;
  const int raw_bc_dtype = bc_vec ? a.bc_dtype : SSM_F32;

  const int ntiles = (L + TL - 1) / TL;
  const float Dv = a.D ? __ldg(a.D + d) : 0.f;

  auto fill_raw = [&](int t0) {
    fill_rows_raw<T, RPW, TL>(rawU, gu, b, D, L, drow0, t0, io_vec, lane, a.row_sb, a.row_sd);
    fill_rows_raw<T, RPW, TL>(rawD, gdl, b, D, L, drow0, t0, io_vec, lane, a.row_sb, a.row_sd);
    fill_rows_raw<T, RPW, TL>(rawO, gdo, b, D, L, drow0, t0, io_vec, lane, a.row_sb, a.row_sd);
    if (gz) fill_rows_raw<T, RPW, TL>(rawZ, gz, b, D, L, drow0, t0, io_vec, lane, a.row_sb, a.row_sd);
    if (SHARED) {
      fill_bc_raw<TL>(rawB, Bbase, a.bc_dtype, a.b_sn, a.b_st, N, t0, L, bc_vec, tid, NT);
      fill_bc_raw<TL>(rawC, Cbase, a.bc_dtype, a.c_sn, a.c_st, N, t0, L, bc_vec, tid, NT);
    }
    cp_async_commit();
  };

  // the checkpoint a tile starts from is fetched one tile ahead
  float2 hck[NS / 2];
  auto load_checkpoint = [&](int kt) {
    const float* ck = a.checkpoints + (row * ntiles + kt) * N;  // TL == checkpoint interval
#pragma unroll
    for (int j = 0; j < NS; j += 2) {
      hck[j / 2].x = (sg * NS + j) < N ? __ldg(ck + sg * NS + j) : 0.f;
      hck[j / 2].y = (sg * NS + j + 1) < N ? __ldg(ck + sg * NS + j + 1) : 0.f;
    }
  };
  if (ntiles > 0) {
    fill_raw((ntiles - 1) * TL);
    load_checkpoint(ntiles - 1);
  }

  for (int k = ntiles - 1; k >= 0; --k) {
    const int t0 = k * TL;
    cp_async_wait_all();
    __syncthreads();  // raw tile k landed; previous tile's working arrays consumed, dB / dC flushed

    // ---- raw -> fp32 working arrays -------------------------------------------------------
    {
      constexpr int CH = TL / V;
      for (int c = lane; c < RPW * CH; c += 32) {
        const int rr = c / CH, ch = c % CH;
        const int dd = min(drow0 + rr, D - 1);
        const int t = t0 + ch * V;
        float fu[V], fd[V], fz[V], fo[V], fdy[V], fzf[V];
        Vec16<T> v;
        v.raw = *reinterpret_cast<const uint4*>(rawU + rr * TL + ch * V);
        v.unpack(fu);
        v.raw = *reinterpret_cast<const uint4*>(rawD + rr * TL + ch * V);
        v.unpack(fd);
        v.raw = *reinterpret_cast<const uint4*>(rawO + rr * TL + ch * V);
        v.unpack(fo);
        if (gz) {
          v.raw = *reinterpret_cast<const uint4*>(rawZ + rr * TL + ch * V);
          v.unpack(fz);
        }
        const float bias = a.dt_bias ? __ldg(a.dt_bias + dd) : 0.f;
#pragma unroll
        for (int i = 0; i < V; ++i) {
          float x = fd[i] + bias;
          if (a.delta_softplus) x = softplus_fast(x);
          if (t + i >= L) x = 0.f;
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
        const int o = rr * TLP + ch * V;
#pragma unroll
        for (int i = 0; i < V; i += 4) {
          *reinterpret_cast<float4*>(sDl + o + i) = make_float4(fd[i], fd[i + 1], fd[i + 2], fd[i + 3]);
          *reinterpret_cast<float4*>(sU + o + i) = make_float4(fu[i], fu[i + 1], fu[i + 2], fu[i + 3]);
          *reinterpret_cast<float4*>(sDy + o + i) = make_float4(fdy[i], fdy[i + 1], fdy[i + 2], fdy[i + 3]);
          *reinterpret_cast<float4*>(sZf + o + i) = make_float4(fzf[i], fzf[i + 1], fzf[i + 2], fzf[i + 3]);
        }
      }
    }
    if (SHARED) {
      convert_bc<TL, NP>(sB, rawB, raw_bc_dtype, N, tid, NT);
      convert_bc<TL, NP>(sC, rawC, raw_bc_dtype, N, tid, NT);
    }
    __syncthreads();
    if (k > 0) fill_raw(t0 - TL);  // next (earlier) tile; overlaps the work below

    const float* rDl = sDl + r * TLP;
    float* rU = sU + r * TLP;
    float* rDy = sDy + r * TLP;
    float* rZf = sZf + r * TLP;
    float* hl = hist + lane * NS;  // this lane's states of slot m live at hl[m * 32 * NS]

    auto load_bc = [&](const float* tile, const char* base, int64_t sn, int64_t st, int tt, float (&v)[NS]) {
      if (SHARED) {
        load_states<NS, NP>(tile, tt, sg, v);
      } else {
        const int t = t0 + tt;
#pragma unroll
        for (int j = 0; j < NS; ++j) {
          const int n = sg * NS + j;
          v[j] = (n < N && t < L) ? load_dyn(base, (int64_t)n * sn + (int64_t)t * st, a.bc_dtype) : 0.f;
        }
      }
    };
    auto hist_store = [&](int slot, const float2 (&h)[NS / 2]) {
#pragma unroll
      for (int j = 0; j < NS; j += 4)
        *reinterpret_cast<float4*>(hl + slot * 32 * NS + j) = make_float4(h[j / 2].x, h[j / 2].y, h[j / 2 + 1].x, h[j / 2 + 1].y);
    };
    auto hist_load = [&](int slot, float2 (&h)[NS / 2]) {
#pragma unroll
      for (int j = 0; j < NS; j += 4) {
        const float4 q = *reinterpret_cast<const float4*>(hl + slot * 32 * NS + j);
        h[j / 2] = make_float2(q.x, q.y), h[j / 2 + 1] = make_float2(q.z, q.w);
      }
    };

    // ---- rebuild the tile's states from the checkpoint -----------------------------------------
    {
      float2 h[NS / 2];
#pragma unroll
      for (int j = 0; j < NS / 2; ++j) h[j] = hck[j];
      if (k > 0) load_checkpoint(k - 1);  // for the next (earlier) tile: its latency hides behind this tile's work
      hist_store(0, h);
#pragma unroll 2
      for (int tb0 = 0; tb0 < TL; tb0 += TB) {
        float p[TB];
#pragma unroll
        for (int q = 0; q < TB; q += 4) {
          const int tt = tb0 + q;
          const float4 dl4 = *reinterpret_cast<const float4*>(rDl + tt);
          const float4 u4 = *reinterpret_cast<const float4*>(rU + tt);
          const float dl[4] = {dl4.x, dl4.y, dl4.z, dl4.w};
          const float du[4] = {dl4.x * u4.x, dl4.y * u4.y, dl4.z * u4.z, dl4.w * u4.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float bv[NS], cv[NS];
            load_bc(sB, Bbase, a.b_sn, a.b_st, tt + i, bv);
            if (gz) load_bc(sC, Cbase, a.c_sn, a.c_st, tt + i, cv);
            const float2 dl2 = make_float2(dl[i], dl[i]);
            const float2 du2 = make_float2(du[i], du[i]);
            float2 acc = make_float2(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < NS; j += 2) {
              const float2 e = __fmul2_rn(dl2, A2[j / 2]);
              const float2 da = make_float2(ex2_approx(e.x), ex2_approx(e.y));
              h[j / 2] = __ffma2_rn(da, h[j / 2], __fmul2_rn(du2, make_float2(bv[j], bv[j + 1])));
              if (gz) acc = __ffma2_rn(make_float2(cv[j], cv[j + 1]), h[j / 2], acc);
            }
            if (i == 3) hist_store((tt + 4) / 4, h);  // the steps in between are rebuilt from their predecessors
            p[q + i] = acc.x + acc.y;
          }
        }
        if (gz) {  // dz = dout * silu'(z) * (sum_n C h + D u)
          reduce_scatter<LPR, 1, TB>(p, lane);
          constexpr int PER = TB / LPR;
#pragma unroll
          for (int i = 0; i < PER; ++i) {
            const int tt = tb0 + sg * PER + i;
            rZf[tt] *= fmaf(Dv, rU[tt], p[i]);
          }
        }
      }
    }
    __syncwarp();

    // ---- adjoint recurrence, last step of the tile first ------------------------------------------
    float2 hc[NS / 2];
    hist_load(TL / 4, hc);  // state after the tile's last step
#pragma unroll 1
    for (int tb0 = TL - TB; tb0 >= 0; tb0 -= TB) {
      float s1[TB], s2[TB];
#pragma unroll
      for (int q = TB - 4; q >= 0; q -= 4) {
        const int tt = tb0 + q;
        const float4 dl4 = *reinterpret_cast<const float4*>(rDl + tt);
        const float4 u4 = *reinterpret_cast<const float4*>(rU + tt);
        const float4 dy4 = *reinterpret_cast<const float4*>(rDy + tt);
        const float dl[4] = {dl4.x, dl4.y, dl4.z, dl4.w};
        const float du[4] = {dl4.x * u4.x, dl4.y * u4.y, dl4.z * u4.z, dl4.w * u4.w};
        const float dy[4] = {dy4.x, dy4.y, dy4.z, dy4.w};
        float vB[4 * NS], vC[4 * NS];  // entry i * NS + j: step tt + i, state j
        // states after steps tt - 1 .. tt + 2 (hs[0] from the history, the rest rebuilt) and the four decays
        float2 hs[4][NS / 2], da[4][NS / 2];
        hist_load(tt / 4, hs[0]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 dl2 = make_float2(dl[i], dl[i]);
#pragma unroll
          for (int j = 0; j < NS; j += 2) {
            const float2 e = __fmul2_rn(dl2, A2[j / 2]);
            da[i][j / 2] = make_float2(ex2_approx(e.x), ex2_approx(e.y));
          }
          if (i < 3) {
            float bv[NS];
            load_bc(sB, Bbase, a.b_sn, a.b_st, tt + i, bv);
            const float2 du2 = make_float2(du[i], du[i]);
#pragma unroll
            for (int j = 0; j < NS; j += 2)
              hs[i + 1][j / 2] = __ffma2_rn(da[i][j / 2], hs[i][j / 2], __fmul2_rn(du2, make_float2(bv[j], bv[j + 1])));
          }
        }
#pragma unroll
        for (int i = 3; i >= 0; --i) {
          // one adjoint step: hcur / hprev are the states after / before step tt + i
          float bv[NS], cv[NS];
          load_bc(sB, Bbase, a.b_sn, a.b_st, tt + i, bv);
          load_bc(sC, Cbase, a.c_sn, a.c_st, tt + i, cv);
          const float2 dl2 = make_float2(dl[i], dl[i]);
          const float2 du2 = make_float2(du[i], du[i]);
          const float2 dy2 = make_float2(dy[i], dy[i]);
          float2 a1 = make_float2(0.f, 0.f), a2 = make_float2(0.f, 0.f);
#pragma unroll
          for (int j = 0; j < NS; j += 2) {
            const float2 hcur = i == 3 ? hc[j / 2] : hs[i == 3 ? 0 : i + 1][j / 2];
            const float2 G = __ffma2_rn(make_float2(cv[j], cv[j + 1]), dy2, carry[j / 2]);
            const float2 vc = __fmul2_rn(dy2, hcur);
            const float2 vb = __fmul2_rn(G, du2);
            vC[i * NS + j] = vc.x, vC[i * NS + j + 1] = vc.y;
            vB[i * NS + j] = vb.x, vB[i * NS + j + 1] = vb.y;
            a1 = __ffma2_rn(G, make_float2(bv[j], bv[j + 1]), a1);
            const float2 gha = __fmul2_rn(__fmul2_rn(G, hs[i][j / 2]), da[i][j / 2]);
            a2 = __ffma2_rn(gha, A2[j / 2], a2);
            dAacc[j / 2] = __ffma2_rn(gha, dl2, dAacc[j / 2]);
            carry[j / 2] = __fmul2_rn(da[i][j / 2], G);
          }
          s1[q + i] = a1.x + a1.y, s2[q + i] = a2.x + a2.y;
        }
#pragma unroll
        for (int j = 0; j < NS / 2; ++j) hc[j] = hs[0][j];
        if (SHARED) {
          // lanes -> staging area: group (output o, row slot) holds the four steps' products
          constexpr int ROT = LPR <= 8 ? 8 / LPR : 0;
          const int slot = (r + ROT * sg) & (RPW - 1);
#pragma unroll
          for (int j = 0; j < NS; ++j) {
            const int o = sg * NS + j;
            *reinterpret_cast<float4*>(stage + ((o * RPW + slot) << 2)) = make_float4(vB[j], vB[NS + j], vB[2 * NS + j], vB[3 * NS + j]);
            *reinterpret_cast<float4*>(stage + (((NP + o) * RPW + slot) << 2)) = make_float4(vC[j], vC[NS + j], vC[2 * NS + j], vC[3 * NS + j]);
          }
          __syncwarp();
          constexpr int O = 2 * NP;                  // outputs: (dB | dC) x state
          constexpr int PARTS = O >= 32 ? 1 : 32 / O;  // lanes sharing one output, each summing RPW / PARTS rows
          constexpr int RP = RPW / PARTS;
#pragma unroll
          for (int m = 0; m < (O >= 32 ? O / 32 : 1); ++m) {
            const int o = O >= 32 ? lane + 32 * m : lane % O;
            const int part = O >= 32 ? 0 : lane / O;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int kk = 0; kk < RP; ++kk) {
              const int sl = part * RP + ((kk + o) & (RP - 1));
              const float4 v = *reinterpret_cast<const float4*>(stage + ((o * RPW + sl) << 2));
              acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
            }
#pragma unroll
            for (int off = O; off < 32; off <<= 1) {
              acc.x += __shfl_xor_sync(0xffffffffu, acc.x, off);
              acc.y += __shfl_xor_sync(0xffffffffu, acc.y, off);
              acc.z += __shfl_xor_sync(0xffffffffu, acc.z, off);
              acc.w += __shfl_xor_sync(0xffffffffu, acc.w, off);
            }
            const int n = o % NP;
            const int t = t0 + tt;
            if (part == 0 && n < N && t < L) {
              float* dst = o < NP ? g.dB + dboff + (int64_t)n * g.db_sn + (int64_t)t * g.db_st
                                  : g.dC + dcoff + (int64_t)n * g.dc_sn + (int64_t)t * g.dc_st;
              const int64_t st = o < NP ? g.db_st : g.dc_st;
              if (st == 1 && t + 3 < L && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(acc.x), "f"(acc.y), "f"(acc.z), "f"(acc.w) : "memory");
              } else {
                const float av[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  if (t + i < L) atomicAdd(dst + i * st, av[i]);
              }
            }
          }
          __syncwarp();  // staging area is free for the next four steps
        } else if (row_ok) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int t = t0 + tt + i;
#pragma unroll
            for (int j = 0; j < NS; ++j) {
              const int n = sg * NS + j;
              if (n < N && t < L) {
                atomicAdd(g.dB + dboff + (int64_t)n * g.db_sn + (int64_t)t * g.db_st, vB[i * NS + j]);
                atomicAdd(g.dC + dcoff + (int64_t)n * g.dc_sn + (int64_t)t * g.dc_st, vC[i * NS + j]);
              }
            }
          }
        }
      }
      reduce_scatter<LPR, 1, TB>(s1, lane);
      reduce_scatter<LPR, 1, TB>(s2, lane);
      constexpr int PER = TB / LPR;
#pragma unroll
      __syncwarp();  // every lane has read this batch's u / dy before they are overwritten
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int tt = tb0 + sg * PER + i;
        const float dlv = rDl[tt], uv = rU[tt], dyv = rDy[tt];
        dDacc = fmaf(dyv, uv, dDacc);
        float dd = fmaf(s1[i], uv, s2[i] * kLn2);
        // d softplus(pre) / d pre = sigmoid(pre) = 1 - exp(-softplus(pre))
        if (a.delta_softplus) dd *= one_minus_exp_neg(dlv);
        if (t0 + tt < L) dBiasAcc += dd;
        rDy[tt] = fmaf(s1[i], dlv, dyv * Dv);  // du
        rU[tt] = dd;                           // ddelta
      }
    }
    __syncwarp();

    // ---- write du / ddelta / dz -----------------------------------------------------------------
    if (io_vec) {
      constexpr int CH = TL / V;
      for (int c = lane; c < RPW * CH; c += 32) {
        const int rr = c / CH, ch = c % CH;
        const int dd = drow0 + rr;
        const int t = t0 + ch * V;
        if (dd < D && t < L) {
          const int o = rr * TLP + ch * V;
          const int64_t base = (int64_t)b * a.row_sb + (int64_t)dd * a.row_sd + t;
          float f[V];
          Vec16<T> v;
#pragma unroll
          for (int i = 0; i < V; i += 4) {
            const float4 q = *reinterpret_cast<const float4*>(sDy + o + i);
            f[i] = q.x, f[i + 1] = q.y, f[i + 2] = q.z, f[i + 3] = q.w;
          }
          v.pack(f);
          v.store_stream(gdu + base);
#pragma unroll
          for (int i = 0; i < V; i += 4) {
            const float4 q = *reinterpret_cast<const float4*>(sU + o + i);
            f[i] = q.x, f[i + 1] = q.y, f[i + 2] = q.z, f[i + 3] = q.w;
          }
          v.pack(f);
          v.store_stream(gdd + base);
          if (gdz) {
#pragma unroll
            for (int i = 0; i < V; i += 4) {
              const float4 q = *reinterpret_cast<const float4*>(sZf + o + i);
              f[i] = q.x, f[i + 1] = q.y, f[i + 2] = q.z, f[i + 3] = q.w;
            }
            v.pack(f);
            v.store_stream(gdz + base);
          }
        }
      }
    } else {
      for (int i = lane; i < RPW * TL; i += 32) {
        const int rr = i / TL, tt = i % TL;
        const int dd = drow0 + rr;
        const int t = t0 + tt;
        if (dd < D && t < L) {
          const int o = rr * TLP + tt;
          const int64_t base = (int64_t)b * a.row_sb + (int64_t)dd * a.row_sd + t;
          gdu[base] = from_f<T>(sDy[o]);
          gdd[base] = from_f<T>(sU[o]);
          if (gdz) gdz[base] = from_f<T>(sZf[o]);
        }
      }
    }
  }

  dDacc = group_sum<LPR, 1>(dDacc);
  dBiasAcc = group_sum<LPR, 1>(dBiasAcc);
  if (g.dinitial_state && row_ok) {  // what the adjoint carries past step 0 is the gradient of the state before it
#pragma unroll
    for (int j = 0; j < NS; j += 2) {
      const int n = sg * NS + j;
      if (n < N) g.dinitial_state[row * N + n] = carry[j / 2].x;
      if (n + 1 < N) g.dinitial_state[row * N + n + 1] = carry[j / 2].y;
    }
  }
  if (row_ok) {
#pragma unroll
    for (int j = 0; j < NS; j += 2) {
      const int n = sg * NS + j;
      if (n < N) atomicAdd(g.dA + (int64_t)d * N + n, dAacc[j / 2].x);
      if (n + 1 < N) atomicAdd(g.dA + (int64_t)d * N + n + 1, dAacc[j / 2].y);
    }
    if (sg == 0) {
      if (g.dD) atomicAdd(g.dD + d, dDacc);
      if (g.ddt_bias) atomicAdd(g.ddt_bias + d, dBiasAcc);
    }
  }
}

template <typename T, int NS, int LPR>
static int launch_bwd(const ssm_scan_bwd_args& g, ScanFlags fl, cudaStream_t st) {
  using S1 = BwdShape<T, NS, LPR, false>;
  // the CTA-wide B / C / dB / dC tiles of more than 128 states do not fit next to the state
  // history; such rows read B / C from global memory and accumulate dB / dC there directly
  constexpr bool kCanShare = NS * LPR <= 128;
  const ssm_scan_fwd_args& a = g.fwd;
  fl.shared_bc = kCanShare && (fl.rows_per_group % S1::ROWS == 0);
  dim3 grid((a.dim + S1::ROWS - 1) / S1::ROWS, a.batch);
  if constexpr (kCanShare) {
    if (fl.shared_bc) {
      const size_t smem = BwdShape<T, NS, LPR, true>::bytes();
      auto kern = scan_bwd_kernel<T, NS, LPR, true>;
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      kern<<<grid, S1::NW * 32, smem, st>>>(g, fl);
      return launch_status("scan_bwd_kernel");
    }
  }
  {
    const size_t smem = BwdShape<T, NS, LPR, false>::bytes();
    auto kern = scan_bwd_kernel<T, NS, LPR, false>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<grid, S1::NW * 32, smem, st>>>(g, fl);
  }
  return launch_status("scan_bwd_kernel");
}

template <typename T>
int dispatch_bwd(const ssm_scan_bwd_args& g, const ScanFlags& fl, cudaStream_t st) {
  const int n = g.fwd.nstate;
  if (n <= 4) return launch_bwd<T, 4, 1>(g, fl, st);
  if (n <= 8) return launch_bwd<T, 4, 2>(g, fl, st);
  if (n <= 16) return launch_bwd<T, 4, 4>(g, fl, st);
  if (n <= 32) return launch_bwd<T, 4, 8>(g, fl, st);
  if (n <= 64) return launch_bwd<T, 4, 16>(g, fl, st);
  if (n <= 128) return launch_bwd<T, 4, 32>(g, fl, st);
  return launch_bwd<T, 8, 32>(g, fl, st);
}

int scan_validate(const ssm_scan_fwd_args* a, ScanFlags* fl, int rows_per_cta);

}  // namespace ssmb

