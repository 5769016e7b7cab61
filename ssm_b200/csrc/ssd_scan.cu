// State-space-dual (Mamba-2) chunked scan with a d_state axis, forward, for sm_100a.
//
//   delta_t = softplus?(dt_t + dt_bias);  S_t = exp(delta_t A) S_{t-1} + delta_t x_t B_t^T;  y_t = S_t C_t + D x_t;  y_t *= silu(z_t)
//
// evaluated chunk by chunk (Q = 256 steps) in the dual, matrix form, with every contraction on
// the tcgen05 tensor cores (bf16 / fp16 operands from shared memory, fp32 accumulators in TMEM):
//
//   ssd_cumsum_kernel   delta and its running log-decay  cum_i = sum_{k<=i} delta_k A  per chunk
//   ssd_state_kernel    per (batch, chunk, head): local state  S_c = sum_j exp(cum_last - cum_j) delta_j x_j B_j^T   [N x P GEMM, K = Q]
//   ssd_pass_kernel     the short serial pass over chunks: incoming state of every chunk (kept in
//                       the operand dtype for the GEMM below) and the final state in fp32
//   ssd_scan_kernel     per (batch, chunk, head), one warpgroup per 128-row block:  G = C B^T  (TMEM), the decay mask
//                       exp(cum_i - cum_j) delta_j [j <= i] applied on the TMEM -> register path and
//                       re-packed as the A operand of  Y_intra = (G o L) X, plus  Y_inter = C S_in;
//                       y = Y_intra + exp(cum_i) Y_inter + D x, gated, stored.
//
// Exponent differences are always formed before exp (never exp(cum_i) / exp(cum_j)), so long
// sequences stay finite.  Every wait on an mbarrier is bounded and reports through the status word.
#include <type_traits>

#include "common.cuh"
#include "scan_common.cuh"
#include "tc05.cuh"

namespace ssmb {

constexpr int kQ = 256;    // chunk length
constexpr int kP = 64;     // head dimension
constexpr int kN = 128;    // state dimension
constexpr int kBlk = 128;  // rows per scan CTA

// ---------------------------------------------------------------------------------------------
// delta and within-chunk cumulative log-decay; one warp per (batch, head, chunk)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) ssd_cumsum_kernel(const ssm_ssd_args a, int nchunks) {
  const int warp = (blockIdx.x * 128 + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int total = a.batch * a.heads * nchunks;
  if (warp >= total) return;
  const int c = warp % nchunks, h = (warp / nchunks) % a.heads, b = warp / (nchunks * a.heads);
  const float Ah = __ldg(a.A + h);
  const float bias = a.dt_bias ? __ldg(a.dt_bias + h) : 0.f;
  const T* dt = reinterpret_cast<const T*>(a.dt);
  float* odt = a.ws_dt + ((int64_t)b * a.heads + h) * nchunks * kQ + (int64_t)c * kQ;
  float* ocum = a.ws_cum + ((int64_t)b * a.heads + h) * nchunks * kQ + (int64_t)c * kQ;
  float d[kQ / 32], run = 0.f;
#pragma unroll
  for (int k = 0; k < kQ / 32; ++k) {
    const int i = lane * (kQ / 32) + k;  // each lane owns 8 consecutive steps
    const int t = c * kQ + i;
    float v = 0.f;
    if (t < a.len) {
      v = to_f<T>(dt[((int64_t)b * a.len + t) * a.heads + h]) + bias;
      if (a.dt_softplus) v = softplus_f(v);
    }
    d[k] = v;
    run += v * Ah;
  }
  // exclusive prefix of the lane sums
  float pre = run;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float o = __shfl_up_sync(0xffffffffu, pre, off);
    if (lane >= off) pre += o;
  }
  float acc = pre - run;
#pragma unroll
  for (int k = 0; k < kQ / 32; ++k) {
    const int i = lane * (kQ / 32) + k;
    acc += d[k] * Ah;
    odt[i] = d[k];
    ocum[i] = acc;
  }
}

// ---------------------------------------------------------------------------------------------
// local chunk states on the tensor cores:  S[n][p] = sum_j B[j][n] * (w_j x[j][p])
//   A operand = B^T, MN-major [n/8][j][8];  B operand = w x, MN-major [p/8][j][8];  M = 128 (n), N = 64 (p), K = 256 (j)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) ssd_state_kernel(const ssm_ssd_args a, int nchunks) {
  extern __shared__ __align__(128) unsigned char smraw[];
  T* sA = reinterpret_cast<T*>(smraw);                       // 16 x 256 units of 16 bytes = 64 KB
  T* sB = reinterpret_cast<T*>(smraw + (kN / 8) * kQ * 16);   //  8 x 256 units           = 32 KB
  __shared__ __align__(8) uint64_t mbar;
  __shared__ uint32_t tmem_slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int g = h / (a.heads / a.groups);
  const int t0 = c * kQ;

  if (warp == 0) tc::tmem_alloc(tc::smem_u32(&tmem_slot), 64);
  if (tid == 0) tc::mbar_init(tc::smem_u32(&mbar), 1);

  // ---- B^T tile: raw 16-byte units, step index fastest across threads -----------------------
  const T* Bg = reinterpret_cast<const T*>(a.Bm);
  for (int id = tid; id < (kN / 8) * kQ; id += 128) {
    const int nc = id / kQ, j = id % kQ;
    const int t = t0 + j;
    const bool okt = t < a.len;
    cp_async16(reinterpret_cast<unsigned char*>(sA) + ((size_t)nc * kQ + j) * 16,
               Bg + (((int64_t)b * a.len + (okt ? t : 0)) * a.groups + g) * kN + nc * 8, okt);
  }
  cp_async_commit();
  // ---- x tile scaled by w_j = exp(cum_last - cum_j) * delta_j ---------------------------------
  const float* wdt = a.ws_dt + (((int64_t)b * a.heads + h) * nchunks + c) * kQ;
  const float* wcum = a.ws_cum + (((int64_t)b * a.heads + h) * nchunks + c) * kQ;
  const float cum_last = __ldg(wcum + kQ - 1);
  const T* Xg = reinterpret_cast<const T*>(a.X);
  constexpr int XU = 8;  // units per thread kept in flight together
  for (int id0 = tid; id0 < (kP / 8) * kQ; id0 += 128 * XU) {
    Vec16<T> v[XU];
    float w[XU];
#pragma unroll
    for (int q = 0; q < XU; ++q) {
      const int id = id0 + q * 128;
      const int pc = id / kQ, j = id % kQ;
      const int t = t0 + j;
      v[q].raw = make_uint4(0, 0, 0, 0);
      w[q] = 0.f;
      if (t < a.len) {
        v[q].load(Xg + (((int64_t)b * a.len + t) * a.heads + h) * kP + pc * 8);
        w[q] = exp_fast(cum_last - __ldg(wcum + j)) * __ldg(wdt + j);
      }
    }
#pragma unroll
    for (int q = 0; q < XU; ++q) {
      const int id = id0 + q * 128;
      const int pc = id / kQ, j = id % kQ;
      float f[8];
      v[q].unpack(f);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] *= w[q];
      Vec16<T> o;
      o.pack(f);
      *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(sB) + ((size_t)pc * kQ + j) * 16) = o.raw;
    }
  }
  cp_async_wait_all();
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_slot;

  if (tid == 0) {
    constexpr uint32_t idesc = tc::instr_desc(kN, kP, std::is_same<T, __nv_bfloat16>::value ? 1 : 0, 1, 1);
    const uint32_t a0 = tc::smem_u32(sA), b0 = tc::smem_u32(sB);
#pragma unroll 1
    for (int kk = 0; kk < kQ / 16; ++kk) {
      const uint64_t da = tc::smem_desc(a0 + kk * 256, 128, kQ * 16);  // two groups of 8 steps = 256 bytes per instruction
      const uint64_t db = tc::smem_desc(b0 + kk * 256, 128, kQ * 16);
      tc::mma_ss(tmem, da, db, idesc, kk > 0);
    }
    tc::commit(tc::smem_u32(&mbar));
  }
  const bool ok = __all_sync(0xffffffffu, tc::mbar_wait(tc::smem_u32(&mbar), 0));  // warp-uniform
  tc::fence_after_sync();
  if (!ok && a.status) atomicExch(a.status, 1);

  // ---- TMEM -> global: thread = state n, 64 columns = p ---------------------------------------
  if (ok) {
    float* out = a.ws_state + ((((int64_t)b * nchunks + c) * a.heads + h) * kP) * kN;
    const int n = warp * 32 + lane;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float v[32];
      tc::tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + half * 32, v);
#pragma unroll
      for (int i = 0; i < 32; ++i) out[(int64_t)(half * 32 + i) * kN + n] = v[i];
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, 64);
}

// ---------------------------------------------------------------------------------------------
// serial pass over chunks: one thread per (batch, head, p, n)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) ssd_pass_kernel(const ssm_ssd_args a, int nchunks) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const int64_t per = (int64_t)kP * kN;
  const int64_t total = (int64_t)a.batch * a.heads * per;
  if (i >= total) return;
  const int64_t bh = i / per, pn = i % per;
  const int b = (int)(bh / a.heads), h = (int)(bh % a.heads);
  float s = a.initial_states ? __ldg(a.initial_states + i) : 0.f;
  T* sin = reinterpret_cast<T*>(a.ws_state_in);
  for (int c = 0; c < nchunks; ++c) {
    const int64_t slot = (((int64_t)b * nchunks + c) * a.heads + h) * per + pn;
    sin[slot] = from_f<T>(s);
    const float decay = exp_fast(__ldg(a.ws_cum + (((int64_t)b * a.heads + h) * nchunks + c) * kQ + kQ - 1));
    s = fmaf(decay, s, a.ws_state[slot]);
  }
  if (a.final_states) a.final_states[i] = s;
}

// ---------------------------------------------------------------------------------------------
// chunk scan: one CTA of two warpgroups per (head, batch * chunk); warpgroup w owns rows
// [128 w, 128 w + 128) of the chunk.  Both share the staged C, B, x and incoming-state tiles.
//   TMEM columns: G0 [0,128) (rows 0..127 x steps 0..127), G1 [128,384) (rows 128..255 x steps
//   0..255), C S_in of block 0 [384,448) and of block 1 [448,512); (G o L) X of block w is
//   accumulated over the first 64 columns of G_w once the warpgroup has consumed G_w.
//   Shared memory: the masked tile of block 0 overwrites the C tile, that of block 1 the B tile
//   (both dead once the first group of MMAs has completed).
// ---------------------------------------------------------------------------------------------
template <typename T>
struct ScanSmem {
  static constexpr int C_BYTES = kQ * kN * 2;   // C rows of the chunk, K-major [n/8][i][8]   64 KB
  static constexpr int B_BYTES = kQ * kN * 2;   // B rows of the chunk, K-major [n/8][j][8]   64 KB
  static constexpr int X_BYTES = kQ * kP * 2;   // x rows, MN-major [p/8][j][8]               32 KB
  static constexpr int S_BYTES = kP * kN * 2;   // incoming state, K-major [n/8][p][8]        16 KB
  static constexpr int VEC_BYTES = 2 * kQ * 4;  // cum and delta of the chunk
  static constexpr int TOTAL = C_BYTES + B_BYTES + X_BYTES + S_BYTES + VEC_BYTES;
};

__device__ __forceinline__ void named_barrier(int id, int nthreads) { asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(nthreads) : "memory"); }

template <typename T>
__global__ void __launch_bounds__(256) ssd_scan_kernel(const ssm_ssd_args a, int nchunks) {
  using M = ScanSmem<T>;
  extern __shared__ __align__(128) unsigned char smraw[];
  unsigned char* sC = smraw;
  unsigned char* sB = sC + M::C_BYTES;
  unsigned char* sX = sB + M::B_BYTES;
  unsigned char* sS = sX + M::X_BYTES;
  float* sCum = reinterpret_cast<float*>(sS + M::S_BYTES);
  float* sDt = sCum + kQ;
  __shared__ __align__(8) uint64_t mbar[3];
  __shared__ uint32_t tmem_slot;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int wg = tid >> 7, wtid = tid & 127;  // warpgroup = row block
  const int h = blockIdx.x;
  const int c = blockIdx.y % nchunks, b = blockIdx.y / nchunks;
  const int g = h / (a.heads / a.groups);
  const int t0 = c * kQ;
  const int KJ = (wg + 1) * kBlk;      // causal: steps j < KJ can reach this warpgroup's rows
  const int i_loc = wg * kBlk + wtid;  // this thread's row within the chunk
  const int t_row = t0 + i_loc;
  constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;

  if (warp == 0) tc::tmem_alloc(tc::smem_u32(&tmem_slot), 512);
  if (tid == 0) {
    tc::mbar_init(tc::smem_u32(&mbar[0]), 1);
    tc::mbar_init(tc::smem_u32(&mbar[1]), 1);
    tc::mbar_init(tc::smem_u32(&mbar[2]), 1);
  }

  // ---- stage operands (asynchronous 16-byte copies, step index fastest across threads) ----------
  const float* wdt = a.ws_dt + (((int64_t)b * a.heads + h) * nchunks + c) * kQ;
  const float* wcum = a.ws_cum + (((int64_t)b * a.heads + h) * nchunks + c) * kQ;
  sCum[tid] = __ldg(wcum + tid), sDt[tid] = __ldg(wdt + tid);
  const T* Cg = reinterpret_cast<const T*>(a.Cm);
  const T* Bg = reinterpret_cast<const T*>(a.Bm);
  const T* Xg = reinterpret_cast<const T*>(a.X);
  for (int id = tid; id < (kN / 8) * kQ; id += 256) {
    const int nc = id / kQ, j = id % kQ;
    const int t = t0 + j;
    const bool okt = t < a.len;
    const int64_t off = (((int64_t)b * a.len + (okt ? t : 0)) * a.groups + g) * kN + nc * 8;
    cp_async16(sC + ((size_t)nc * kQ + j) * 16, Cg + off, okt);
    cp_async16(sB + ((size_t)nc * kQ + j) * 16, Bg + off, okt);
  }
  for (int id = tid; id < (kP / 8) * kQ; id += 256) {
    const int pc = id / kQ, j = id % kQ;
    const int t = t0 + j;
    const bool okt = t < a.len;
    cp_async16(sX + ((size_t)pc * kQ + j) * 16, Xg + (((int64_t)b * a.len + (okt ? t : 0)) * a.heads + h) * kP + pc * 8, okt);
  }
  {
    const T* Sg = reinterpret_cast<const T*>(a.ws_state_in) + ((((int64_t)b * nchunks + c) * a.heads + h) * kP) * kN;
    for (int id = tid; id < (kN / 8) * kP; id += 256) {
      const int nc = id / kP, p = id % kP;
      cp_async16(sS + ((size_t)nc * kP + p) * 16, Sg + (int64_t)p * kN + nc * 8, true);
    }
  }
  cp_async_commit();
  cp_async_wait_all();
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t tG = tmem + (wg == 0 ? 0 : 128);    // this warpgroup's G, later its (G o L) X
  const uint32_t tYs = tmem + 384 + wg * 64;         // this warpgroup's C S_in

  // ---- G = C B^T and Y_inter = C S_in for both row blocks ------------------------------------------
  if (tid == 0) {
    const uint32_t c0 = tc::smem_u32(sC), b0 = tc::smem_u32(sB), s0 = tc::smem_u32(sS);
    const uint32_t idS = tc::instr_desc(kBlk, kP, fmt, 0, 0);
#pragma unroll 1
    for (int blk = 0; blk < 2; ++blk) {
      const uint32_t idG = tc::instr_desc(kBlk, (blk + 1) * kBlk, fmt, 0, 0);
      const uint32_t dG = tmem + (blk == 0 ? 0 : 128), dS = tmem + 384 + blk * 64;
#pragma unroll 1
      for (int kk = 0; kk < kN / 16; ++kk) {
        const uint64_t da = tc::smem_desc(c0 + blk * (kBlk * 16) + kk * 2 * (kQ * 16), kQ * 16, 128);
        const uint64_t db = tc::smem_desc(b0 + kk * 2 * (kQ * 16), kQ * 16, 128);
        const uint64_t ds = tc::smem_desc(s0 + kk * 2 * (kP * 16), kP * 16, 128);
        tc::mma_ss(dG, da, db, idG, kk > 0);
        tc::mma_ss(dS, da, ds, idS, kk > 0);
      }
    }
    tc::commit(tc::smem_u32(&mbar[0]));
  }
  bool ok = __all_sync(0xffffffffu, tc::mbar_wait(tc::smem_u32(&mbar[0]), 0));  // warp-uniform
  tc::fence_after_sync();

  // ---- decay mask on the TMEM -> register path; the masked tile (K-major over j, 128 rows) replaces
  // ---- a dead operand tile: unit (i, j/8) at (j/8) * (128 * 16) + i * 16 -----------------------------
  unsigned char* sA = wg == 0 ? sC : sB;
  const float cum_i = sCum[i_loc];
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  if (ok) {
    for (int jb = 0; jb < KJ; jb += 32) {
      float v[32];
      tc::tmem_ld32(tG + lane_base + jb, v);
#pragma unroll
      for (int q = 0; q < 32; q += 8) {
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int j = jb + q + e;
          const float m = (j <= i_loc) ? exp_fast(cum_i - sCum[j]) * sDt[j] : 0.f;
          f[e] = v[q + e] * m;
        }
        Vec16<T> o;
        o.pack(f);
        *reinterpret_cast<uint4*>(sA + ((size_t)((jb + q) / 8) * kBlk + wtid) * 16) = o.raw;
      }
    }
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  // Both warpgroups must have left the first MMA group's operands before either overwrites them
  // (block 0's masked tile lands on the C tile that block 1's G also read): that is guaranteed by
  // the wait on mbar[0] above, which covers all of those MMAs.  From here the warpgroups run apart.
  named_barrier(1 + wg, 128);
  tc::fence_after_sync();

  // ---- Y_intra = (G o L) X over this warpgroup's own columns ----------------------------------------
  if (wtid == 0) {
    const uint32_t g0 = tc::smem_u32(sA), x0 = tc::smem_u32(sX);
    const uint32_t idY = tc::instr_desc(kBlk, kP, fmt, 0, 1);
#pragma unroll 1
    for (int kk = 0; kk < KJ / 16; ++kk) {
      const uint64_t da = tc::smem_desc(g0 + kk * 2 * (kBlk * 16), kBlk * 16, 128);
      const uint64_t dx = tc::smem_desc(x0 + kk * 256, 128, kQ * 16);
      tc::mma_ss(tG, da, dx, idY, kk > 0);
    }
    tc::commit(tc::smem_u32(&mbar[1 + wg]));
  }
  ok = __all_sync(0xffffffffu, tc::mbar_wait(tc::smem_u32(&mbar[1 + wg]), 0)) && ok;
  tc::fence_after_sync();
  if (!ok && a.status) atomicExch(a.status, 2);

  // ---- epilogue: y = Y_intra + exp(cum_i) Y_inter + D x, gate, store ----------------------------------
  if (ok) {
    const bool live = t_row < a.len;  // the TMEM loads below are warp-wide; only the stores are per row
    const float escale = exp_fast(cum_i);
    const T* zrow = a.z ? reinterpret_cast<const T*>(a.z) + (((int64_t)b * a.len + t_row) * a.heads + h) * kP : nullptr;
    T* yrow = reinterpret_cast<T*>(a.Y) + (((int64_t)b * a.len + t_row) * a.heads + h) * kP;
    const float Dh = (a.D && !a.d_has_p) ? __ldg(a.D + h) : 0.f;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float yi[32], ys[32];
      tc::tmem_ld32(tG + lane_base + half * 32, yi);
      tc::tmem_ld32(tYs + lane_base + half * 32, ys);
      Vec16<T> zr[4];
      if (zrow && live) {
#pragma unroll
        for (int q = 0; q < 4; ++q) zr[q].load(zrow + half * 32 + q * 8);
      }
#pragma unroll
      for (int q = 0; q < 32; q += 8) {
        const int p0 = half * 32 + q;
        float f[8], xv[8];
        Vec16<T> xr;
        xr.raw = *reinterpret_cast<const uint4*>(sX + ((size_t)(p0 / 8) * kQ + i_loc) * 16);
        xr.unpack(xv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float Dv = (a.D && a.d_has_p) ? __ldg(a.D + h * kP + p0 + e) : Dh;
          f[e] = fmaf(escale, ys[q + e], yi[q + e]) + Dv * xv[e];
        }
        if (zrow && live) {
          float zv[8];
          zr[q / 8].unpack(zv);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] *= silu_fast(zv[e]);
        }
        Vec16<T> o;
        o.pack(f);
        if (live) o.store(yrow + p0);
      }
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, 512);
}

template <typename T>
static int ssd_launch(const ssm_ssd_args& a, cudaStream_t st) {
  const int nchunks = (a.len + kQ - 1) / kQ;
  if (a.phase != 2) {
    const int warps = a.batch * a.heads * nchunks;
    ssd_cumsum_kernel<T><<<(warps * 32 + 127) / 128, 128, 0, st>>>(a, nchunks);
    if (int rc = launch_status("ssd_cumsum_kernel")) return rc;
  }
  if (a.phase != 2) {
    const size_t smem = (kN / 8 + kP / 8) * kQ * 16;
    cudaFuncSetAttribute(ssd_state_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ssd_state_kernel<T><<<dim3(nchunks, a.heads, a.batch), 128, smem, st>>>(a, nchunks);
    if (int rc = launch_status("ssd_state_kernel")) return rc;
  }
  {
    const int64_t total = (int64_t)a.batch * a.heads * kP * kN;
    ssd_pass_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(a, nchunks);
    if (int rc = launch_status("ssd_pass_kernel")) return rc;
  }
  if (a.phase != 1) {
    const size_t smem = ScanSmem<T>::TOTAL;
    cudaFuncSetAttribute(ssd_scan_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ssd_scan_kernel<T><<<dim3(a.heads, a.batch * nchunks), 256, smem, st>>>(a, nchunks);
    if (int rc = launch_status("ssd_scan_kernel")) return rc;
  }
  return SSM_OK;
}

}  // namespace ssmb

using namespace ssmb;

extern "C" int ssm_ssd_supported(int32_t headdim, int32_t nstate, int32_t chunk_size, int32_t io_dtype) {
  return headdim == kP && nstate == kN && chunk_size == kQ && (io_dtype == SSM_BF16 || io_dtype == SSM_F16);
}

extern "C" int64_t ssm_ssd_scratch_bytes(int32_t batch, int32_t len, int32_t heads) {
  const int64_t nchunks = (len + kQ - 1) / kQ;
  const int64_t vec = (int64_t)batch * heads * nchunks * kQ * 4;      // delta, cum (each)
  const int64_t st = (int64_t)batch * nchunks * heads * kP * kN;      // states per chunk
  return 2 * vec + st * 4 + st * 2;
}

extern "C" int ssm_ssd_fwd(const ssm_ssd_args* a, ssm_stream_t stream) {
  SSM_REQUIRE(a != nullptr, SSM_ERR_NULL, "ssd_scan: args is NULL");
  SSM_REQUIRE(a->batch >= 0 && a->len >= 0 && a->heads >= 1 && a->groups >= 1, SSM_ERR_SHAPE, "ssd_scan: bad shape");
  SSM_REQUIRE(a->heads % a->groups == 0, SSM_ERR_SHAPE, "Group dimension must divide H.");
  SSM_REQUIRE(ssm_ssd_supported(a->headdim, a->nstate, a->chunk_size, a->io_dtype), SSM_ERR_UNSUPPORTED,
              "ssd_scan: the tensor-core path is built for headdim 64, d_state 128, chunk 256, bf16 / fp16");
  if (a->batch == 0 || a->len == 0) return SSM_OK;
  SSM_REQUIRE(a->phase >= 0 && a->phase <= 2, SSM_ERR_SHAPE, "ssd_scan: phase must be 0, 1 or 2");
  SSM_REQUIRE(a->X && a->dt && a->A && a->Bm && a->Cm && (a->Y || a->phase == 1), SSM_ERR_NULL, "ssd_scan: missing tensor");
  SSM_REQUIRE(a->ws_dt && a->ws_cum && a->ws_state && a->ws_state_in, SSM_ERR_NULL, "ssd_scan: missing scratch");
  SSM_REQUIRE(aligned_to(a->X, 16) && aligned_to(a->Bm, 16) && aligned_to(a->Cm, 16) && (!a->Y || aligned_to(a->Y, 16)) && aligned_to(a->ws_state_in, 16) &&
                  (!a->z || aligned_to(a->z, 16)),
              SSM_ERR_ALIGN, "ssd_scan: tensors must be 16-byte aligned");
  const int64_t nchunks = (a->len + kQ - 1) / kQ;
  SSM_REQUIRE((int64_t)a->batch * nchunks <= 65535 && a->heads <= 65535, SSM_ERR_TOO_LARGE, "ssd_scan: grid too large");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a->io_dtype == SSM_BF16) return ssd_launch<__nv_bfloat16>(*a, st);
  return ssd_launch<__half>(*a, st);
}
