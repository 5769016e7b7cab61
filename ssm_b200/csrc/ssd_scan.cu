// State-space-dual (Mamba-2) chunked scan with a d_state axis, forward, for sm_100a.
//
//   delta_t = softplus?(dt_t + dt_bias);  S_t = exp(delta_t A) S_{t-1} + delta_t x_t B_t^T;  y_t = S_t C_t + D x_t;  y_t *= silu(z_t)
//
// evaluated chunk by chunk (Q = 256 steps) in the dual, matrix form, with every contraction on
// the tcgen05 tensor cores (bf16 / fp16 operands in shared memory, staged by TMA, fp32 accumulators in TMEM):
//
//   ssd_cumsum_kernel   per chunk the running decay exponent  c_i = log2(e) sum_{k<=i} delta_k A  and  c_i - log2(delta_i)
//   ssd_state_kernel    per (batch, a few heads), chunks in order: local state  S_c = sum_j exp2(c_last - c_j) delta_j x_j B_j^T
//                       [N x P GEMM, K = Q] folded into the running state in registers; writes the state before every
//                       chunk (in the operand dtype and order of the GEMM below), the final state in fp32, and what a
//                       sequence shard hands to the other ranks
//   ssd_fold_shards_kernel / ssd_fold_init_kernel   (sequence shards only) fold the other ranks' summaries into this
//                       shard's incoming state, and add that late-arriving state to the per-chunk states by linearity
//   ssd_scan_kernel     per (batch, chunk, 128-row block, part of a head group):  G = C B^T once (TMEM -> registers), then per
//                       head the decay mask exp2(c_i - c_j) delta_j [j <= i] (+ D on the diagonal) written back to TMEM
//                       (tcgen05.st) as the A operand of Y_intra = (G o L) X, plus  Y_inter = C S_in;
//                       y = Y_intra + exp2(c_i) Y_inter, gated, stored by TMA.  Sixteen warps form masks and epilogues; an
//                       elected lane of the warp with the least mask work issues the MMAs, one thread the copies.
//
// Exponent differences are always formed before exp2 (never exp2(c_i) / exp2(c_j)), so long
// sequences stay finite.  Every wait on an mbarrier is bounded and reports through the status word.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "tc05.cuh"

namespace ssmb {

constexpr int kQ = 256;    // chunk length
constexpr int kP = 64;     // head dimension
constexpr int kN = 128;    // state dimension
constexpr int kBlk = 128;  // rows per scan CTA

// floats of the shard summary (final state, then total log-decay), rounded up to whole 256-byte lines
__host__ __device__ inline int64_t ssd_summary_floats_padded(int batch, int heads) {
  return ((int64_t)batch * heads * (kP * kN + 1) + 63) / 64 * 64;
}

// ---------------------------------------------------------------------------------------------
// delta and within-chunk cumulative log-decay.  One CTA per (batch, chunk, 32 heads): the step sizes are read the way they
// lie in memory (heads innermost: each thread the 32 heads of one step), activated, transposed through shared memory, and
// each warp then scans whole heads, a lane owning 8 consecutive steps and writing them as 16-byte pieces.
// ---------------------------------------------------------------------------------------------
constexpr int kCumHeads = 32;
constexpr int kCumLd = kQ + 8;  // row pitch of the transposed tile (floats): rows stay 16-byte aligned, lanes 32 bytes apart

template <typename T>
__global__ void __launch_bounds__(kQ) ssd_cumsum_kernel(const ssm_ssd_args a, int nchunks) {
  __shared__ __align__(16) float sD[kCumHeads * kCumLd];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h0 = blockIdx.x * kCumHeads, c = blockIdx.y, b = blockIdx.z;
  const int nh = min(kCumHeads, a.heads - h0);
  {
    const int t = c * kQ + tid;
    if (t < a.len) {
      const int64_t at = ((int64_t)b * a.len + t) * a.heads + h0;
      if (a.dt_mode & 1) {  // fp32 step sizes, already activated
        const float* p = reinterpret_cast<const float*>(a.dt) + at;
        for (int hh = 0; hh < nh; ++hh) sD[hh * kCumLd + tid] = __ldg(p + hh);
      } else {
        const T* p = reinterpret_cast<const T*>(a.dt) + at;
        if (nh == kCumHeads && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
#pragma unroll
          for (int q = 0; q < kCumHeads / 8; ++q) {
            Vec16<T> v;
            v.load(p + q * 8);
            float f[8];
            v.unpack(f);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              float x = f[e] + (a.dt_bias ? __ldg(a.dt_bias + h0 + q * 8 + e) : 0.f);
              if (a.dt_softplus) x = softplus_f(x);
              sD[(q * 8 + e) * kCumLd + tid] = x;
            }
          }
        } else {
          for (int hh = 0; hh < nh; ++hh) {
            float x = to_f<T>(p[hh]) + (a.dt_bias ? __ldg(a.dt_bias + h0 + hh) : 0.f);
            if (a.dt_softplus) x = softplus_f(x);
            sD[hh * kCumLd + tid] = x;
          }
        }
      }
    } else {
      for (int hh = 0; hh < nh; ++hh) sD[hh * kCumLd + tid] = 0.f;  // steps beyond the sequence: no decay, no input
    }
  }
  __syncthreads();
  for (int hh = warp; hh < nh; hh += kQ / 32) {
    const int h = h0 + hh;
    const float Ah = __ldg(a.A + h);
    float* odt = a.ws_dt + (((int64_t)b * a.heads + h) * nchunks + c) * kQ + lane * 8;
    float* ocum = a.ws_cum + (((int64_t)b * a.heads + h) * nchunks + c) * kQ + lane * 8;
    float d[8], run = 0.f;  // each lane owns 8 consecutive steps
    {
      const float4 d0 = *reinterpret_cast<const float4*>(sD + hh * kCumLd + lane * 8);
      const float4 d1 = *reinterpret_cast<const float4*>(sD + hh * kCumLd + lane * 8 + 4);
      d[0] = d0.x, d[1] = d0.y, d[2] = d0.z, d[3] = d0.w, d[4] = d1.x, d[5] = d1.y, d[6] = d1.z, d[7] = d1.w;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) run += d[k] * Ah;
    // exclusive prefix of the lane sums
    float pre = run;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const float o = __shfl_up_sync(0xffffffffu, pre, off);
      if (lane >= off) pre += o;
    }
    float acc = pre - run;
    float oc[8], od[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      acc += d[k] * Ah;
      const float c2 = acc * kLog2e;
      oc[k] = c2;                      // running decay exponent, base 2
      // the same with delta folded in: exp2(x - odt[j]) = exp2(x - c2_j) * delta_j  (delta 0 -> +inf -> weight 0);
      // dt_mode & 2: the inputs enter with unit weight, only the decay uses delta
      od[k] = (a.dt_mode & 2) ? c2 : c2 - lg2_approx(d[k]);
    }
    reinterpret_cast<float4*>(ocum)[0] = make_float4(oc[0], oc[1], oc[2], oc[3]);
    reinterpret_cast<float4*>(ocum)[1] = make_float4(oc[4], oc[5], oc[6], oc[7]);
    reinterpret_cast<float4*>(odt)[0] = make_float4(od[0], od[1], od[2], od[3]);
    reinterpret_cast<float4*>(odt)[1] = make_float4(od[4], od[5], od[6], od[7]);
  }
}

// ---------------------------------------------------------------------------------------------
// chunk states, local and carried, in one pass:  one CTA per (batch, a few heads) walks the chunks in order.
// Per chunk the tensor cores form  S_c[n][p] = sum_j B[j][n] * (w_j x[j][p]),  w_j = exp2(c_last - (c_j - log2 delta_j)),
// in four stages of 64 steps from a ring of TMA-filled buffers:
//   A operand = B^T, MN-major;  B operand = w x of the CTA's heads side by side, MN-major;  M = 128 (n), N = 64 per head (p),
//   K = 64 per stage.  (Units that are neighbours along M / N are 128 bytes apart, so the tensor core's reads of one K slice
//   fall on different banks; with units 2 KB apart the MMAs ran 4-5x slower.)
// Eight compute warps scale the x rows of a landed stage in place and keep the running state in registers (thread = state n,
// 32 of the 64 columns p):  state <- exp2(c_last) * state + S_c ;  the state BEFORE each chunk goes out in the operand dtype,
// in the operand order of the scan kernel (MN-major units [p/8][n][8]).  The per-chunk local states never touch global memory.
// A ninth warp issues the copies (a buffer is refilled once the MMAs that read it have completed: tcgen05.commit -> mbarrier),
// a tenth the MMAs (once the eight compute warps have arrived on the stage's barrier).
// ---------------------------------------------------------------------------------------------
// HPC heads of one B / C group per CTA share the B^T tile of every stage (the grid is sized to about one CTA per SM).
// Tiles are rows of 128 bytes (64 elements along M / N) written by TMA with the 128-byte swizzle, 64 steps each:
// B^T as two blocks (states 0..63, 64..127), then one x block per head; blocks are 8 KB apart.
template <int HPC>
struct StateSmem {
  static constexpr int kStep = 64;                            // steps per stage
  static constexpr int BLK_BYTES = kStep * 128;               // 8 KB: 64 steps x 64 elements
  static constexpr int A_BYTES = 2 * BLK_BYTES;               // 16 KB
  static constexpr int STAGE = A_BYTES + HPC * BLK_BYTES;
  // one head per CTA: four stages (100 KB), so that two CTAs share an SM when there are more heads than SMs
  static constexpr int NSTAGE = HPC == 1 ? 4 : (HPC == 2 ? 6 : (HPC == 3 ? 5 : 4));
  static constexpr int VEC_BYTES = HPC * kQ * 4;              // c - log2(delta) of a chunk, per head
  // The copies run up to NSTAGE stages ahead of the MMAs, so a chunk's vectors may arrive while the chunk before last is still
  // being scaled: three buffers (NSTAGE <= 6 stages = one and a half chunks).
  static constexpr int NVEC = 3;
  static constexpr int LAST_BYTES = HPC * 16;                 // the last four running exponents of a chunk, per head
  static constexpr int TOTAL = NSTAGE * STAGE + NVEC * (VEC_BYTES + LAST_BYTES);
  static constexpr int ALLOC = TOTAL + 1024;
};

// tensor maps of the state kernel: B rows (box 64 states x 64 steps) and x rows (box 64 p x 64 steps)
struct StateMaps {
  CUtensorMap b, x;
};

// Threads: eight warps scale the x rows and keep the running states; one warp issues the copies, one the MMAs.  The stages pass
// from role to role through mbarriers only (landed -> scaled -> multiplied -> free), so no warp waits for another role's
// instruction issue.
constexpr int kStateComputeThreads = 256;
constexpr int kStateThreads = kStateComputeThreads + 64;
constexpr int kStateCopyWarp = 8, kStateMmaWarp = 9;

template <typename T, int HPC>
__global__ void __launch_bounds__(kStateThreads, HPC == 1 ? 2 : 1) ssd_state_kernel(const ssm_ssd_args a, const __grid_constant__ StateMaps maps, int nchunks) {
  using M = StateSmem<HPC>;
  constexpr int kStep = M::kStep, NS = M::NSTAGE;
  constexpr int SPC = kQ / kStep;  // stages per chunk
  extern __shared__ unsigned char smdyn[];
  unsigned char* smraw = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smdyn) + 1023) & ~(uintptr_t)1023);
  float* sVec = reinterpret_cast<float*>(smraw + NS * M::STAGE);  // [NVEC][HPC][kQ]
  float* sLast = sVec + M::NVEC * HPC * kQ;                       // [NVEC][HPC][4]: c at the chunk's last four steps
  __shared__ __align__(8) uint64_t mbar_full[NS];   // a stage's copies have landed
  __shared__ __align__(8) uint64_t mbar_scaled[NS]; // every compute warp has scaled its part of a stage's x rows
  __shared__ __align__(8) uint64_t mbar_free[NS];   // the MMAs that read a stage's buffer have completed
  __shared__ __align__(8) uint64_t mbar_acc[2];     // a chunk's accumulators are complete
  __shared__ uint32_t tmem_slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wg = tid >> 7;
  const int h0 = blockIdx.x * HPC, b = blockIdx.y;
  const int g = h0 / (a.heads / a.groups);
  const int n = (warp & 3) * 32 + lane;  // this thread's state index = TMEM lane
  constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  constexpr uint32_t kCols = HPC <= 1 ? 128 : (HPC == 2 ? 256 : 512);  // 2 accumulators of 64 columns per head, a power of two

  if (warp == 0) tc::tmem_alloc(tc::smem_u32(&tmem_slot), kCols);
  if (tid == 0) {
    for (int i = 0; i < NS; ++i) {
      tc::mbar_init(tc::smem_u32(&mbar_full[i]), 1);
      tc::mbar_init(tc::smem_u32(&mbar_scaled[i]), kStateComputeThreads / 32);
      tc::mbar_init(tc::smem_u32(&mbar_free[i]), 1);
    }
    tc::mbar_init(tc::smem_u32(&mbar_acc[0]), 1);
    tc::mbar_init(tc::smem_u32(&mbar_acc[1]), 1);
  }
  __syncthreads();  // TMEM address and barriers are set up
  const uint32_t tmem = __shfl_sync(0xffffffffu, tmem_slot, 0);
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  const int role = __shfl_sync(0xffffffffu, warp, 0);  // the same in every lane, and visibly so

  const int64_t vrow0 = ((int64_t)b * a.heads + h0) * nchunks * kQ;  // exponent vectors of head h0 (next head: + nchunks * kQ)
  const int nst = SPC * nchunks;
  // stage s = steps [s * 64, s * 64 + 64), issued by one thread: two boxes of B, one box of x per head, and with a
  // chunk's first stage the exponent vectors of its heads.  Steps beyond the sequence read as zero.
  auto copy_stage = [&](int s) {
    const uint32_t base = tc::smem_u32(smraw + (s % NS) * M::STAGE);
    const uint32_t full = tc::smem_u32(&mbar_full[s % NS]);
    const bool first = s % SPC == 0;
    tc::mbar_expect_tx(full, M::STAGE + (first ? HPC * kQ * 4 + M::LAST_BYTES : 0));
    tc::tma_load_4d(base, &maps.b, full, 0, g, s * kStep, b);
    tc::tma_load_4d(base + M::BLK_BYTES, &maps.b, full, 64, g, s * kStep, b);
#pragma unroll
    for (int hh = 0; hh < HPC; ++hh)
      tc::tma_load_4d(base + M::A_BYTES + hh * M::BLK_BYTES, &maps.x, full, 0, a.x_heads ? (h0 + hh) % a.x_heads : h0 + hh, s * kStep, b);
    if (first) {
      const int c = s / SPC;
#pragma unroll
      for (int hh = 0; hh < HPC; ++hh) {
        tc::bulk_load(tc::smem_u32(sVec + ((c % M::NVEC) * HPC + hh) * kQ), a.ws_dt + vrow0 + ((int64_t)hh * nchunks + c) * kQ, kQ * 4, full);
        tc::bulk_load(tc::smem_u32(sLast + ((c % M::NVEC) * HPC + hh) * 4), a.ws_cum + vrow0 + ((int64_t)hh * nchunks + c) * kQ + kQ - 4, 16, full);
      }
    }
  };
  int fail = 0;
  if (role == kStateCopyWarp) {
    // ---- copies: a buffer is refilled once the MMAs of the stage that used it before have completed ------------
#pragma unroll 1
    for (int s = 0; s < nst; ++s) {
      bool okf = true;
      if (s >= NS) okf = __all_sync(0xffffffffu, tc::mbar_wait(tc::smem_u32(&mbar_free[s % NS]), ((s - NS) / NS) & 1));
      if (!okf) {  // the stage never lands and the waits of the other warps report it too
        fail = 1;
        break;
      }
      if (tc::elect_one()) copy_stage(s);
      __syncwarp();
    }
  } else if (role == kStateMmaWarp) {
    // ---- MMAs: S_c (+)= B^T (w x) over the 64 steps of a stage, as soon as the eight compute warps have scaled it ----
#pragma unroll 1
    for (int s = 0; s < nst; ++s) {
      const int c = s / SPC, part = s % SPC;
      const bool okm = __all_sync(0xffffffffu, tc::mbar_wait(tc::smem_u32(&mbar_scaled[s % NS]), (s / NS) & 1));
      if (!okm) {
        fail = 1;
        break;
      }
      tc::fence_after_sync();
      if (tc::elect_one()) {
        // M = 128 states = two 64-element blocks, N = 64 HPC = one block per head; blocks 8 KB apart, 8 steps 1 KB apart
        unsigned char* base = smraw + (s % NS) * M::STAGE;
        constexpr uint32_t idesc = tc::instr_desc(kN, HPC * kP, fmt, 1, 1);
        const uint64_t da0 = tc::smem_desc_sw128(tc::smem_u32(base), M::BLK_BYTES, 1024);
        const uint64_t db0 = tc::smem_desc_sw128(tc::smem_u32(base + M::A_BYTES), M::BLK_BYTES, 1024);
#pragma unroll
        for (int kk = 0; kk < kStep / 16; ++kk)  // 16 steps = 16 rows of 128 bytes
          tc::mma_ss(tmem + (c & 1) * HPC * 64, da0 + (uint64_t)(kk * (2048 >> 4)), db0 + (uint64_t)(kk * (2048 >> 4)), idesc, part > 0 || kk > 0);
        tc::commit(tc::smem_u32(&mbar_free[s % NS]));
        if (part == SPC - 1) tc::commit(tc::smem_u32(&mbar_acc[c & 1]));
      }
      __syncwarp();
    }
  } else {
  // ======== compute warps ========================================================================================
  // running states: st[hh][i] = S_{h0 + hh}[n][wg * 32 + i]
  float st[HPC][32];
#pragma unroll
  for (int hh = 0; hh < HPC; ++hh) {
    const float* init = a.initial_states ? a.initial_states + (((int64_t)b * a.heads + h0 + hh) * kP + wg * 32) * kN + n : nullptr;
#pragma unroll
    for (int i = 0; i < 32; ++i) st[hh][i] = init ? __ldg(init + (int64_t)i * kN) : 0.f;
  }
  T* sin = reinterpret_cast<T*>(a.ws_state_in);
  // the states before chunk c, in the operand dtype: unit (p / 8, n) of the (batch, chunk, head) tile
  auto emit_state_in = [&](int c) {
#pragma unroll
    for (int hh = 0; hh < HPC; ++hh) {
      T* blk = sin + (((int64_t)b * nchunks + c) * a.heads + h0 + hh) * (int64_t)(kP * kN);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        Vec16<T> o;
        o.pack(*reinterpret_cast<const float(*)[8]>(&st[hh][q * 8]));
        *reinterpret_cast<uint4*>(blk + ((size_t)(wg * 4 + q) * kN + n) * 8) = o.raw;
      }
      if (a.ws_state_in_f32) {  // the same tile unrounded (the backward pass forms <adjoint state, state> from it)
        float* blk32 = a.ws_state_in_f32 + (((int64_t)b * nchunks + c) * a.heads + h0 + hh) * (int64_t)(kP * kN);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float4* dst = reinterpret_cast<float4*>(blk32 + ((size_t)(wg * 4 + q) * kN + n) * 8);
          dst[0] = make_float4(st[hh][q * 8], st[hh][q * 8 + 1], st[hh][q * 8 + 2], st[hh][q * 8 + 3]);
          dst[1] = make_float4(st[hh][q * 8 + 4], st[hh][q * 8 + 5], st[hh][q * 8 + 6], st[hh][q * 8 + 7]);
        }
      }
    }
  };
  // last exponent of the current / previous chunk per head (the decay across the chunk is exp2 of it)
  float clast[HPC], clast_prev[HPC], ctot[HPC];
#pragma unroll
  for (int hh = 0; hh < HPC; ++hh) clast[hh] = 0.f, clast_prev[hh] = 0.f, ctot[hh] = 0.f;
  // fold chunk c's finished accumulators into the running states
  auto fold_chunk = [&](int c, const float (&cl)[HPC]) -> bool {
    const bool ok = __all_sync(0xffffffffu, tc::mbar_wait(tc::smem_u32(&mbar_acc[c & 1]), (c >> 1) & 1));
    tc::fence_after_sync();
    if (ok) {
#pragma unroll
      for (int hh = 0; hh < HPC; ++hh) {
        const float decay = ex2_approx(cl[hh]);
        float v[32];
        tc::tmem_ld32(tmem + lane_base + ((c & 1) * HPC + hh) * 64 + wg * 32, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) st[hh][i] = fmaf(decay, st[hh][i], v[i]);
      }
    }
    return ok;
  };

#pragma unroll 1
  for (int s = 0; s < nst; ++s) {
    const int c = s / SPC, part = s % SPC;
    if (part == 0 && c == 0) emit_state_in(0);
    // ---- one stage into a chunk its predecessor's MMAs have surely finished: fold them, hand out the states
    // ---- before this chunk (its accumulators are the other pair, so the stage already issued is not disturbed)
    if (part == 1 && c >= 1) {
      if (!fail) fail = !fold_chunk(c - 1, clast_prev);
      emit_state_in(c);
    }
    if (!fail) fail = !__all_sync(0xffffffffu, tc::mbar_wait(tc::smem_u32(&mbar_full[s % NS]), (s / NS) & 1));  // this stage's copies
    if (part == 0) {  // a new chunk begins: its last exponent arrived with the stage
#pragma unroll
      for (int hh = 0; hh < HPC; ++hh) {
        clast_prev[hh] = clast[hh];
        clast[hh] = sLast[((c % M::NVEC) * HPC + hh) * 4 + 3];
        // exponent (base 2) of the decay from the start of the sequence to the start of this chunk: what a state
        // that arrives later (phase 2 of a sequence shard) is multiplied by before it joins this chunk's state
        if (tid == 0) a.ws_state[ssd_summary_floats_padded(a.batch, a.heads) + ((int64_t)b * a.heads + h0 + hh) * nchunks + c] = ctot[hh];
        ctot[hh] += clast[hh];
      }
    }

    // ---- scale the x rows in place: w_j x_j (a row is one step, whatever the swizzle does inside it) ------------
    unsigned char* base = smraw + (s % NS) * M::STAGE;
#pragma unroll
    for (int hh = 0; hh < HPC; ++hh) {
      const float* vcp = sVec + ((c % M::NVEC) * HPC + hh) * kQ + part * kStep;
      const float c_last = clast[hh];
#pragma unroll
      for (int k = 0; k < M::BLK_BYTES / 16 / 256; ++k) {
        const int u = tid + 256 * k;  // 16-byte unit of this head's tile; 8 units per step
        const float w = ex2_approx(c_last - vcp[u >> 3]);
        unsigned char* px = base + M::A_BYTES + hh * M::BLK_BYTES + (size_t)u * 16;
        Vec16<T> v;
        v.raw = *reinterpret_cast<const uint4*>(px);
        float f[8];
        v.unpack(f);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] *= w;
        v.pack(f);
        *reinterpret_cast<uint4*>(px) = v.raw;
      }
    }
    // the scaled rows become visible to the tensor cores' reads; the accumulator reads of an earlier fold precede the MMAs
    // that will overwrite that pair.  A warp whose wait ran out still arrives, so that the others do not wait for it.
    tc::fence_async_smem();
    tc::fence_before_sync();
    __syncwarp();
    if (lane == 0) tc::mbar_arrive(tc::smem_u32(&mbar_scaled[s % NS]));
  }
  if (nchunks > 0 && !fail) fail = !fold_chunk(nchunks - 1, clast);
  // final states in fp32, (p, n) order: to the caller, and kept in scratch for a later phase 2
  if (!fail) {
#pragma unroll
    for (int hh = 0; hh < HPC; ++hh) {
      const int64_t off = (((int64_t)b * a.heads + h0 + hh) * kP + wg * 32) * kN + n;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (a.final_states) a.final_states[off + (int64_t)i * kN] = st[hh][i];
        a.ws_state[off + (int64_t)i * kN] = st[hh][i];
      }
      // the shard's total log-decay (natural log) follows the states in the scratch: together they are what a
      // sequence shard sends to the other ranks
      if (tid == 0) a.ws_state[(int64_t)a.batch * a.heads * kP * kN + (int64_t)b * a.heads + h0 + hh] = ctot[hh] * kLn2;
    }
  }
  }  // compute warps
  if (fail && lane == 0 && a.status) atomicExch(a.status, 1);
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, kCols);
}

// ---------------------------------------------------------------------------------------------
// phase 2 of a sequence shard: the shard's incoming state S0 arrives after the chunk states were
// formed from a zero state.  By linearity  state_before_chunk_c += exp2(sum_{c' < c} c_last[c']) * S0
// and  final += exp2(sum_c c_last[c]) * S0.  One thread per element, operand order of the scan kernel.
// ---------------------------------------------------------------------------------------------
constexpr int kFoldChunks = 8;  // chunks per thread: the eight values of S0 are read once for them, their loads go out together
template <typename T>
__global__ void __launch_bounds__(256) ssd_fold_init_kernel(const ssm_ssd_args a, int nchunks) {
  // thread = one 16-byte unit (p / 8, n) of the states before kFoldChunks chunks; blockIdx.y = group of chunks (the row after
  // the last chunk: final states)
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;  // unit of one (batch, head): 1024 units each
  const int64_t units = (int64_t)a.batch * a.heads * (kP * kN / 8);
  if (i >= units) return;
  const int64_t bh = i / (kP * kN / 8);
  const int u = (int)(i % (kP * kN / 8));
  const int n = u % kN, pc = u / kN;
  const int b = (int)(bh / a.heads), h = (int)(bh % a.heads);
  const int c0 = blockIdx.y * kFoldChunks;
  const float* s0p = a.initial_states + bh * (int64_t)(kP * kN) + (int64_t)(pc * 8) * kN + n;  // 8 values p = 8 pc .. 8 pc + 7 of state n
  const float* pre = a.ws_state + ssd_summary_floats_padded(a.batch, a.heads);
  float s0[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) s0[e] = __ldg(s0p + (int64_t)e * kN);
  T* blk0 = reinterpret_cast<T*>(a.ws_state_in) + (((int64_t)b * nchunks) * a.heads + h) * (int64_t)(kP * kN) + (int64_t)u * 8;
  const int64_t cstride = (int64_t)a.heads * (kP * kN);
  uint4 raw[kFoldChunks];
  float wl[kFoldChunks];
#pragma unroll
  for (int k = 0; k < kFoldChunks; ++k) {
    const int c = min(c0 + k, nchunks - 1);  // beyond the last chunk: a valid address, dropped below
    raw[k] = *reinterpret_cast<const uint4*>(blk0 + c * cstride);
    wl[k] = __ldg(pre + bh * nchunks + c);
  }
#pragma unroll
  for (int k = 0; k < kFoldChunks; ++k) {
    const int c = c0 + k;
    if (c < nchunks) {
      const float w = ex2_approx(wl[k]);
      Vec16<T> v;
      v.raw = raw[k];
      float f[8];
      v.unpack(f);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = fmaf(w, s0[e], f[e]);
      v.pack(f);
      *reinterpret_cast<uint4*>(blk0 + c * cstride) = v.raw;
    } else if (c == nchunks && a.final_states) {
      const float w = __expf(__ldg(a.ws_state + (int64_t)a.batch * a.heads * kP * kN + bh));  // total log-decay of the call
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int64_t off = bh * (int64_t)(kP * kN) + (int64_t)(pc * 8 + e) * kN + n;
        a.final_states[off] = fmaf(w, s0[e], a.ws_state[off]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// chunk scan: one CTA (256 threads) per (batch, chunk, 128-row block m, part of the heads of one
// B / C group).  Heads of a group share B and C, so  G = C_m B^T  (128 x 128 (m+1), causal: only
// steps before the block's last row) is formed ONCE per CTA; every thread then keeps its part of
// G (one row, half of the steps) in registers while the CTA walks its heads:
//   per head:  G times the head's decay mask exp2(c_i - c_j) delta_j [j <= i], packed as the A
//              operand (overwrites the dead B tile);  Y_intra = (G o L) X  and  Y_inter = C_m S_in
//              accumulate in TMEM while the previous head's result is read back, gated and staged.
//   Copies (cp.async, whole 128 / 256-byte rows per group of lanes) run one head ahead into the
//   other half of a double buffer: x, the incoming state, the exponent vectors; z goes through
//   the same 16 KB staging tile that carries y back out, so that every global access of the
//   head loop touches whole 128-byte lines.
//   TMEM columns: G [0,256); per buffer b: Y_intra [256+128b, +64), Y_inter [320+128b, +64).
// ---------------------------------------------------------------------------------------------
template <typename T>
struct ScanSmem {
  static constexpr int C_BYTES = kBlk * kN * 2;     // C rows of the block: two blocks (states 0..63, 64..127) of [i][128 B], swizzled   32 KB
  static constexpr int B_BYTES = kQ * kN * 2;       // B rows likewise, [j][128 B] per block; later the masked tile, K-major [j/8][i][8]  64 KB
  static constexpr int X_BYTES = kQ * kP * 2;       // x rows [j][64 p], 128-byte rows, TMA 128-byte swizzle  32 KB (x2)
  static constexpr int S_BYTES = kP * kN * 2;       // incoming state, MN-major [p/8][n][8]                 16 KB (x2)
  static constexpr int VEC_BYTES = 2 * kQ * 4;      // c and c - log2(delta) of the chunk                     2 KB (x2)
  static constexpr int Z_BYTES = kBlk * kP * 2;     // z in / y out of one head: [row][64 p], same swizzle    16 KB
  static constexpr int W_BYTES = 1024 * 4;          // per warp: the column factors of its mask chunks (16 warps x 64)          4 KB
  static constexpr int TOTAL = C_BYTES + B_BYTES + 2 * (X_BYTES + S_BYTES + VEC_BYTES) + Z_BYTES + W_BYTES;
  static constexpr int ALLOC = TOTAL + 1024;        // the tiles TMA swizzles must start on 1024-byte boundaries
};

constexpr int kScanThreads = 512;
constexpr int kScanWG = kScanThreads / 128;  // warpgroups: each owns every kScanWG-th 32-step column chunk of the mask and kP / kScanWG output columns
constexpr int kEC = kP / kScanWG;             // epilogue columns per thread
constexpr int kEU = kEC / 8;                  // ... in 16-byte units
// Thread that issues the bulk copies (TMA): lane 0 of the warp with the least mask work (rows 0..31 of the block, odd
// chunks), so that its issue time hides behind the other warps' mask stage; thread 0 issues the MMAs.
constexpr int kCopyThread = 128;
// Issues the per-head MMAs: lane 0 of the warp with the least mask work (rows 0..31 of the block, last column slice).
constexpr int kMmaWarp = 12;

// tensor maps of one call: x (box of 128 or 256 steps), z and y (boxes of 128 rows); rank 4 (p, head, step, batch)
struct ScanMaps {
  CUtensorMap x0, x1, z, y;
  CUtensorMap c, bm;  // C and B rows: rank 4 (state, group, step, batch), boxes of 64 states x 128 steps
};

// Body for row block MB (0: rows 0..127, steps 0..127; 1: rows 128..255, steps 0..255).  XSKIP: the skip term D x is added
// in the epilogue (a weight per channel, or the row sums of the backward pass are wanted), which carries each thread's x row
// from one iteration to the next; without it a weight per head rides on the diagonal of the masked operand.
template <typename T, int MB, bool XSKIP>
__device__ __forceinline__ void ssd_scan_body(const ssm_ssd_args& a, const ScanMaps& maps, int nchunks, int hpc, int nparts, unsigned char* smraw,
                                              uint64_t* mbar, uint32_t* tmem_slot) {
  using M = ScanSmem<T>;
  constexpr int KJ = (MB + 1) * kBlk;  // steps that can reach this block's rows
  constexpr int NCH = KJ / (32 * kScanWG);  // 32-step column chunks per thread (the warpgroups interleave chunks)
  unsigned char* sC = smraw;
  unsigned char* sBA = sC + M::C_BYTES;
  unsigned char* sX = sBA + M::B_BYTES;        // two buffers
  unsigned char* sS = sX + 2 * M::X_BYTES;     // two buffers
  float* sVec = reinterpret_cast<float*>(sS + 2 * M::S_BYTES);  // two buffers of [c | c - log2 delta]
  unsigned char* sZ = reinterpret_cast<unsigned char*>(sVec) + 2 * M::VEC_BYTES;
  // mbar: 0 G done; 1 + b MMAs of a head into accumulator pair b done; 3 + b operands of buffer b landed; 5, 7 gate tiles landed;
  // 6 C and B tiles landed
  const uint32_t mb_g = tc::smem_u32(&mbar[0]);
  auto mb_z = [&](int bf) { return tc::smem_u32(&mbar[bf ? 7 : 5]); };  // gate tile of buffer bf landed
  auto mb_mma = [&](int bf) { return tc::smem_u32(&mbar[1 + bf]); };
  auto mb_full = [&](int bf) { return tc::smem_u32(&mbar[3 + bf]); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wg = tid >> 7;                     // column chunks wg, wg + kScanWG, ... in the mask stage; column slice in the epilogue
  float* sW = reinterpret_cast<float*>(sZ + M::Z_BYTES) + warp * (NCH * 32);  // this warp's column factors
  // The gate rows of a head get buffers of their own, over the B tile (dead once G is formed: the masked operand lives in
  // tensor memory): head h's tile is requested at the top of its own iteration and read by its epilogue one iteration later,
  // instead of waiting, in the shared staging tile, for the previous head's y to be stored first.
  auto sZin = [&](int bf) { return sBA + bf * M::Z_BYTES; };
  const int half_grid = gridDim.x >> 1;
  const int rem = (int)blockIdx.x % half_grid;
  const int part = rem % nparts, bc = rem / nparts;
  const int c = bc % nchunks, b = bc / nchunks;
  const int h0 = part * hpc;
  const int nh = min(hpc, a.heads - h0);
  const int g = h0 / (a.heads / a.groups);
  const int t0 = c * kQ;
  const int i_loc = (warp & 3) * 32 + lane;    // row within the block = TMEM lane
  const int i_chunk = MB * kBlk + i_loc;       // row within the chunk
  const int rc = MB * 4 + (warp & 3);          // this warp's rows as a 32-step chunk index
  constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  const bool has_z = a.z != nullptr;
  const CUtensorMap* mapx = MB ? &maps.x1 : &maps.x0;

  // ---- C rows of the block, B rows of the reachable steps, by TMA: per half of the states one block of 128-byte rows
  const uint32_t mb_cb = tc::smem_u32(&mbar[6]);
  if (tid == kCopyThread) {
    tc::mbar_expect_tx(mb_cb, M::C_BYTES + KJ * kN * 2);
#pragma unroll
    for (int nb2 = 0; nb2 < 2; ++nb2) {
      tc::tma_load_4d(tc::smem_u32(sC + nb2 * (kBlk * 128)), &maps.c, mb_cb, nb2 * 64, g, t0 + MB * kBlk, b);
#pragma unroll
      for (int jb2 = 0; jb2 <= MB; ++jb2)
        tc::tma_load_4d(tc::smem_u32(sBA + nb2 * (KJ * 128) + jb2 * (kBlk * 128)), &maps.bm, mb_cb, nb2 * 64, g, t0 + jb2 * kBlk, b);
    }
  }

  // One head's operands, by bulk copies issued from one thread: x rows through the tensor map (128-byte rows, swizzled),
  // the incoming state and the two exponent vectors as contiguous pieces.  Steps beyond the sequence read as zero.
  constexpr uint32_t kOperandBytes = KJ * kP * 2 + M::S_BYTES + 2 * KJ * 4;
  auto prefetch = [&](int h, int buf) {
    const uint32_t full = mb_full(buf);
    tc::mbar_expect_tx(full, kOperandBytes);
    tc::tma_load_4d(tc::smem_u32(sX + buf * M::X_BYTES), mapx, full, 0, a.x_heads ? h % a.x_heads : h, t0, b);
    const T* ss = reinterpret_cast<const T*>(a.ws_state_in) + (((int64_t)b * nchunks + c) * a.heads + h) * (int64_t)(kP * kN);
    tc::bulk_load(tc::smem_u32(sS + buf * M::S_BYTES), ss, M::S_BYTES, full);
    const int64_t voff = (((int64_t)b * a.heads + h) * nchunks + c) * kQ;
    float* dV = sVec + buf * (2 * kQ);
    tc::bulk_load(tc::smem_u32(dV), a.ws_cum + voff, KJ * 4, full);
    tc::bulk_load(tc::smem_u32(dV + kQ), a.ws_dt + voff, KJ * 4, full);
  };
  // slot of (row, 16-byte chunk) in a tile of 128-byte rows written / read by TMA with the 128-byte swizzle
  auto swz = [&](unsigned char* tile, int row, int chunk) { return tile + ((size_t)row * 8 + (chunk ^ (row & 7))) * 16; };

  if (tid == kCopyThread) prefetch(h0, 0);

  bool ok = __all_sync(0xffffffffu, tc::mbar_wait(mb_cb, 0));  // C and B have landed
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = __shfl_sync(0xffffffffu, *tmem_slot, 0);
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  const bool mma_warp = __shfl_sync(0xffffffffu, warp, 0) == kMmaWarp;  // the same in every lane, and visibly so

  // ---- G = C_m B^T ------------------------------------------------------------------------------------
  // K-major operands in 128-byte-swizzled rows: 16 states = 32 bytes further along the row, 64 states = the next block
  if (tid == 0 && ok) {
    const uint64_t dc0 = tc::smem_desc_sw128(tc::smem_u32(sC), 16, 1024);
    const uint64_t db0 = tc::smem_desc_sw128(tc::smem_u32(sBA), 16, 1024);
    constexpr uint32_t idG = tc::instr_desc(kBlk, KJ, fmt, 0, 0);
#pragma unroll
    for (int kk = 0; kk < kN / 16; ++kk)
      tc::mma_ss(tmem, dc0 + (uint64_t)(((kk >> 2) * (kBlk * 128) + (kk & 3) * 32) >> 4), db0 + (uint64_t)(((kk >> 2) * (KJ * 128) + (kk & 3) * 32) >> 4), idG,
                 kk > 0);
    tc::commit(mb_g);
  }
  ok = __all_sync(0xffffffffu, ok && tc::mbar_wait(mb_g, 0));  // warp-uniform
  tc::fence_after_sync();

  // This thread's part of G stays in registers for all heads: row i_loc, chunks wg, wg + kScanWG, ...
  float vG[NCH][32];
#pragma unroll
  for (int k = 0; k < NCH; ++k) {
    const int cc = wg + kScanWG * k;
    if (ok && cc <= rc) {
      tc::tmem_ld32(tmem + lane_base + cc * 32, vG[k]);
    } else {
#pragma unroll
      for (int e = 0; e < 32; ++e) vG[k][e] = 0.f;
    }
  }

  // A skip weight per head (not per channel) rides on the diagonal of the masked operand: (G o L + D I) X = Y_intra + D x.
  // The row sums for the backward pass want y without the skip term, so that mode keeps the explicit form.
  const bool fold_d = !XSKIP && a.D;
  const bool pair_reuse = (a.dt_mode & 4) && !a.D && !a.row_scale;  // nothing per head may ride on the mask
  constexpr bool skip_explicit = XSKIP;

  // epilogue of head h from accumulator pair `buf`: y = Y_intra + exp2(c_i) Y_inter (+ D x where it is not folded), gated by
  // the z row, staged for the bulk store.  Thread = row i_loc, this warpgroup's 16 columns; the arithmetic runs on pairs.
  constexpr int kXR = XSKIP ? kEU : 1;  // x row registers exist only where the explicit skip term needs them
  auto epilogue = [&](int h, int buf, float ct, const uint4 (&xr)[kXR]) {
    const float escale = ex2_approx(ct);
    const float2 es2 = make_float2(escale, escale);
    float yi[kEC], ys[kEC];
    tc::tmem_ld16(tmem + lane_base + 256 + buf * 128 + wg * kEC, yi);
    tc::tmem_ld16(tmem + lane_base + 320 + buf * 128 + wg * kEC, ys);
    const float Dh = (skip_explicit && !a.d_has_p) ? __ldg(a.D + h) : 0.f;
    const bool dots = a.row_dots != nullptr;
    float dot = 0.f;  // row_dots: this thread's 16 columns of  sum_p y[p] z[p]  (y before the skip term and unrounded)
#pragma unroll
    for (int q = 0; q < kEU; ++q) {
      float2 f2[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        f2[e] = __ffma2_rn(es2, make_float2(ys[q * 8 + 2 * e], ys[q * 8 + 2 * e + 1]), make_float2(yi[q * 8 + 2 * e], yi[q * 8 + 2 * e + 1]));
      float zv[8];
      if (has_z) {
        Vec16<T> zz;
        zz.raw = *reinterpret_cast<const uint4*>(swz(sZin(buf), i_loc, wg * kEU + q));
        zz.unpack(zv);
        if (dots) {
#pragma unroll
          for (int e = 0; e < 4; ++e) dot = fmaf(f2[e].x, zv[2 * e], dot), dot = fmaf(f2[e].y, zv[2 * e + 1], dot);
        }
      }
      if (skip_explicit) {
        float xv[8];
        Vec16<T> xx;
        xx.raw = xr[XSKIP ? q : 0];
        xx.unpack(xv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 d2 = a.d_has_p ? make_float2(__ldg(a.D + h * kP + wg * kEC + q * 8 + 2 * e), __ldg(a.D + h * kP + wg * kEC + q * 8 + 2 * e + 1))
                                      : make_float2(Dh, Dh);
          f2[e] = __ffma2_rn(d2, make_float2(xv[2 * e], xv[2 * e + 1]), f2[e]);
        }
      }
      if (has_z && !dots) {  // y silu(z), silu(z) = h + h tanh(h) with h = z / 2
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 h2 = __fmul2_rn(make_float2(zv[2 * e], zv[2 * e + 1]), make_float2(0.5f, 0.5f));
          float2 t2;
          asm("tanh.approx.f32 %0, %1;" : "=f"(t2.x) : "f"(h2.x));
          asm("tanh.approx.f32 %0, %1;" : "=f"(t2.y) : "f"(h2.y));
          f2[e] = __fmul2_rn(f2[e], __ffma2_rn(h2, t2, h2));
        }
      }
      float f[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) f[2 * e] = f2[e].x, f[2 * e + 1] = f2[e].y;
      Vec16<T> o;
      o.pack(f);
      *reinterpret_cast<uint4*>(swz(sZ, i_loc, wg * kEU + q)) = o.raw;
    }
    if (dots && has_z) {
      const int t = t0 + MB * kBlk + i_loc;
      // the threads of a row (column slices) add to one zero-initialised word: the sum does not depend on their order
      if (t < a.len) atomicAdd(a.row_dots + ((int64_t)b * a.len + t) * a.heads + h, dot);
    }
    tc::fence_async_smem();  // the staged rows leave through a bulk store
  };
  const int t_blk = t0 + MB * kBlk;  // first step of this block's rows

  float ct_prev = 0.f;   // the previous head's row exponent and x row, carried into its (deferred) epilogue
  uint4 xr_prev[kXR];
#pragma unroll
  for (int q = 0; q < kXR; ++q) xr_prev[q] = make_uint4(0, 0, 0, 0);
  int fail = 0;
#pragma unroll 1
  for (int hi = 0; hi < nh; ++hi) {
    const int h = h0 + hi, buf = hi & 1;
    ok = !fail && tc::mbar_wait(mb_full(buf), (hi >> 1) & 1);  // this head's operands (no more waiting once a wait ran out)
    // ---- factors of the decay mask, formed before the CTA-wide barrier below so that their latency (shared-memory reads, ex2,
    // the exchange of the column factors through sW) overlaps the wait for the slowest warp; the barrier also orders the
    // writes to sW before the reads of the other lanes
    const float* vc = sVec + buf * (2 * kQ);
    const float* vcp = vc + kQ;
    const float Dfold = fold_d ? __ldg(a.D + h) : 0.f;
    float ct = vc[i_chunk];
    if (a.row_scale) {
      // optional weight of this thread's row, folded into the row exponent: it scales the mask before rounding and the
      // carried-state term alike
      const int t_row = t0 + MB * kBlk + i_loc;
      ct += lg2_approx(t_row < a.len ? __ldg(a.row_scale + ((int64_t)b * a.len + t_row) * a.heads + h) : 1.f);
    }
    // The weight exp2(c_i - c'_j) of a 32-step chunk factors as exp2(c_i - r) * exp2(r - c'_j) with r = c at the
    // chunk's first step (row factor <= 1 for causal rows, column factor bounded by the decay inside the chunk).
    // Each lane forms one column factor per chunk, each thread one row factor per chunk: 2 ex2 per 32 elements
    // instead of 32.  Chunks whose internal decay exceeds 2^60 keep the exact per-element form.
    // dt_mode & 4: heads 2 i and 2 i + 1 have the same step sizes and decay, so the masked operand the even head left in
    // tensor memory serves the odd head as it is (its MMAs have completed and only read it)
    const bool reuse = pair_reuse && (h & 1) && hi > 0;
    float arow[NCH];
    bool fast[NCH];
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int cc = wg + kScanWG * k;
      arow[k] = 0.f, fast[k] = false;
      if (cc <= rc && !reuse) {
        const float r = vc[cc * 32];
        fast[k] = r - vc[cc * 32 + 31] < 60.f;  // same for every lane
        arow[k] = ex2_approx(ct - r);
        sW[k * 32 + lane] = ex2_approx(r - vcp[cc * 32 + lane]);
      }
    }
    // MMAs of the previous head: the masked tile, the other buffer and its accumulators are free / ready
    if (hi > 0) ok = tc::mbar_wait(mb_mma(buf ^ 1), ((hi - 1) >> 1) & 1) && ok;
    tc::fence_after_sync();
    tc::fence_before_sync();     // the accumulator reads of the previous epilogue precede the MMAs issued below
    ok = __syncthreads_and(ok);  // the staged y of the head before last is complete; the outcome of the waits is CTA-wide
    if (!ok) {
      fail = 1;
      break;
    }
    if (mma_warp && tc::elect_one()) {
      // Y_inter = C_m S_in needs nothing of the mask: issued first, it runs on the tensor cores while the mask is formed
      tc::fence_after_sync();
      const uint64_t dc0 = tc::smem_desc_sw128(tc::smem_u32(sC), 16, 1024);
      const uint64_t ds0 = tc::smem_desc(tc::smem_u32(sS + buf * M::S_BYTES), 128, kN * 16);
      constexpr uint32_t idS = tc::instr_desc(kBlk, kP, fmt, 0, 1);
      const uint32_t dS = tmem + 256 + buf * 128 + 64;
#pragma unroll
      for (int kk = 0; kk < kN / 16; ++kk)
        tc::mma_ss(dS, dc0 + (uint64_t)(((kk >> 2) * (kBlk * 128) + (kk & 3) * 32) >> 4), ds0 + (uint64_t)(kk * (256 >> 4)), idS, kk > 0);
    }
    if (tid == kCopyThread) {
      if (hi + 1 < nh) prefetch(h + 1, buf ^ 1);
      if (has_z) {  // its buffer was last read by the epilogue of head h - 2, one iteration ago
        tc::mbar_expect_tx(mb_z(buf), M::Z_BYTES);
        tc::tma_load_4d(tc::smem_u32(sZin(buf)), &maps.z, mb_z(buf), 0, h, t_blk, b);
      }
      if (hi >= 2) {  // staged by the epilogue of the previous iteration; its reads are awaited after the mask, below
        tc::tma_store_4d(&maps.y, tc::smem_u32(sZ), 0, h - 2, t_blk, b);
        tc::bulk_commit();
      }
      if (hi + 2 < nh) {  // the tiles of the head after next on their way into the L2: one iteration alone does not cover the latency
        tc::tma_prefetch_4d(mapx, 0, a.x_heads ? (h + 2) % a.x_heads : h + 2, t0, b);
        if (has_z) tc::tma_prefetch_4d(&maps.z, 0, h + 2, t_blk, b);
        tc::bulk_prefetch(reinterpret_cast<const T*>(a.ws_state_in) + (((int64_t)b * nchunks + c) * a.heads + h + 2) * (int64_t)(kP * kN), M::S_BYTES);
      }
    }

    // ---- decay mask: G (registers) x the factors formed above -> the A operand in tensor memory
    if (!reuse) {
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int cc = wg + kScanWG * k;  // chunk of 32 steps: fully causal (cc < rc), diagonal (cc == rc) or empty (cc > rc) for this warp's rows
      const int jb = cc * 32;
      // the masked row goes to tensor memory as the A operand: 32 steps = 16 columns of two 16-bit values
      const uint32_t dst = tmem + lane_base + cc * 16;
      uint32_t packed[16];
      if (cc > rc) {
#pragma unroll
        for (int q = 0; q < 16; ++q) packed[q] = 0u;
        tc::tmem_st16(dst, packed);
        continue;
      }
      const bool diag = cc == rc;
      if (fast[k] && !diag) {  // the common case: every step of the chunk precedes every row of this warp, nothing to cut
        const float2 a2 = make_float2(arow[k], arow[k]);
#pragma unroll
        for (int q = 0; q < 32; q += 8) {
          const float4 b0 = *reinterpret_cast<const float4*>(sW + k * 32 + q);
          const float4 b1 = *reinterpret_cast<const float4*>(sW + k * 32 + q + 4);
          const float2 bp[4] = {make_float2(b0.x, b0.y), make_float2(b0.z, b0.w), make_float2(b1.x, b1.y), make_float2(b1.z, b1.w)};
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            const float2 w = __fmul2_rn(__fmul2_rn(make_float2(vG[k][q + e], vG[k][q + e + 1]), bp[e / 2]), a2);
            f[e] = w.x, f[e + 1] = w.y;
          }
          Vec16<T> o;
          o.pack(f);
          packed[q / 2] = o.raw.x, packed[q / 2 + 1] = o.raw.y, packed[q / 2 + 2] = o.raw.z, packed[q / 2 + 3] = o.raw.w;
        }
      } else if (fast[k]) {  // the chunk of this warp's own rows: steps after the row are cut
        const float2 a2 = make_float2(arow[k], arow[k]);
#pragma unroll
        for (int q = 0; q < 32; q += 8) {
          const float4 b0 = *reinterpret_cast<const float4*>(sW + k * 32 + q);
          const float4 b1 = *reinterpret_cast<const float4*>(sW + k * 32 + q + 4);
          const float2 bp[4] = {make_float2(b0.x, b0.y), make_float2(b0.z, b0.w), make_float2(b1.x, b1.y), make_float2(b1.z, b1.w)};
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            float2 w = __fmul2_rn(__fmul2_rn(make_float2(vG[k][q + e], vG[k][q + e + 1]), bp[e / 2]), a2);
            if (q + e > lane) w.x = 0.f;
            if (q + e + 1 > lane) w.y = 0.f;
            if (q + e == lane) w.x += Dfold;
            if (q + e + 1 == lane) w.y += Dfold;
            f[e] = w.x, f[e + 1] = w.y;
          }
          Vec16<T> o;
          o.pack(f);
          packed[q / 2] = o.raw.x, packed[q / 2 + 1] = o.raw.y, packed[q / 2 + 2] = o.raw.z, packed[q / 2 + 3] = o.raw.w;
        }
      } else {
#pragma unroll
        for (int q = 0; q < 32; q += 8) {
          const float4 c0 = *reinterpret_cast<const float4*>(vcp + jb + q);
          const float4 c1 = *reinterpret_cast<const float4*>(vcp + jb + q + 4);
          const float cj[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            float w = ex2_approx(ct - cj[e]);
            if (diag && q + e > lane) w = 0.f;
            f[e] = vG[k][q + e] * w;
            if (diag && q + e == lane) f[e] += Dfold;
          }
          Vec16<T> o;
          o.pack(f);
          packed[q / 2] = o.raw.x, packed[q / 2 + 1] = o.raw.y, packed[q / 2 + 2] = o.raw.z, packed[q / 2 + 3] = o.raw.w;
        }
      }
      tc::tmem_st16(dst, packed);
    }
    tc::tmem_wait_st();
    }
    // this row of x (for D x in the epilogue one iteration later)
    uint4 xr[kXR];
#pragma unroll
    for (int q = 0; q < kXR; ++q)
      xr[q] = XSKIP ? *reinterpret_cast<const uint4*>(swz(sX + buf * M::X_BYTES, i_chunk, wg * kEU + q)) : make_uint4(0, 0, 0, 0);


    if (tid == kCopyThread && hi >= 2) tc::bulk_wait_read();  // the staging tile may be overwritten by the epilogue below
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();

    // ---- Y_intra = (G o L) X  for this head; the commit also covers the Y_inter MMAs issued above --------------
    if (mma_warp && tc::elect_one()) {
      // descriptors differ from instruction to instruction only in the start address (16-byte units, low bits)
      const uint64_t dx0 = tc::smem_desc_sw128(tc::smem_u32(sX + buf * M::X_BYTES), 16, 1024);
      constexpr uint32_t idY = tc::instr_desc(kBlk, kP, fmt, 0, 1);
      const uint32_t dY = tmem + 256 + buf * 128;
#pragma unroll
      for (int kk = 0; kk < KJ / 16; ++kk)  // 16 steps = 16 rows of 128 bytes of the x tile
        tc::mma_ts(dY, tmem + kk * 8, dx0 + (uint64_t)(kk * (2048 >> 4)), idY, kk > 0);  // A: 16 steps = 8 columns of the masked rows
      tc::commit(mb_mma(buf));
    }
    // ---- the previous head's result, while the tensor cores work on this one ---------------------------------
    if (hi > 0) {
      if (has_z) ok = tc::mbar_wait(mb_z(buf ^ 1), ((hi - 1) >> 1) & 1);
      if (ok) epilogue(h - 1, buf ^ 1, ct_prev, xr_prev);
      else fail = 1;  // becomes CTA-wide at the next iteration's barrier (or right after the loop)
    }
    ct_prev = ct;
#pragma unroll
    for (int q = 0; q < kXR; ++q) xr_prev[q] = xr[q];
  }
  // leave the loop together: a thread that saw a wait run out above still reaches the same barriers
  fail = __syncthreads_or(fail);
  if (!fail && nh > 0) {
    const int last = nh - 1, buf = last & 1;
    ok = tc::mbar_wait(mb_mma(buf), (last >> 1) & 1);
    tc::fence_after_sync();
    ok = __syncthreads_and(ok);
    if (ok) {
      if (tid == kCopyThread) {
        if (nh >= 2) {
          tc::tma_store_4d(&maps.y, tc::smem_u32(sZ), 0, h0 + last - 1, t_blk, b);
          tc::bulk_commit();
          tc::bulk_wait_read();
        }
      }
      if (has_z) ok = tc::mbar_wait(mb_z(buf), (last >> 1) & 1);
      ok = __syncthreads_and(ok);  // also orders thread 0's wait on the store's reads before everyone's writes
      if (ok) {
        epilogue(h0 + last, buf, ct_prev, xr_prev);
        __syncthreads();
        if (tid == kCopyThread) {
          tc::tma_store_4d(&maps.y, tc::smem_u32(sZ), 0, h0 + last, t_blk, b);
          tc::bulk_commit();
        }
      } else {
        fail = 1;
      }
    } else {
      fail = 1;
    }
  }
  if (tid == kCopyThread) tc::bulk_wait_all();  // the staging tile must outlive the stores that read it
  if (fail && tid == 0 && a.status) atomicExch(a.status, 2);
}

template <typename T, bool XSKIP>
__global__ void __launch_bounds__(kScanThreads, 1)
    ssd_scan_kernel(const ssm_ssd_args a, const __grid_constant__ ScanMaps maps, int nchunks, int hpc, int nparts) {
  extern __shared__ unsigned char smdyn[];
  unsigned char* smraw = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smdyn) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t mbar[8];
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5;
  if (warp == 0) tc::tmem_alloc(tc::smem_u32(&tmem_slot), 512);
  if (threadIdx.x == 0) {
    for (int i = 0; i < 8; ++i) tc::mbar_init(tc::smem_u32(&mbar[i]), 1);
  }
  __syncthreads();  // barriers and the TMEM address are set up before anyone arms or polls them
  // the heavier blocks (rows 128..255) are scheduled first
  if ((int)blockIdx.x < (int)(gridDim.x >> 1)) ssd_scan_body<T, 1, XSKIP>(a, maps, nchunks, hpc, nparts, smraw, mbar, &tmem_slot);
  else ssd_scan_body<T, 0, XSKIP>(a, maps, nchunks, hpc, nparts, smraw, mbar, &tmem_slot);
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_slot, 512);
}

// ---- tensor maps (driver entry point fetched through the runtime; no link-time dependency on the driver) -------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}
// (batch, len, outer, inner) tensor of 16-bit elements seen as rank 4 (inner, outer, step, batch);
// box = 64 inner elements of one outer index x `rows` steps
static int encode_rows_map(CUtensorMap* m, const void* base, const ssm_ssd_args& a, int rows, int inner = kP, int outer = -1) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return ::ssmb::fail(SSM_ERR_DEVICE, "ssd_scan: cuTensorMapEncodeTiled is not available from this driver");
  if (outer < 0) outer = a.heads;
  const cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)a.len, (cuuint64_t)a.batch};
  const cuuint64_t strides[3] = {(cuuint64_t)inner * 2, (cuuint64_t)outer * inner * 2, (cuuint64_t)a.len * outer * inner * 2};
  const cuuint32_t box[4] = {(cuuint32_t)kP, 1, (cuuint32_t)rows, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = a.io_dtype == SSM_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult rc = fn(m, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return ::ssmb::fail(SSM_ERR_DEVICE, "ssd_scan: cuTensorMapEncodeTiled rejected the tensor");
  return SSM_OK;
}

template <typename T, int HPC>
static int ssd_state_launch(const ssm_ssd_args& a, int nchunks, cudaStream_t st) {
  StateMaps maps;
  if (int rc = encode_rows_map(&maps.b, a.Bm, a, StateSmem<HPC>::kStep, a.bc_width ? a.bc_width : kN, a.groups)) return rc;
  if (int rc = encode_rows_map(&maps.x, a.X, a, StateSmem<HPC>::kStep, kP, a.x_heads ? a.x_heads : a.heads)) return rc;
  const size_t smem = StateSmem<HPC>::ALLOC;
  cudaFuncSetAttribute(ssd_state_kernel<T, HPC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  ssd_state_kernel<T, HPC><<<dim3(a.heads / HPC, a.batch), kStateThreads, smem, st>>>(a, maps, nchunks);
  return launch_status("ssd_state_kernel");
}

// ---------------------------------------------------------------------------------------------
// incoming state of sequence shard `rank` from every rank's (final state from a zero start | total log-decay):
//   S_in = sum_{q < rank} exp(sum_{q < m < rank} logP_m) S_q  (+ exp(sum_{m < rank} logP_m) initial)
// `gathered`: world x per_rank floats, each rank's block = batch_heads * elems states then batch_heads log-decays.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ssd_fold_shards_kernel(const float* __restrict__ gathered, int rank, int64_t per_rank, int batch_heads, int elems,
                                                              const float* __restrict__ initial, float* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= (int64_t)batch_heads * elems) return;
  const int bh = (int)(i / elems);
  float s = initial ? __ldg(initial + i) : 0.f;
  for (int q = 0; q < rank; ++q) {
    const float* blk = gathered + (int64_t)q * per_rank;
    s = fmaf(__expf(__ldg(blk + (int64_t)batch_heads * elems + bh)), s, __ldg(blk + i));
  }
  out[i] = s;
}

// Self-test of the bounded waits: one warp waits on an mbarrier that nothing ever arms, with a limit of `probes` probes
// (about a microsecond each).  The wait runs out, the kernel records status 3 and returns normally: the path every
// kernel above takes if one of its copies or MMAs never completes, exercised without a fault.
__global__ void __launch_bounds__(32) ssd_wait_selftest_kernel(int32_t* status, int probes) {
  __shared__ __align__(8) uint64_t mbar;
  if (threadIdx.x == 0) tc::mbar_init(tc::smem_u32(&mbar), 1);
  __syncwarp();
  const bool ok = tc::mbar_wait(tc::smem_u32(&mbar), 0, probes);
  if (!ok && threadIdx.x == 0 && status) atomicExch(status, 3);
}

template <typename T>
static int ssd_launch(const ssm_ssd_args& a, cudaStream_t st) {
  const int nchunks = (a.len + kQ - 1) / kQ;
  // heads per scan CTA (a divisor of the heads of one B / C group, so that a CTA's heads share their G): every CTA
  // pays a prologue (C / B tiles, G) of about two heads' worth of time, and the grid runs in whole waves of one CTA
  // per SM; take the divisor with the least (waves x (prologue + heads)).
  const int hpg = a.heads / a.groups;
  int sm_count = 148;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  int hpc = 1;
  {
    double best = 1e300;
    for (int d = 1; d <= hpg && d <= 32; ++d) {
      if (hpg % d) continue;
      const int64_t ctas = 2ll * a.batch * nchunks * (a.heads / d);
      const double cost = (double)((ctas + sm_count - 1) / sm_count) * (2.0 + d);
      if (cost < best) best = cost, hpc = d;
    }
  }
  const int nparts = a.heads / hpc;
  if (a.phase != 2) {
    ssd_cumsum_kernel<T><<<dim3((a.heads + kCumHeads - 1) / kCumHeads, nchunks, a.batch), kQ, 0, st>>>(a, nchunks);
    if (int rc = launch_status("ssd_cumsum_kernel")) return rc;
  }
  if (a.phase != 2) {
    // heads per CTA of the sequential state kernel: enough to bring the grid down to about one CTA per SM
    // (its CTAs all run for the whole sequence, so a second, partial wave would double the time), at most 4,
    // and a divisor of the heads of one B / C group
    int shpc = (int)(((int64_t)a.batch * a.heads + sm_count - 1) / sm_count);
    shpc = shpc < 1 ? 1 : (shpc > 4 ? 4 : shpc);
    while (hpg % shpc != 0) --shpc;
    // between one and two (batch, head) pairs per SM: two heads per CTA would leave almost half of the SMs idle; one head per
    // CTA, two CTAs per SM (they fit) keeps every SM busy and halves what the longest SM has to walk
    if ((int64_t)a.batch * a.heads > sm_count && (int64_t)a.batch * a.heads <= 2 * (int64_t)sm_count) shpc = 1;
    int rc;
    switch (shpc) {
      case 1: rc = ssd_state_launch<T, 1>(a, nchunks, st); break;
      case 2: rc = ssd_state_launch<T, 2>(a, nchunks, st); break;
      case 3: rc = ssd_state_launch<T, 3>(a, nchunks, st); break;
      default: rc = ssd_state_launch<T, 4>(a, nchunks, st); break;
    }
    if (rc) return rc;
  } else if (a.initial_states) {
    const int64_t units = (int64_t)a.batch * a.heads * (kP * kN / 8);
    ssd_fold_init_kernel<T><<<dim3((unsigned)((units + 255) / 256), (nchunks + 1 + kFoldChunks - 1) / kFoldChunks), 256, 0, st>>>(a, nchunks);
    if (int rc = launch_status("ssd_fold_init_kernel")) return rc;
  } else if (a.final_states) {  // nothing arrives: the final state is the one phase 1 left in the scratch
    const cudaError_t e = cudaMemcpyAsync(a.final_states, a.ws_state, sizeof(float) * (size_t)a.batch * a.heads * kP * kN, cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return ::ssmb::fail((int)e, "ssd_scan: copying the final state failed");
  }
  if (a.phase != 1) {
    ScanMaps maps;
    const int xh = a.x_heads ? a.x_heads : a.heads;  // input heads stored
    if (int rc = encode_rows_map(&maps.x0, a.X, a, kBlk, kP, xh)) return rc;
    if (int rc = encode_rows_map(&maps.x1, a.X, a, kQ, kP, xh)) return rc;
    if (int rc = encode_rows_map(&maps.z, a.z ? a.z : a.Y, a, kBlk)) return rc;
    if (int rc = encode_rows_map(&maps.y, a.Y, a, kBlk)) return rc;
    // narrower stored rows (bc_width 64): the copies of the upper 64 states start outside the tensor and bring zeros
    const int bcw = a.bc_width ? a.bc_width : kN;
    if (int rc = encode_rows_map(&maps.c, a.Cm, a, kBlk, bcw, a.groups)) return rc;
    if (int rc = encode_rows_map(&maps.bm, a.Bm, a, kBlk, bcw, a.groups)) return rc;
    const size_t smem = ScanSmem<T>::ALLOC;
    const unsigned ctas = 2u * nparts * a.batch * nchunks;
    if (a.D && (a.d_has_p || a.row_dots)) {
      cudaFuncSetAttribute(ssd_scan_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      ssd_scan_kernel<T, true><<<ctas, kScanThreads, smem, st>>>(a, maps, nchunks, hpc, nparts);
    } else {
      cudaFuncSetAttribute(ssd_scan_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      ssd_scan_kernel<T, false><<<ctas, kScanThreads, smem, st>>>(a, maps, nchunks, hpc, nparts);
    }
    if (int rc = launch_status("ssd_scan_kernel")) return rc;
  }
  return SSM_OK;
}

}  // namespace ssmb

using namespace ssmb;

extern "C" int ssm_ssd_supported(int32_t headdim, int32_t nstate, int32_t chunk_size, int32_t io_dtype) {
  return headdim == kP && nstate == kN && chunk_size == kQ && (io_dtype == SSM_BF16 || io_dtype == SSM_F16);
}

extern "C" int64_t ssm_ssd_state_scratch_bytes(int32_t batch, int32_t len, int32_t heads) {
  const int64_t nchunks = (len + kQ - 1) / kQ;
  return ((ssd_summary_floats_padded(batch, heads) + (int64_t)batch * heads * nchunks) * 4 + 255) / 256 * 256;
}

extern "C" int64_t ssm_ssd_scratch_bytes(int32_t batch, int32_t len, int32_t heads) {
  const int64_t nchunks = (len + kQ - 1) / kQ;
  const int64_t vec = (int64_t)batch * heads * nchunks * kQ * 4;      // delta, cum (each)
  const int64_t fin = ssm_ssd_state_scratch_bytes(batch, len, heads);  // shard-local final state, total log-decay, per-chunk decay prefixes
  const int64_t st = (int64_t)batch * nchunks * heads * kP * kN * 2;  // state before every chunk, operand dtype
  return 2 * vec + fin + st;
}

extern "C" int64_t ssm_ssd_shard_summary_floats(int32_t batch, int32_t heads) { return (int64_t)batch * heads * (kP * kN + 1); }

extern "C" int ssm_ssd_fold_shards(const float* gathered, int32_t world, int32_t rank, int32_t batch, int32_t heads, const float* initial_states,
                                   float* incoming, ssm_stream_t stream) {
  SSM_REQUIRE(gathered && incoming, SSM_ERR_NULL, "ssd_fold_shards: missing tensor");
  SSM_REQUIRE(world >= 1 && rank >= 0 && rank < world && batch >= 0 && heads >= 1, SSM_ERR_SHAPE, "ssd_fold_shards: bad shape");
  const int64_t total = (int64_t)batch * heads * kP * kN;
  if (total == 0) return SSM_OK;
  ssd_fold_shards_kernel<<<(unsigned)((total + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      gathered, rank, ssm_ssd_shard_summary_floats(batch, heads), batch * heads, kP * kN, initial_states, incoming);
  return launch_status("ssd_fold_shards_kernel");
}

extern "C" int ssm_ssd_wait_selftest(int32_t* status, int32_t probes, ssm_stream_t stream) {
  SSM_REQUIRE(status != nullptr, SSM_ERR_NULL, "ssd_wait_selftest: status is NULL");
  SSM_REQUIRE(probes >= 1 && probes <= 100000, SSM_ERR_SHAPE, "ssd_wait_selftest: probes must be in [1, 100000]");
  ssd_wait_selftest_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(status, probes);
  return launch_status("ssd_wait_selftest_kernel");
}

extern "C" int ssm_ssd_fwd(const ssm_ssd_args* a, ssm_stream_t stream) {
  SSM_REQUIRE(a != nullptr, SSM_ERR_NULL, "ssd_scan: args is NULL");
  SSM_REQUIRE(a->batch >= 0 && a->len >= 0 && a->heads >= 1 && a->groups >= 1, SSM_ERR_SHAPE, "ssd_scan: bad shape");
  SSM_REQUIRE(a->heads % a->groups == 0, SSM_ERR_SHAPE, "Group dimension must divide H.");
  SSM_REQUIRE(ssm_ssd_supported(a->headdim, a->nstate, a->chunk_size, a->io_dtype), SSM_ERR_UNSUPPORTED,
              "ssd_scan: the tensor-core path is built for headdim 64, d_state 128, chunk 256, bf16 / fp16");
  if (a->batch == 0 || a->len == 0) return SSM_OK;
  SSM_REQUIRE(a->phase >= 0 && a->phase <= 2, SSM_ERR_SHAPE, "ssd_scan: phase must be 0, 1 or 2");
  SSM_REQUIRE(a->dt_mode >= 0 && a->dt_mode <= 7 && (a->dt_mode & 3) != 2, SSM_ERR_SHAPE, "ssd_scan: dt_mode must be 0, 1 or 3, optionally + 4");
  SSM_REQUIRE(a->bc_width == 0 || a->bc_width == kN || a->bc_width == 64, SSM_ERR_SHAPE, "ssd_scan: bc_width must be 0, 64 or nstate");
  SSM_REQUIRE(a->x_heads >= 0 && (a->x_heads == 0 || a->heads % a->x_heads == 0), SSM_ERR_SHAPE, "ssd_scan: x_heads must be 0 or divide heads");
  SSM_REQUIRE(a->X && a->dt && a->A && a->Bm && a->Cm && (a->Y || a->phase == 1), SSM_ERR_NULL, "ssd_scan: missing tensor");
  SSM_REQUIRE(a->ws_dt && a->ws_cum && a->ws_state && a->ws_state_in, SSM_ERR_NULL, "ssd_scan: missing scratch");
  SSM_REQUIRE(aligned_to(a->X, 16) && aligned_to(a->Bm, 16) && aligned_to(a->Cm, 16) && (!a->Y || aligned_to(a->Y, 16)) && aligned_to(a->ws_state_in, 16) &&
                  (!a->z || aligned_to(a->z, 16)),
              SSM_ERR_ALIGN, "ssd_scan: tensors must be 16-byte aligned");
  const int64_t nchunks = (a->len + kQ - 1) / kQ;
  SSM_REQUIRE((int64_t)a->batch * nchunks <= 65535 && a->heads <= 65535 && (int64_t)a->batch * nchunks * a->heads * 2 < (1ll << 31), SSM_ERR_TOO_LARGE,
              "ssd_scan: grid too large");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a->io_dtype == SSM_BF16) return ssd_launch<__nv_bfloat16>(*a, st);
  return ssd_launch<__half>(*a, st);
}
