// Element-wise and reduction kernels around the dual-form backward of the state-space-dual scan.
//
// The contractions of that backward pass run on the forward pass's tensor-core kernels (ssd_scan.cu) applied to
// transformed operands: the time-reversed sequence for the adjoint recurrence, and the head / state axes exchanged for
// dB and dC.  What is left is bandwidth work over (batch, len, heads, headdim) tensors, done here in as few passes as
// the data flow allows:
//
//   ssd_bwd_gate_kernel     dy = gY * silu(z)  (or gY), written in time order and time-reversed
//   time_flip_kernel        rows of one (batch, len, row) tensor in reverse time order
//   ssd_bwd_finish_kernel   dz = gY * (y + D x) * silu'(z);  dX = reversed(dX_adj) + D dy;  dD = sum dy x
//   ssd_bwd_group_sum_kernel  per-head rows (batch, len, heads, 128) summed over the heads of a B / C group, optionally
//                           read in reverse time order and weighted per (step, head)
//   ssd_state_dot_kernel    <state before chunk c of one pass, state before chunk nchunks - c of the other>
//
// Every thread moves 16-byte units; rows are contiguous.
#include <type_traits>

#include "common.cuh"

namespace ssmb {

constexpr int kUnit = 8;  // 16-bit elements per 16-byte unit

// thread = one unit column of the (heads * headdim) row; grid.y = slices of the time axis; grid.z = batch
template <typename T>
__global__ void __launch_bounds__(256) ssd_bwd_gate_kernel(const ssm_ssd_bwd_args a, int steps_per_block) {
  const int units = a.heads * a.headdim / kUnit;
  const int u = blockIdx.x * 256 + threadIdx.x;
  if (u >= units) return;
  const int b = blockIdx.z;
  const int t_begin = blockIdx.y * steps_per_block;
  const int t_end = min(t_begin + steps_per_block, a.len);
  const int64_t row = (int64_t)a.heads * a.headdim;
  const T* gy = reinterpret_cast<const T*>(a.gY);
  const T* z = reinterpret_cast<const T*>(a.z);
  T* dy = reinterpret_cast<T*>(a.dy);
  T* dyr = reinterpret_cast<T*>(a.dy_rev);
#pragma unroll 4
  for (int t = t_begin; t < t_end; ++t) {
    const int64_t at = ((int64_t)b * a.len + t) * row + (int64_t)u * kUnit;
    const int64_t rt = ((int64_t)b * a.len + (a.len - 1 - t)) * row + (int64_t)u * kUnit;
    Vec16<T> g;
    float f[8];
    if (t < a.len_valid) {
      g.load_stream(gy + ((int64_t)b * a.len_valid + t) * row + (int64_t)u * kUnit);
      if (z) {
        Vec16<T> zz;
        float zv[8];
        zz.load(z + ((int64_t)b * a.len_valid + t) * row + (int64_t)u * kUnit);
        g.unpack(f);
        zz.unpack(zv);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] *= silu_fast(zv[e]);
        g.pack(f);
      }
    } else {
      g.raw = make_uint4(0, 0, 0, 0);  // padding up to whole chunks
    }
    g.store(dy + at);
    g.store(dyr + rt);
  }
}

// dst[b, len - 1 - t, :] = src[b, t, :]; src has len_valid rows per batch element, the rest of dst's rows are zero
__global__ void __launch_bounds__(256) time_flip_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int len, int len_valid, int row_units,
                                                        int steps_per_block) {
  const int u = blockIdx.x * 256 + threadIdx.x;
  if (u >= row_units) return;
  const int b = blockIdx.z;
  const int t_begin = blockIdx.y * steps_per_block;
  const int t_end = min(t_begin + steps_per_block, len);
#pragma unroll 4
  for (int t = t_begin; t < t_end; ++t) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t < len_valid) v = __ldcs(src + ((int64_t)b * len_valid + t) * row_units + u);
    dst[((int64_t)b * len + (len - 1 - t)) * row_units + u] = v;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) ssd_bwd_finish_kernel(const ssm_ssd_bwd_args a, int steps_per_block) {
  const int units = a.heads * a.headdim / kUnit;
  const int u = blockIdx.x * 256 + threadIdx.x;
  const bool live = u < units;
  const int b = blockIdx.z;
  const int t_begin = blockIdx.y * steps_per_block;
  const int t_end = min(t_begin + steps_per_block, a.len_valid);
  const int64_t row = (int64_t)a.heads * a.headdim;
  const int upr = a.headdim / kUnit;  // units per head
  const int h = live ? u / upr : 0, p0 = (u % upr) * kUnit;
  float Dv[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) Dv[e] = !a.D ? 0.f : (a.d_has_p ? __ldg(a.D + h * a.headdim + p0 + e) : __ldg(a.D + h));
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  const T* gy = reinterpret_cast<const T*>(a.gY);
  const T* z = reinterpret_cast<const T*>(a.z);
  const T* X = reinterpret_cast<const T*>(a.X);
  const T* yp = reinterpret_cast<const T*>(a.y_plain);
  const T* dy = reinterpret_cast<const T*>(a.dy);
  const T* dxr = reinterpret_cast<const T*>(a.dx_rev);
  T* dX = reinterpret_cast<T*>(a.dX);
  T* dz = reinterpret_cast<T*>(a.dz);
  if (live) {
#pragma unroll 2
    for (int t = t_begin; t < t_end; ++t) {
      const int64_t off = (int64_t)u * kUnit;
      const int64_t at_v = ((int64_t)b * a.len_valid + t) * row + off;       // tensors of the caller (unpadded)
      const int64_t at_p = ((int64_t)b * a.len + t) * row + off;             // padded work tensors
      const int64_t rt_p = ((int64_t)b * a.len + (a.len - 1 - t)) * row + off;
      Vec16<T> vx, vdy, vdx;
      float x[8], d[8], g[8];
      vx.load_stream(X + at_v);
      vdy.load_stream(dy + at_p);
      vdx.load_stream(dxr + rt_p);
      vx.unpack(x);
      vdy.unpack(d);
      vdx.unpack(g);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        acc[e] = fmaf(d[e], x[e], acc[e]);
        g[e] = fmaf(Dv[e], d[e], g[e]);
      }
      Vec16<T> o;
      o.pack(g);
      o.store_stream(dX + at_v);
      if (z) {
        Vec16<T> vg, vz, vy;
        float gg[8], zv[8], y[8];
        vg.load_stream(gy + at_v);
        vz.load_stream(z + at_v);
        vy.load_stream(yp + at_p);
        vg.unpack(gg);
        vz.unpack(zv);
        vy.unpack(y);
#pragma unroll
        for (int e = 0; e < 8; ++e) gg[e] *= fmaf(Dv[e], x[e], y[e]) * silu_grad_fast(zv[e]);
        o.pack(gg);
        o.store_stream(dz + at_v);
      }
    }
  }
  if (!a.dD) return;
  if (a.d_has_p) {
    if (live) {
#pragma unroll
      for (int e = 0; e < 8; ++e) atomicAdd(a.dD + h * a.headdim + p0 + e, acc[e]);
    }
  } else {
    // the units of one head are `upr` neighbouring lanes (headdim 64: 8 lanes): fold them, one atomic per head and warp
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) s += acc[e];
    if (!live) s = 0.f;
    for (int off = 1; off < upr && off < 32; off <<= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (live && (u % upr == 0 || upr > 32)) atomicAdd(a.dD + h, s);
  }
}

// out[b, t, g, :] = sum over the heads h of group g of  w[b, t, h] * y[b, ts, h, :],  ts = t or len - 1 - t;  rows of 128 states
template <typename T, typename TO>
__global__ void __launch_bounds__(256) ssd_bwd_group_sum_kernel(const T* __restrict__ y, const float* __restrict__ w, TO* __restrict__ out, int batch,
                                                                int len, int len_out, int heads, int groups, int nstate, int reversed) {
  const int upr = nstate / kUnit;
  const int64_t total = (int64_t)batch * len_out * groups * upr;
  const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (idx >= total) return;
  const int u = (int)(idx % upr);
  const int g = (int)((idx / upr) % groups);
  const int t = (int)((idx / ((int64_t)upr * groups)) % len_out);
  const int b = (int)(idx / ((int64_t)upr * groups * len_out));
  const int rep = heads / groups;
  const int ts = reversed ? len - 1 - t : t;
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  for (int r = 0; r < rep; ++r) {
    const int h = g * rep + r;
    Vec16<T> v;
    float f[8];
    v.load_stream(y + (((int64_t)b * len + ts) * heads + h) * nstate + (int64_t)u * kUnit);
    v.unpack(f);
    const float wt = w ? __ldg(w + ((int64_t)b * len + t) * heads + h) : 1.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = fmaf(wt, f[e], acc[e]);
  }
  TO* dst = out + (((int64_t)b * len_out + t) * groups + g) * nstate + (int64_t)u * kUnit;
  if constexpr (std::is_same<TO, float>::value) {
    *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
  } else {
    Vec16<TO> o;
    o.pack(acc);
    o.store(dst);
  }
}

// dst[r, h, :] = src[r, h / rep, :] for rows r = (batch, step): the rows of a B / C group handed to each of its heads
__global__ void __launch_bounds__(256) ssd_bwd_spread_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int64_t rows, int heads, int rep,
                                                             int units) {
  const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (idx >= rows * heads * units) return;
  const int u = (int)(idx % units);
  const int h = (int)((idx / units) % heads);
  const int64_t r = idx / ((int64_t)units * heads);
  dst[idx] = __ldg(src + (r * (heads / rep) + h / rep) * units + u);
}

// one warp per (batch, chunk c >= 1, head): out[b, c, h] = <fwd[b, c, h, :], adj[b, nchunks - c, h, :]>; out[b, 0, h] = 0
template <typename T>
__global__ void __launch_bounds__(128) ssd_state_dot_kernel(const T* __restrict__ fwd, const T* __restrict__ adj, float* __restrict__ out, int batch,
                                                            int nchunks, int heads, int elems) {
  const int warp = (blockIdx.x * 128 + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= batch * nchunks * heads) return;
  const int h = warp % heads, c = (warp / heads) % nchunks, b = warp / (heads * nchunks);
  float s = 0.f;
  if (c > 0) {
    const T* pa = fwd + (((int64_t)b * nchunks + c) * heads + h) * elems;
    const T* pb = adj + (((int64_t)b * nchunks + (nchunks - c)) * heads + h) * elems;
#pragma unroll 4
    for (int i = lane * kUnit; i < elems; i += 32 * kUnit) {
      Vec16<T> va, vb;
      float fa[8], fb[8];
      va.load_stream(pa + i);
      vb.load_stream(pb + i);
      va.unpack(fa);
      vb.unpack(fb);
#pragma unroll
      for (int e = 0; e < 8; ++e) s = fmaf(fa[e], fb[e], s);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  }
  if (lane == 0) out[warp] = s;
}

static int bwd_common_checks(const ssm_ssd_bwd_args* a, const char* what) {
  SSM_REQUIRE(a != nullptr, SSM_ERR_NULL, "ssd backward: args is NULL");
  SSM_REQUIRE(a->batch >= 0 && a->len >= 0 && a->len_valid >= 0 && a->len_valid <= a->len && a->heads >= 1 && a->headdim >= kUnit &&
                  a->headdim % kUnit == 0,
              SSM_ERR_SHAPE, "ssd backward: bad shape");
  SSM_REQUIRE(a->io_dtype == SSM_BF16 || a->io_dtype == SSM_F16, SSM_ERR_DTYPE, "ssd backward: operands must be bf16 or fp16");
  SSM_REQUIRE((int64_t)a->batch <= 65535, SSM_ERR_TOO_LARGE, "ssd backward: batch too large for one launch");
  (void)what;
  return SSM_OK;
}

__global__ void __launch_bounds__(128) ssd_state_dot_f32_kernel(const float* __restrict__ fwd, const float* __restrict__ adj, float* __restrict__ out,
                                                                int batch, int nchunks, int heads, int elems) {
  const int warp = (blockIdx.x * 128 + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= batch * nchunks * heads) return;
  const int h = warp % heads, c = (warp / heads) % nchunks, b = warp / (heads * nchunks);
  float s = 0.f;
  if (c > 0) {
    const float4* pa = reinterpret_cast<const float4*>(fwd + (((int64_t)b * nchunks + c) * heads + h) * elems);
    const float4* pb = reinterpret_cast<const float4*>(adj + (((int64_t)b * nchunks + (nchunks - c)) * heads + h) * elems);
    float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int i = lane; i < elems / 4; i += 32) {
      const float4 x = __ldcs(pa + i), y = __ldcs(pb + i);
      s4[0] = fmaf(x.x, y.x, s4[0]), s4[1] = fmaf(x.y, y.y, s4[1]), s4[2] = fmaf(x.z, y.z, s4[2]), s4[3] = fmaf(x.w, y.w, s4[3]);
    }
    s = (s4[0] + s4[1]) + (s4[2] + s4[3]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  }
  if (lane == 0) out[warp] = s;
}

}  // namespace ssmb

using namespace ssmb;

constexpr int kStepsPerBlock = 64;

extern "C" int ssm_ssd_bwd_gate(const ssm_ssd_bwd_args* a, ssm_stream_t stream) {
  if (int rc = bwd_common_checks(a, "gate")) return rc;
  if (a->batch == 0 || a->len == 0) return SSM_OK;
  SSM_REQUIRE(a->gY && a->dy && a->dy_rev, SSM_ERR_NULL, "ssd_bwd_gate: missing tensor");
  SSM_REQUIRE(aligned_to(a->gY, 16) && aligned_to(a->dy, 16) && aligned_to(a->dy_rev, 16) && (!a->z || aligned_to(a->z, 16)), SSM_ERR_ALIGN,
              "ssd_bwd_gate: tensors must be 16-byte aligned");
  const int units = a->heads * a->headdim / kUnit;
  const dim3 grid((units + 255) / 256, (a->len + kStepsPerBlock - 1) / kStepsPerBlock, a->batch);
  SSM_REQUIRE(grid.y <= 65535, SSM_ERR_TOO_LARGE, "ssd_bwd_gate: sequence too long for one launch");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a->io_dtype == SSM_BF16) ssd_bwd_gate_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(*a, kStepsPerBlock);
  else ssd_bwd_gate_kernel<__half><<<grid, 256, 0, st>>>(*a, kStepsPerBlock);
  return launch_status("ssd_bwd_gate_kernel");
}

extern "C" int ssm_ssd_bwd_finish(const ssm_ssd_bwd_args* a, ssm_stream_t stream) {
  if (int rc = bwd_common_checks(a, "finish")) return rc;
  if (a->batch == 0 || a->len_valid == 0) return SSM_OK;
  SSM_REQUIRE(a->X && a->dy && a->dx_rev && a->dX, SSM_ERR_NULL, "ssd_bwd_finish: missing tensor");
  SSM_REQUIRE(!a->z || (a->gY && a->y_plain && a->dz), SSM_ERR_NULL, "ssd_bwd_finish: a gate needs gY, y_plain and dz");
  SSM_REQUIRE(aligned_to(a->X, 16) && aligned_to(a->dy, 16) && aligned_to(a->dx_rev, 16) && aligned_to(a->dX, 16) && (!a->z || aligned_to(a->z, 16)) &&
                  (!a->gY || aligned_to(a->gY, 16)) && (!a->y_plain || aligned_to(a->y_plain, 16)) && (!a->dz || aligned_to(a->dz, 16)),
              SSM_ERR_ALIGN, "ssd_bwd_finish: tensors must be 16-byte aligned");
  const int units = a->heads * a->headdim / kUnit;
  const dim3 grid((units + 255) / 256, (a->len_valid + kStepsPerBlock - 1) / kStepsPerBlock, a->batch);
  SSM_REQUIRE(grid.y <= 65535, SSM_ERR_TOO_LARGE, "ssd_bwd_finish: sequence too long for one launch");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a->io_dtype == SSM_BF16) ssd_bwd_finish_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(*a, kStepsPerBlock);
  else ssd_bwd_finish_kernel<__half><<<grid, 256, 0, st>>>(*a, kStepsPerBlock);
  return launch_status("ssd_bwd_finish_kernel");
}

extern "C" int ssm_time_flip(const void* src, void* dst, int32_t batch, int32_t len, int32_t len_valid, int64_t row_bytes, ssm_stream_t stream) {
  SSM_REQUIRE(batch >= 0 && len >= 0 && len_valid >= 0 && len_valid <= len && row_bytes >= 0, SSM_ERR_SHAPE, "time_flip: bad shape");
  if (batch == 0 || len == 0 || row_bytes == 0) return SSM_OK;
  SSM_REQUIRE(src && dst, SSM_ERR_NULL, "time_flip: missing tensor");
  SSM_REQUIRE(row_bytes % 16 == 0 && aligned_to(src, 16) && aligned_to(dst, 16), SSM_ERR_ALIGN, "time_flip: rows must be whole 16-byte units");
  SSM_REQUIRE(batch <= 65535 && row_bytes / 16 < (1ll << 31), SSM_ERR_TOO_LARGE, "time_flip: too large for one launch");
  const int units = (int)(row_bytes / 16);
  const int spb = units >= 256 ? 16 : 64;
  const dim3 grid((units + 255) / 256, (len + spb - 1) / spb, batch);
  SSM_REQUIRE(grid.y <= 65535, SSM_ERR_TOO_LARGE, "time_flip: sequence too long for one launch");
  time_flip_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst), len, len_valid,
                                                                            units, spb);
  return launch_status("time_flip_kernel");
}

extern "C" int ssm_ssd_bwd_group_sum(const void* y, const float* weight, void* out, int32_t batch, int32_t len, int32_t len_out, int32_t heads,
                                     int32_t groups, int32_t nstate, int32_t reversed, int32_t io_dtype, int32_t out_dtype, ssm_stream_t stream) {
  SSM_REQUIRE(batch >= 0 && len >= 0 && len_out >= 0 && len_out <= len && heads >= 1 && groups >= 1 && heads % groups == 0 && nstate >= kUnit &&
                  nstate % kUnit == 0,
              SSM_ERR_SHAPE, "ssd_bwd_group_sum: bad shape");
  SSM_REQUIRE(io_dtype == SSM_BF16 || io_dtype == SSM_F16, SSM_ERR_DTYPE, "ssd_bwd_group_sum: rows must be bf16 or fp16");
  SSM_REQUIRE(out_dtype == io_dtype || out_dtype == SSM_F32, SSM_ERR_DTYPE, "ssd_bwd_group_sum: the sum is written in the rows' dtype or fp32");
  if (batch == 0 || len_out == 0) return SSM_OK;
  SSM_REQUIRE(y && out, SSM_ERR_NULL, "ssd_bwd_group_sum: missing tensor");
  SSM_REQUIRE(aligned_to(y, 16) && aligned_to(out, 16), SSM_ERR_ALIGN, "ssd_bwd_group_sum: tensors must be 16-byte aligned");
  const int64_t total = (int64_t)batch * len_out * groups * (nstate / kUnit);
  SSM_REQUIRE((total + 255) / 256 < (1ll << 31), SSM_ERR_TOO_LARGE, "ssd_bwd_group_sum: too large for one launch");
  const unsigned grid = (unsigned)((total + 255) / 256);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define SSM_GS(T, TO) \
  ssd_bwd_group_sum_kernel<T, TO><<<grid, 256, 0, st>>>(reinterpret_cast<const T*>(y), weight, reinterpret_cast<TO*>(out), batch, len, len_out, heads, \
                                                        groups, nstate, reversed)
  if (io_dtype == SSM_BF16) {
    if (out_dtype == SSM_F32) SSM_GS(__nv_bfloat16, float);
    else SSM_GS(__nv_bfloat16, __nv_bfloat16);
  } else {
    if (out_dtype == SSM_F32) SSM_GS(__half, float);
    else SSM_GS(__half, __half);
  }
#undef SSM_GS
  return launch_status("ssd_bwd_group_sum_kernel");
}

extern "C" int ssm_ssd_bwd_spread(const void* src, void* dst, int64_t rows, int32_t heads, int32_t groups, int64_t row_bytes, ssm_stream_t stream) {
  SSM_REQUIRE(rows >= 0 && heads >= 1 && groups >= 1 && heads % groups == 0 && row_bytes >= 0, SSM_ERR_SHAPE, "ssd_bwd_spread: bad shape");
  if (rows == 0 || row_bytes == 0) return SSM_OK;
  SSM_REQUIRE(src && dst, SSM_ERR_NULL, "ssd_bwd_spread: missing tensor");
  SSM_REQUIRE(row_bytes % 16 == 0 && aligned_to(src, 16) && aligned_to(dst, 16), SSM_ERR_ALIGN, "ssd_bwd_spread: rows must be whole 16-byte units");
  const int64_t total = rows * heads * (row_bytes / 16);
  SSM_REQUIRE((total + 255) / 256 < (1ll << 31), SSM_ERR_TOO_LARGE, "ssd_bwd_spread: too large for one launch");
  ssd_bwd_spread_kernel<<<(unsigned)((total + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst), rows, heads, heads / groups, (int)(row_bytes / 16));
  return launch_status("ssd_bwd_spread_kernel");
}

extern "C" int ssm_ssd_state_dot(const void* fwd_states, const void* adj_states, float* out, int32_t batch, int32_t nchunks, int32_t heads, int32_t elems,
                                 int32_t io_dtype, ssm_stream_t stream) {
  SSM_REQUIRE(batch >= 0 && nchunks >= 0 && heads >= 1 && elems >= 0 && elems % (32 * kUnit) == 0, SSM_ERR_SHAPE, "ssd_state_dot: bad shape");
  SSM_REQUIRE(io_dtype == SSM_BF16 || io_dtype == SSM_F16 || io_dtype == SSM_F32, SSM_ERR_DTYPE, "ssd_state_dot: states must be bf16, fp16 or fp32");
  if (batch == 0 || nchunks == 0) return SSM_OK;
  SSM_REQUIRE(fwd_states && adj_states && out, SSM_ERR_NULL, "ssd_state_dot: missing tensor");
  SSM_REQUIRE(aligned_to(fwd_states, 16) && aligned_to(adj_states, 16), SSM_ERR_ALIGN, "ssd_state_dot: tensors must be 16-byte aligned");
  const int64_t warps = (int64_t)batch * nchunks * heads;
  SSM_REQUIRE(warps < (1ll << 28), SSM_ERR_TOO_LARGE, "ssd_state_dot: too large for one launch");
  const unsigned grid = (unsigned)((warps * 32 + 127) / 128);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (io_dtype == SSM_F32)
    ssd_state_dot_f32_kernel<<<grid, 128, 0, st>>>(reinterpret_cast<const float*>(fwd_states), reinterpret_cast<const float*>(adj_states), out, batch, nchunks,
                                                   heads, elems);
  else if (io_dtype == SSM_BF16)
    ssd_state_dot_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(fwd_states),
                                                              reinterpret_cast<const __nv_bfloat16*>(adj_states), out, batch, nchunks, heads, elems);
  else
    ssd_state_dot_kernel<__half><<<grid, 128, 0, st>>>(reinterpret_cast<const __half*>(fwd_states), reinterpret_cast<const __half*>(adj_states), out, batch,
                                                       nchunks, heads, elems);
  return launch_status("ssd_state_dot_kernel");
}
