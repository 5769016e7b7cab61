// C-ABI entry point of the selective-scan forward; the kernels live in selective_scan_fwd.cuh and are
// instantiated per element type in selective_scan_fwd_*.cu.
#include "scan_common.cuh"
#include "selective_scan_fwd_tiles.cuh"

namespace ssmb {
template <typename T>
int dispatch_fwd(const ssm_scan_fwd_args& a, const ScanFlags& fl, cudaStream_t st);
extern template int dispatch_fwd<float>(const ssm_scan_fwd_args&, const ScanFlags&, cudaStream_t);
extern template int dispatch_fwd<__nv_bfloat16>(const ssm_scan_fwd_args&, const ScanFlags&, cudaStream_t);
extern template int dispatch_fwd<__half>(const ssm_scan_fwd_args&, const ScanFlags&, cudaStream_t);
int scan_validate(const ssm_scan_fwd_args* a, ScanFlags* fl, int rows_per_cta);
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
  SSM_REQUIRE(a->row_sb >= 0 && a->row_sd >= a->len, SSM_ERR_SHAPE, "selective_scan: bad row strides");
  fl->io_vec = (a->len % v == 0) && (a->row_sb % v == 0) && (a->row_sd % v == 0) && aligned_to(a->u, 16) && aligned_to(a->delta, 16) && (!a->z || aligned_to(a->z, 16)) &&
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

extern "C" int ssm_scan_checkpoint_interval(void) { return kScanCkpt; }

extern "C" int ssm_scan_split_segments(int32_t batch, int32_t dim, int32_t len, int32_t nstate) {
  if (batch <= 0 || dim <= 0 || len <= 0 || nstate > 32) return 1;  // the split lives in the tile kernel (d_state <= 32)
  return ssmb::fwd_split_segments(batch, dim, len);
}

extern "C" int ssm_selective_scan_fwd(const ssm_scan_fwd_args* a, ssm_stream_t stream) {
  if (a && a->io_dtype == SSM_F64) return f64_scan_fwd(*a, reinterpret_cast<cudaStream_t>(stream));
  ScanFlags fl{};
  if (int rc = scan_validate(a, &fl, 1)) return rc;
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
