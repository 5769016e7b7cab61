// C-ABI entry point of the selective-scan backward; the kernels live in selective_scan_bwd.cuh and are
// instantiated per element type in selective_scan_bwd_*.cu.
#include "scan_common.cuh"

namespace ssmb {
template <typename T>
int dispatch_bwd(const ssm_scan_bwd_args& a, const ScanFlags& fl, cudaStream_t st);
extern template int dispatch_bwd<float>(const ssm_scan_bwd_args&, const ScanFlags&, cudaStream_t);
extern template int dispatch_bwd<__nv_bfloat16>(const ssm_scan_bwd_args&, const ScanFlags&, cudaStream_t);
extern template int dispatch_bwd<__half>(const ssm_scan_bwd_args&, const ScanFlags&, cudaStream_t);
int scan_validate(const ssm_scan_fwd_args* a, ScanFlags* fl, int rows_per_cta);
}  // namespace ssmb

using namespace ssmb;

extern "C" int ssm_selective_scan_bwd(const ssm_scan_bwd_args* g, ssm_stream_t stream) {
  SSM_REQUIRE(g != nullptr, SSM_ERR_NULL, "selective_scan_backward: args is NULL");
  const ssm_scan_fwd_args* a = &g->fwd;
  if (a->io_dtype == SSM_F64) return f64_scan_bwd(*g, reinterpret_cast<cudaStream_t>(stream));
  ScanFlags fl{};
  if (int rc = scan_validate(a, &fl, 1)) return rc;
  if (a->batch == 0 || a->dim == 0 || a->len == 0) return SSM_OK;
  SSM_REQUIRE(a->checkpoints, SSM_ERR_NULL, "selective_scan_backward: forward checkpoints are required");
  SSM_REQUIRE(g->dout && g->du && g->ddelta && g->dA && g->dB && g->dC, SSM_ERR_NULL, "selective_scan_backward: missing pointer");
  SSM_REQUIRE(!a->z == !g->dz, SSM_ERR_NULL, "selective_scan_backward: dz must be given exactly when z is");
  fl.io_vec = fl.io_vec && aligned_to(g->dout, 16) && aligned_to(g->du, 16) && aligned_to(g->ddelta, 16) && (!g->dz || aligned_to(g->dz, 16));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (a->io_dtype) {
    case SSM_F32: return dispatch_bwd<float>(*g, fl, st);
    case SSM_BF16: return dispatch_bwd<__nv_bfloat16>(*g, fl, st);
    default: return dispatch_bwd<__half>(*g, fl, st);
  }
}
