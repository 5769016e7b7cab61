// Instantiates the selective-scan forward kernels for __nv_bfloat16 activations (one element type per
// translation unit so that the variants compile in parallel).
#include "selective_scan_fwd.cuh"

namespace ssmb {
template int dispatch_fwd<__nv_bfloat16>(const ssm_scan_fwd_args&, const ScanFlags&, cudaStream_t);
}  // namespace ssmb
