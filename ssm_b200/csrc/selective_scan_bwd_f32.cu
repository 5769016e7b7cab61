// Instantiates the selective-scan backward kernels for float activations (one element type per
// translation unit so that the variants compile in parallel).
#include "selective_scan_bwd.cuh"

namespace ssmb {
template int dispatch_bwd<float>(const ssm_scan_bwd_args&, const ScanFlags&, cudaStream_t);
}  // namespace ssmb
