// TEST INFRASTRUCTURE. Link-time stand-ins that let the reference's fused-CE module (wenhaochai/marin.cpp,
// src/kernels/cross_entropy + src/core) be built by itself for sm_100a, outside its own build system, as a GPU-side
// cross-check for the parity tests and a timing anchor. They replace only what that module references but a B200
// never runs: the three sm_90a (WGMMA) launchers, which the reference's dispatch calls only when the device is compute
// capability 9.0 (src/kernels/cross_entropy/ce_api.cpp:113-123), and the RMSNorm pair used by its readout entry point
// (not exercised through this build).
#include <cuda_runtime.h>

#include "kernels/cross_entropy/ce_internal.hpp"
#include "kernels/elementwise/ew_api.hpp"

namespace nm::ce {
bool launch_logits_stats_sm90(DType, const LogitsArgs&, cudaStream_t) { return false; }
bool launch_dgrad_sm90(DType, const DgradArgs&, cudaStream_t) { return false; }
bool launch_wgrad_sm90(DType, const WgradArgs&, cudaStream_t) { return false; }
}  // namespace nm::ce

namespace nm::ew {
void rmsnorm_fwd_dt(DType, const RmsNormFwd&, Rounding, cudaStream_t) {
  fatal(NM_WHERE, "readout norms are not part of this stand-alone build of the reference CE module");
}
void rmsnorm_bwd_add_dt(DType, const RmsNormBwdAdd&, Rounding, cudaStream_t) {
  fatal(NM_WHERE, "readout norms are not part of this stand-alone build of the reference CE module");
}
}  // namespace nm::ew
