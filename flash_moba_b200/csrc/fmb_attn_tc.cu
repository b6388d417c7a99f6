// tcgen05 tensor-core engine of the block-sparse attention (placeholder until validated).
#include "fmb_attn.cuh"

namespace fmb {
bool tc_supported(const AttnArgs&, bool) { return false; }
int launch_fwd_main_tc(const AttnArgs&, const AttnWorkspace&, cudaStream_t) {
  return fail(FMB_ERR_UNSUPPORTED, "tensor-core engine not built");
}
int launch_bwd_main_tc(const AttnArgs&, const AttnWorkspace&, cudaStream_t) {
  return fail(FMB_ERR_UNSUPPORTED, "tensor-core engine not built");
}
}  // namespace fmb
