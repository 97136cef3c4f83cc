// Tensor-core (tcgen05 / TMEM) prefill attention.  Placeholder translation unit until the
// kernel lands: reports "unsupported" so that every prefill goes through the general kernel.
#include "attn.cuh"
#include "common.cuh"

namespace piekv {

bool prefill_tc_supported(const AttnArgs &, int) { return false; }

int64_t prefill_tc_workspace_bytes(int, int, int) { return 65536; }

int launch_prefill_tc(const AttnArgs &, int, void *, int64_t, cudaStream_t) {
  set_error("prefill: tensor-core kernel not built");
  return 1;
}

}  // namespace piekv
