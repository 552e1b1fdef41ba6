// gemm_tc.cu — tcgen05 prefill GEMM (placeholder until the tensor-memory kernel lands):
// reports "shape not covered" so callers take the mma.sync kernel.
#include "common.cuh"

namespace tq {

int launch_gemm_tc(const GemmTcArgs &) { return -1; }

}  // namespace tq
