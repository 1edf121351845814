// W4A4 prefill GEMM (placeholder until the tcgen05 kernel lands).
#include "engine.h"

namespace q35b {
int launch_gemm_w4a4(q35b_weight *, const uint8_t *, const uint8_t *, const float *, int, void *, int, unsigned int *,
                     cudaStream_t) {
  return fail(Q35B_ERR_SHAPE, "W4A4 GEMM is not built into this library.");
}
}  // namespace q35b
