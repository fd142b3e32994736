// Tropical (min-plus, max-plus) and bottleneck (min-max, max-min) rings over 32-bit integers on the TMA kernel.
// Integers have no NaN to pad a ragged K with, so these run here only when K is a multiple of the K step.
#include "srgemm_launch_impl.cuh"
namespace cuasr_b200 {
CUASR_INSTANTIATE_TMA(CUASR_OP_MINIMUM, CUASR_OP_PLUS, int32_t)
CUASR_INSTANTIATE_TMA(CUASR_OP_MAXIMUM, CUASR_OP_PLUS, int32_t)
CUASR_INSTANTIATE_TMA(CUASR_OP_MINIMUM, CUASR_OP_MAXIMUM, int32_t)
CUASR_INSTANTIATE_TMA(CUASR_OP_MAXIMUM, CUASR_OP_MINIMUM, int32_t)
}  // namespace cuasr_b200
