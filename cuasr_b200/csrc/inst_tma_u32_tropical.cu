// Tropical (min-plus, max-plus) and bottleneck (min-max, max-min) rings over unsigned 32-bit integers on the TMA
// kernel (only when K is a multiple of the K step: there is no padding value for them).
#include "srgemm_launch_impl.cuh"
namespace cuasr_b200 {
CUASR_INSTANTIATE_TMA(CUASR_OP_MINIMUM, CUASR_OP_PLUS, uint32_t)
CUASR_INSTANTIATE_TMA(CUASR_OP_MAXIMUM, CUASR_OP_PLUS, uint32_t)
CUASR_INSTANTIATE_TMA(CUASR_OP_MINIMUM, CUASR_OP_MAXIMUM, uint32_t)
CUASR_INSTANTIATE_TMA(CUASR_OP_MAXIMUM, CUASR_OP_MINIMUM, uint32_t)
}  // namespace cuasr_b200
