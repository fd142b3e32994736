// fp64 min-max and max-min (bottleneck / capacity) rings on the TMA kernel.
#include "srgemm_launch_impl.cuh"
namespace cuasr_b200 {
CUASR_INSTANTIATE_TMA(CUASR_OP_MINIMUM, CUASR_OP_MAXIMUM, double)
CUASR_INSTANTIATE_TMA(CUASR_OP_MAXIMUM, CUASR_OP_MINIMUM, double)
}  // namespace cuasr_b200
