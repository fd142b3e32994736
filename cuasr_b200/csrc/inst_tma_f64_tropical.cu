// fp64 min-plus and max-plus (tropical) rings on the TMA kernel.
#include "srgemm_launch_impl.cuh"
namespace cuasr_b200 {
CUASR_INSTANTIATE_TMA(CUASR_OP_MINIMUM, CUASR_OP_PLUS, double)
CUASR_INSTANTIATE_TMA(CUASR_OP_MAXIMUM, CUASR_OP_PLUS, double)
}  // namespace cuasr_b200
