// fp64 plus-times (ordinary GEMM), min-times and max-times rings on the TMA kernel.
#include "srgemm_launch_impl.cuh"
namespace cuasr_b200 {
CUASR_INSTANTIATE_TMA(CUASR_OP_PLUS, CUASR_OP_MULTIPLIES, double)
CUASR_INSTANTIATE_TMA(CUASR_OP_MINIMUM, CUASR_OP_MULTIPLIES, double)
CUASR_INSTANTIATE_TMA(CUASR_OP_MAXIMUM, CUASR_OP_MULTIPLIES, double)
}  // namespace cuasr_b200
