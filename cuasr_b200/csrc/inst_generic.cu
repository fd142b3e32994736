// Every supported ring on the generic (any alignment, any shape) kernel.
#include "srgemm_launch_impl.cuh"
namespace cuasr_b200 {
#define CUASR_ALL_TYPES(ADD, MUL)              \
  CUASR_INSTANTIATE_GENERIC(ADD, MUL, float)   \
  CUASR_INSTANTIATE_GENERIC(ADD, MUL, double)  \
  CUASR_INSTANTIATE_GENERIC(ADD, MUL, int32_t) \
  CUASR_INSTANTIATE_GENERIC(ADD, MUL, uint32_t)
#define CUASR_INT_TYPES(ADD, MUL)              \
  CUASR_INSTANTIATE_GENERIC(ADD, MUL, int32_t) \
  CUASR_INSTANTIATE_GENERIC(ADD, MUL, uint32_t)
CUASR_ALL_TYPES(CUASR_OP_PLUS, CUASR_OP_MULTIPLIES)
CUASR_ALL_TYPES(CUASR_OP_MINIMUM, CUASR_OP_PLUS)
CUASR_ALL_TYPES(CUASR_OP_MAXIMUM, CUASR_OP_PLUS)
CUASR_ALL_TYPES(CUASR_OP_MINIMUM, CUASR_OP_MAXIMUM)
CUASR_ALL_TYPES(CUASR_OP_MAXIMUM, CUASR_OP_MINIMUM)
CUASR_ALL_TYPES(CUASR_OP_MINIMUM, CUASR_OP_MULTIPLIES)
CUASR_ALL_TYPES(CUASR_OP_MAXIMUM, CUASR_OP_MULTIPLIES)
CUASR_ALL_TYPES(CUASR_OP_BINARY_OR, CUASR_OP_BINARY_AND)
CUASR_INT_TYPES(CUASR_OP_BIT_XOR, CUASR_OP_BIT_AND)
CUASR_INT_TYPES(CUASR_OP_BIT_OR, CUASR_OP_BIT_AND)
CUASR_INT_TYPES(CUASR_OP_BIT_XOR, CUASR_OP_BINARY_AND)
cudaError_t launch_transpose_f32(const float* src, long long ld_src, int rows, int K, float* dst, long long ld_dst,
                                 cudaStream_t stream) {
  dim3 grid((rows + 31) / 32, (K + 31) / 32);
  transpose_to_kcontig_kernel<float><<<grid, 256, 0, stream>>>(src, ld_src, rows, K, dst, ld_dst);
  return cudaGetLastError();
}
}  // namespace cuasr_b200
