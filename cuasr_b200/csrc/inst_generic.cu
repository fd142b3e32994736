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
cudaError_t launch_repack(const void* src, long long ld_src, bool src_kcontig, int rows, int K, int K_out,
                          unsigned long long pad_bits, void* dst, long long ld_dst, size_t element_bytes,
                          cudaStream_t stream) {
  const long long tiles_r = (rows + 31) / 32, tiles_k = (K_out + 31) / 32;
  if (tiles_r * tiles_k > 2147483647LL) return cudaErrorInvalidValue;
  const unsigned grid = static_cast<unsigned>(tiles_r * tiles_k);
  if (element_bytes == 8)
    repack_to_kcontig_kernel<unsigned long long><<<grid, 256, 0, stream>>>(
        static_cast<const unsigned long long*>(src), ld_src, src_kcontig, rows, K, K_out, pad_bits,
        static_cast<unsigned long long*>(dst), ld_dst, static_cast<int>(tiles_r));
  else
    repack_to_kcontig_kernel<unsigned int><<<grid, 256, 0, stream>>>(
        static_cast<const unsigned int*>(src), ld_src, src_kcontig, rows, K, K_out, static_cast<unsigned int>(pad_bits),
        static_cast<unsigned int*>(dst), ld_dst, static_cast<int>(tiles_r));
  return cudaGetLastError();
}
}  // namespace cuasr_b200
