// Host-side launchers of the SRGEMM kernels, one template per kernel family.  The definitions live in
// srgemm_launch_impl.cuh and are instantiated explicitly, ring by ring, in the inst_*.cu files so that
// the rings compile in parallel; abi.cu only sees these declarations.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "srgemm_generic.cuh"
#include "srgemm_tma.cuh"

namespace cuasr_b200 {

// Launches srgemm_tma_kernel<Ring<ADD, MUL, T>, a_kcontig, b_kcontig> on `grid` persistent CTAs.
template <int ADD, int MUL, typename T>
cudaError_t launch_tma(bool a_kcontig, bool b_kcontig, const CUtensorMap& map_a, const CUtensorMap& map_b,
                       const TmaParams<T>& params, int grid, cudaStream_t stream);

// Which (ring, element type) pairs have the TMA kernel compiled in (see the inst_tma_*.cu files); every
// other supported pair runs on the generic kernel.
template <int ADD, int MUL, typename T>
constexpr bool tma_instantiated() {
  constexpr bool tropical = (ADD == CUASR_OP_MINIMUM || ADD == CUASR_OP_MAXIMUM) && MUL == CUASR_OP_PLUS;
  constexpr bool minmax = (ADD == CUASR_OP_MINIMUM && MUL == CUASR_OP_MAXIMUM) ||
                          (ADD == CUASR_OP_MAXIMUM && MUL == CUASR_OP_MINIMUM);
  constexpr bool times = (ADD == CUASR_OP_MINIMUM || ADD == CUASR_OP_MAXIMUM || ADD == CUASR_OP_PLUS) &&
                         MUL == CUASR_OP_MULTIPLIES;
  constexpr bool bits = (ADD == CUASR_OP_BIT_XOR || ADD == CUASR_OP_BIT_OR) &&
                        (MUL == CUASR_OP_BIT_AND || MUL == CUASR_OP_BINARY_AND) &&
                        !(ADD == CUASR_OP_BIT_OR && MUL == CUASR_OP_BINARY_AND);
  if (std::is_same<T, float>::value) return tropical || minmax || times;
  if (std::is_same<T, double>::value) return tropical || minmax || times;
  return bits || tropical || minmax;  // int32_t, uint32_t
}

// Launches srgemm_generic_kernel<Ring<ADD, MUL, T>> on a (ceil(N/64), ceil(M/64), slices) grid.
template <int ADD, int MUL, typename T>
cudaError_t launch_generic(const GenericParams<T>& params, int slices, cudaStream_t stream);

// Second step of a split-K run on the generic kernel: D = epilogue((+) over slices of partial), the work of
// the reference's ReduceSplitK (include/cuasr/reduction/kernel/reduce_split_k.h:162-236).
template <int ADD, int MUL, typename T>
cudaError_t launch_generic_reduce(const GenericParams<T>& params, int slices, cudaStream_t stream);

// Copies a rows x K operand of 4- or 8-byte elements, K-contiguous or MN-contiguous with any leading dimension and
// alignment, into K-contiguous storage with leading dimension ld_dst; columns K .. K_out - 1 of the copy are set to
// the element whose bits are `pad_bits` (see repack_to_kcontig_kernel).
cudaError_t launch_repack(const void* src, long long ld_src, bool src_kcontig, int rows, int K, int K_out,
                          unsigned long long pad_bits, void* dst, long long ld_dst, size_t element_bytes,
                          cudaStream_t stream);

}  // namespace cuasr_b200
