// Definitions of the launchers declared in srgemm_launch.h; included only by the inst_*.cu files.
#pragma once

#include "srgemm_launch.h"

namespace cuasr_b200 {

template <typename RingT, bool kAK, bool kBK>
cudaError_t launch_tma_variant(const CUtensorMap& map_a, const CUtensorMap& map_b,
                               const TmaParams<typename RingT::Element>& params, int grid, cudaStream_t stream) {
  auto kernel = srgemm_tma_kernel<RingT, kAK, kBK>;
  // more than 48 KiB of dynamic shared memory has to be opted into, once per kernel and device
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTmaSmemBytes);
  if (err != cudaSuccess) return err;
  kernel<<<grid, kTmaThreads, kTmaSmemBytes, stream>>>(map_a, map_b, params);
  return cudaGetLastError();
}

template <int ADD, int MUL, typename T>
cudaError_t launch_tma(bool a_kcontig, bool b_kcontig, const CUtensorMap& map_a, const CUtensorMap& map_b,
                       const TmaParams<T>& params, int grid, cudaStream_t stream) {
  using R = Ring<ADD, MUL, T>;
  if (a_kcontig) {
    return b_kcontig ? launch_tma_variant<R, true, true>(map_a, map_b, params, grid, stream)
                     : launch_tma_variant<R, true, false>(map_a, map_b, params, grid, stream);
  }
  return b_kcontig ? launch_tma_variant<R, false, true>(map_a, map_b, params, grid, stream)
                   : launch_tma_variant<R, false, false>(map_a, map_b, params, grid, stream);
}

template <int ADD, int MUL, typename T>
cudaError_t launch_generic(const GenericParams<T>& params, int slices, cudaStream_t stream) {
  const long long tiles_m = (params.M + kGenTile - 1) / kGenTile, tiles_n = (params.N + kGenTile - 1) / kGenTile;
  if (tiles_m * tiles_n > 2147483647LL || slices > 65535) return cudaErrorInvalidValue;
  GenericParams<T> p = params;
  p.tiles_n = static_cast<int>(tiles_n);
  dim3 grid(static_cast<unsigned>(tiles_m * tiles_n), 1, slices);
  srgemm_generic_kernel<Ring<ADD, MUL, T>><<<grid, kGenThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

template <int ADD, int MUL, typename T>
cudaError_t launch_generic_reduce(const GenericParams<T>& params, int slices, cudaStream_t stream) {
  const long long total = static_cast<long long>(params.M) * params.N;
  if ((total + 255) / 256 > 2147483647LL) return cudaErrorInvalidValue;
  const int blocks = static_cast<int>((total + 255) / 256);
  splitk_reduce_kernel<Ring<ADD, MUL, T>><<<blocks, 256, 0, stream>>>(params, slices);
  return cudaGetLastError();
}

#define CUASR_INSTANTIATE_TMA(ADD, MUL, T)                                                                   \
  template cudaError_t launch_tma<ADD, MUL, T>(bool, bool, const CUtensorMap&, const CUtensorMap&,           \
                                               const TmaParams<T>&, int, cudaStream_t);
#define CUASR_INSTANTIATE_GENERIC(ADD, MUL, T) \
  template cudaError_t launch_generic<ADD, MUL, T>(const GenericParams<T>&, int, cudaStream_t);  \
  template cudaError_t launch_generic_reduce<ADD, MUL, T>(const GenericParams<T>&, int, cudaStream_t);

}  // namespace cuasr_b200
