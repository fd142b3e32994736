// Path-tracking tropical SRGEMM: the any-layout kernel (fp32 and fp64) and the TMA-pipeline kernel (fp32).
#include <cuda_runtime.h>
#include "srgemm_path.cuh"
#include "srgemm_path_tma.cuh"
namespace cuasr_b200 {
template <typename T>
cudaError_t launch_path(const PathParams<T>& p, bool maximize, cudaStream_t stream) {
  const long long tiles_m = (p.M + kPathTile - 1) / kPathTile, tiles_n = (p.N + kPathTile - 1) / kPathTile;
  if (tiles_m * tiles_n > 2147483647LL) return cudaErrorInvalidValue;
  PathParams<T> q = p;
  q.tiles_n = static_cast<int>(tiles_n);
  const unsigned grid = static_cast<unsigned>(tiles_m * tiles_n);
  if (maximize) srgemm_path_kernel<T, true><<<grid, kPathThreads, 0, stream>>>(q);
  else          srgemm_path_kernel<T, false><<<grid, kPathThreads, 0, stream>>>(q);
  return cudaGetLastError();
}
template <bool kMaximize, bool kAK, bool kBK>
static cudaError_t launch_path_tma_variant(const CUtensorMap& map_a, const CUtensorMap& map_b, const PathTmaParams& params,
                                           int grid, cudaStream_t stream) {
  auto kernel = srgemm_path_tma_kernel<kMaximize, kAK, kBK>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPathTmaSmemBytes);
  if (err != cudaSuccess) return err;
  kernel<<<grid, kTmaThreads, kPathTmaSmemBytes, stream>>>(map_a, map_b, params);
  return cudaGetLastError();
}
template <bool kMaximize>
static cudaError_t launch_path_tma_layouts(bool a_kcontig, bool b_kcontig, const CUtensorMap& map_a,
                                           const CUtensorMap& map_b, const PathTmaParams& params, int grid,
                                           cudaStream_t stream) {
  if (a_kcontig)
    return b_kcontig ? launch_path_tma_variant<kMaximize, true, true>(map_a, map_b, params, grid, stream)
                     : launch_path_tma_variant<kMaximize, true, false>(map_a, map_b, params, grid, stream);
  return b_kcontig ? launch_path_tma_variant<kMaximize, false, true>(map_a, map_b, params, grid, stream)
                   : launch_path_tma_variant<kMaximize, false, false>(map_a, map_b, params, grid, stream);
}
cudaError_t launch_path_tma(bool maximize, bool a_kcontig, bool b_kcontig, const CUtensorMap& map_a,
                            const CUtensorMap& map_b, const PathTmaParams& params, int grid, cudaStream_t stream) {
  return maximize ? launch_path_tma_layouts<true>(a_kcontig, b_kcontig, map_a, map_b, params, grid, stream)
                  : launch_path_tma_layouts<false>(a_kcontig, b_kcontig, map_a, map_b, params, grid, stream);
}
template cudaError_t launch_path<float>(const PathParams<float>&, bool, cudaStream_t);
template cudaError_t launch_path<double>(const PathParams<double>&, bool, cudaStream_t);
}  // namespace cuasr_b200
