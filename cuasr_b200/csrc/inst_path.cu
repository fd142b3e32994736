// Path-tracking tropical SRGEMM, fp32 and fp64.
#include <cuda_runtime.h>
#include "srgemm_path.cuh"
namespace cuasr_b200 {
template <typename T>
cudaError_t launch_path(const PathParams<T>& p, bool maximize, cudaStream_t stream) {
  dim3 grid((p.N + kPathTile - 1) / kPathTile, (p.M + kPathTile - 1) / kPathTile);
  if (maximize) srgemm_path_kernel<T, true><<<grid, kPathThreads, 0, stream>>>(p);
  else          srgemm_path_kernel<T, false><<<grid, kPathThreads, 0, stream>>>(p);
  return cudaGetLastError();
}
template cudaError_t launch_path<float>(const PathParams<float>&, bool, cudaStream_t);
template cudaError_t launch_path<double>(const PathParams<double>&, bool, cudaStream_t);
}  // namespace cuasr_b200
