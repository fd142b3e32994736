// Path-tracking tropical SRGEMM: distances AND the contraction index that produced them.
//
// Device counterpart of the reference's legacy CPU routine cpu_fwgemm_naive
// (test/regress/include/fwgpu/cpu_srgemm.hpp:20-48): dist[m, n] = min(dist[m, n], min_k A[m, k] + B[k, n]) and
// parent[m, n] = the k that gave the strictly best product (first such k; untouched when nothing improved).
// Every output element is owned by one thread that walks k in ascending order, so "first k" needs no tie-break
// between threads.  Any layout and alignment (element loads through strides), min-plus or max-plus, fp32 or fp64.
#pragma once

#include <cstdint>

namespace cuasr_b200 {

template <typename T>
struct PathParams {
  int M, N, K;
  const T* A;  long long a_row, a_col;     // A(m, k) at A[m * a_row + k * a_col]
  const T* B;  long long b_row, b_col;     // B(k, n) at B[k * b_row + n * b_col]
  T* dist;     long long d_row, d_col;     // in/out
  int32_t* parent; long long p_row, p_col; // in/out
  int k_offset;                            // added to the recorded k
  int tiles_n;                             // tiles along N; the tile index runs along grid.x
};

constexpr int kPathTile = 64;
constexpr int kPathK = 16;
constexpr int kPathThreads = 256;

template <typename T, bool kMaximize>
__global__ void __launch_bounds__(kPathThreads)
srgemm_path_kernel(PathParams<T> p) {
  __shared__ T As[kPathK][kPathTile + 1];
  __shared__ T Bs[kPathK][kPathTile + 1];
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int m0 = (blockIdx.x / p.tiles_n) * kPathTile, n0 = (blockIdx.x % p.tiles_n) * kPathTile;

  T acc[4][4];
  int32_t idx[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + ty + 16 * i, n = n0 + tx + 16 * j;
      const bool in = m < p.M && n < p.N;
      acc[i][j] = in ? p.dist[m * p.d_row + n * p.d_col] : T(0);
      idx[i][j] = in ? p.parent[m * p.p_row + n * p.p_col] : 0;
    }

  for (int k0 = 0; k0 < p.K; k0 += kPathK) {
    const int kt = min(kPathK, p.K - k0);
    for (int e = tid; e < kPathK * kPathTile; e += kPathThreads) {
      int kk, mm, nn;
      if (p.a_col == 1) { kk = e % kPathK; mm = e / kPathK; } else { mm = e % kPathTile; kk = e / kPathTile; }
      if (kk < kt && m0 + mm < p.M) As[kk][mm] = p.A[(long long)(m0 + mm) * p.a_row + (long long)(k0 + kk) * p.a_col];
      if (p.b_row == 1) { kk = e % kPathK; nn = e / kPathK; } else { nn = e % kPathTile; kk = e / kPathTile; }
      if (kk < kt && n0 + nn < p.N) Bs[kk][nn] = p.B[(long long)(k0 + kk) * p.b_row + (long long)(n0 + nn) * p.b_col];
    }
    __syncthreads();
    for (int kk = 0; kk < kt; ++kk) {
      T a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty + 16 * i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx + 16 * j];
      const int32_t k = k0 + kk + p.k_offset;
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const T t = a[i] + b[j];
          const bool better = kMaximize ? (acc[i][j] < t) : (t < acc[i][j]);
          acc[i][j] = better ? t : acc[i][j];
          idx[i][j] = better ? k : idx[i][j];
        }
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + ty + 16 * i, n = n0 + tx + 16 * j;
      if (m < p.M && n < p.N) {
        p.dist[m * p.d_row + n * p.d_col] = acc[i][j];
        p.parent[m * p.p_row + n * p.p_col] = idx[i][j];
      }
    }
}

template <typename T>
cudaError_t launch_path(const PathParams<T>& p, bool maximize, cudaStream_t stream);

}  // namespace cuasr_b200
