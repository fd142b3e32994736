// SRGEMM for functor types the library has no operator code for.
//
// The reference accepts ANY pair of functors as its AdditionOp / MultiplicationOp template arguments
// (include/cuasr/gemm/device/srgemm.h:28-84; the contract a user functor has to meet is shown at
// examples/01_userdefined_semiring/userdefined_semiring.cu:56-99: a host-device operator()(T, T const&) and the
// constants Identity / Annihilator) and calls them from its kernel (include/cuasr/arch/srmma.h:84-91).  The
// prebuilt library only knows a fixed set of operators, so a functor outside that set is compiled into a kernel
// right here, in the translation unit of the caller, exactly as the reference does with every functor.
//
// The kernel is a plain shared-memory tiled one (64 x 64 outputs per CTA, 4 x 4 per thread, 16 k per stage):
// it cannot know anything about the operators, so there are no fused or packed instruction forms to use.  It
// honours the same contract as the library path: accumulators start at AdditionOp::Identity, products enter in
// ascending k as add(mult(a, b), accumulator) like the host SRGEMM
// (tools/include/cuasr/reference/srgemm/host_srgemm.h:75-91), the epilogue is
// add(mult(alpha, accumulator), mult(beta, C)) and C is not read when mult(beta, MultiplicationOp::Identity)
// equals AdditionOp::Identity (include/cuasr/gemm/epilogue/thread/semiring_linear_combination.h:118-125).
// Any layout, leading dimension and alignment; C may alias D.  Split-K slice counts are accepted and the
// contraction is done in one pass (for an associative (+) the result is the same).
//
// Only a CUDA compiler can read this file; a host-only translation unit sees nothing of it.
#pragma once

#if defined(__CUDACC__)

#include <cuda_runtime.h>

namespace cuasr {
namespace gemm {
namespace device {
namespace detail {

template <typename T>
struct UserFunctorParams {
  int M, N, K;
  const T* A;  long long a_row, a_col;   // element (m, k) at A[m * a_row + k * a_col]
  const T* B;  long long b_row, b_col;   // element (k, n) at B[k * b_row + n * b_col]
  const T* C;  long long c_row, c_col;   // may alias D; may be null when !read_c
  T* D;        long long d_row, d_col;
  T alpha, beta, add_identity;
  int read_c;
  int tiles_n;                            // tiles along N; the tile index is linear in blockIdx.x
};

constexpr int kUserTile = 64;
constexpr int kUserK = 16;
constexpr int kUserThreads = 256;

template <typename AdditionOp, typename MultiplicationOp, typename T>
__global__ void __launch_bounds__(kUserThreads) user_functor_srgemm_kernel(UserFunctorParams<T> p) {
  __shared__ T As[kUserK][kUserTile + 1];
  __shared__ T Bs[kUserK][kUserTile + 1];
  AdditionOp add_op;
  MultiplicationOp mult_op;

  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int tile_m = blockIdx.x / p.tiles_n, tile_n = blockIdx.x % p.tiles_n;
  const int m0 = tile_m * kUserTile, n0 = tile_n * kUserTile;

  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = p.add_identity;

  for (int k0 = 0; k0 < p.K; k0 += kUserK) {
    const int kt = min(kUserK, p.K - k0);
    for (int e = tid; e < kUserK * kUserTile; e += kUserThreads) {
      // the contiguous dimension of each operand varies fastest across threads
      int kk, mm, nn;
      if (p.a_col == 1) { kk = e % kUserK; mm = e / kUserK; } else { mm = e % kUserTile; kk = e / kUserTile; }
      if (kk < kt && m0 + mm < p.M) As[kk][mm] = p.A[(long long)(m0 + mm) * p.a_row + (long long)(k0 + kk) * p.a_col];
      if (p.b_row == 1) { kk = e % kUserK; nn = e / kUserK; } else { nn = e % kUserTile; kk = e / kUserTile; }
      if (kk < kt && n0 + nn < p.N) Bs[kk][nn] = p.B[(long long)(k0 + kk) * p.b_row + (long long)(n0 + nn) * p.b_col];
    }
    __syncthreads();
    for (int kk = 0; kk < kt; ++kk) {
      T a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty + 16 * i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = add_op(mult_op(a[i], b[j]), acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty + 16 * i;
    if (m >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx + 16 * j;
      if (n >= p.N) continue;
      T v = mult_op(p.alpha, acc[i][j]);
      if (p.read_c) v = add_op(v, mult_op(p.beta, p.C[(long long)m * p.c_row + (long long)n * p.c_col]));
      p.D[(long long)m * p.d_row + (long long)n * p.d_col] = v;
    }
  }
}

// Launches the kernel above.  Status numbers are cutlass::Status values (0 success, 4 invalid problem,
// 7 internal error); the launch is asynchronous on `stream` like every other path.
template <typename AdditionOp, typename MultiplicationOp, typename T>
inline int run_user_functor_srgemm(int m, int n, int k, const T* A, long long lda, bool a_row_major, const T* B,
                                   long long ldb, bool b_row_major, const T* C, long long ldc, T* D, long long ldd,
                                   bool c_row_major, T alpha, T beta, cudaStream_t stream) {
  if (m <= 0 || n <= 0 || k <= 0 || A == nullptr || B == nullptr || D == nullptr) return 4;
  AdditionOp add_op;
  MultiplicationOp mult_op;
  (void)add_op;
  UserFunctorParams<T> p;
  p.M = m; p.N = n; p.K = k;
  p.A = A; p.a_row = a_row_major ? lda : 1; p.a_col = a_row_major ? 1 : lda;
  p.B = B; p.b_row = b_row_major ? ldb : 1; p.b_col = b_row_major ? 1 : ldb;
  p.C = C; p.c_row = c_row_major ? ldc : 1; p.c_col = c_row_major ? 1 : ldc;
  p.D = D; p.d_row = c_row_major ? ldd : 1; p.d_col = c_row_major ? 1 : ldd;
  p.alpha = alpha; p.beta = beta;
  p.add_identity = AdditionOp::Identity;
  p.read_c = !(mult_op(beta, MultiplicationOp::Identity) == AdditionOp::Identity);
  if (p.read_c && C == nullptr) return 4;
  const long long tiles_m = (m + kUserTile - 1) / kUserTile, tiles_n = (n + kUserTile - 1) / kUserTile;
  if (tiles_m * tiles_n > 2147483647LL) return 4;
  p.tiles_n = static_cast<int>(tiles_n);
  user_functor_srgemm_kernel<AdditionOp, MultiplicationOp, T>
      <<<static_cast<unsigned>(tiles_m * tiles_n), kUserThreads, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 7;
}

}  // namespace detail
}  // namespace device
}  // namespace gemm
}  // namespace cuasr

#endif  // __CUDACC__
