// Functors the library has no operator code for, through the drop-in templates: the reference compiles whatever
// AdditionOp / MultiplicationOp it is given (include/cuasr/gemm/device/srgemm.h:28-84, functor contract at
// examples/01_userdefined_semiring/userdefined_semiring.cu:56-99).  Every case below runs the reference's test-bed
// grid (test/device/testbed.h:313-319: M in {1, 509}, N in {1, 510}, K in {1, 23}) in all eight layout combinations
// and compares with a host loop that calls the same functor objects, value for value.
// Exit code 0 = every check passed.
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include <cuda_runtime.h>

#include "cuasr/functional.h"
#include "cuasr/gemm/device/srgemm.h"
#include "cuasr/gemm/device/srgemm_splitk_parallel.h"

using ColumnMajor = cutlass::layout::ColumnMajor;
using RowMajor = cutlass::layout::RowMajor;

#define CHECK_CUDA(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::printf("CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__); std::exit(2); } } while (0)

// (x) of a tropical ring over bounded path lengths: sums saturate at a cap instead of overflowing.  It agrees with
// plain plus on small values, which is exactly why it must not be mistaken for it.
template <typename T>
struct saturating_plus {
  static constexpr T Identity = static_cast<T>(0);
  static constexpr T Annihilator = static_cast<T>(100);
  __host__ __device__ T operator()(T lhs, T const& rhs) const {
    T s = lhs + rhs;
    return s < static_cast<T>(100) ? s : static_cast<T>(100);
  }
};
// a minimum written by the user: no operator code, but it behaves like the built-in one everywhere
template <typename T>
struct user_minimum {
  static constexpr T Identity = static_cast<T>(100);
  static constexpr T Annihilator = static_cast<T>(-100);
  __host__ __device__ T operator()(T lhs, T const& rhs) const { return rhs < lhs ? rhs : lhs; }
};
// (x) that is not commutative: the operand order of every call matters
template <typename T>
struct left_shifted_sum {
  static constexpr T Identity = static_cast<T>(0);
  static constexpr T Annihilator = static_cast<T>(0);
  __host__ __device__ T operator()(T lhs, T const& rhs) const { return static_cast<T>(2) * lhs + rhs; }
};

template <typename T>
static T* to_device(std::vector<T> const& h) {
  T* d = nullptr;
  CHECK_CUDA(cudaMalloc(&d, h.size() * sizeof(T)));
  CHECK_CUDA(cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice));
  return d;
}

template <typename Layout>
static long long offset(int r, int c, int ld) {
  return std::is_same<Layout, RowMajor>::value ? static_cast<long long>(r) * ld + c : static_cast<long long>(c) * ld + r;
}
template <typename Layout>
static int lead(int rows, int cols, int pad) {
  return (std::is_same<Layout, RowMajor>::value ? cols : rows) + pad;
}
template <typename Layout>
static size_t extent(int rows, int cols, int ld) {
  return static_cast<size_t>(ld) * (std::is_same<Layout, RowMajor>::value ? rows : cols);
}

template <typename Gemm>
static int one_case(int M, int N, int K, int slices, std::mt19937_64& rng, const char* what) {
  using T = typename Gemm::ElementC;
  using Add = typename Gemm::AdditionOp;
  using Mul = typename Gemm::MultiplicationOp;
  using LA = typename Gemm::LayoutA;
  using LB = typename Gemm::LayoutB;
  using LC = typename Gemm::LayoutC;
  const int lda = lead<LA>(M, K, 3), ldb = lead<LB>(K, N, 1), ldc = lead<LC>(M, N, 2);
  std::uniform_int_distribution<int> dist(-8, 8);       // the test bed's data: test/device/testbed.h:85-108
  std::vector<T> A(extent<LA>(M, K, lda)), B(extent<LB>(K, N, ldb)), C(extent<LC>(M, N, ldc));
  for (auto& v : A) v = static_cast<T>(dist(rng));
  for (auto& v : B) v = static_cast<T>(dist(rng));
  for (auto& v : C) v = static_cast<T>(dist(rng));
  const T alpha = Mul::Identity, beta = Mul::Identity;   // C takes part
  Add add;
  Mul mul;
  std::vector<T> want = C;
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      T acc = Add::Identity;
      for (int k = 0; k < K; ++k) acc = add(mul(A[offset<LA>(m, k, lda)], B[offset<LB>(k, n, ldb)]), acc);
      want[offset<LC>(m, n, ldc)] = add(mul(alpha, acc), mul(beta, C[offset<LC>(m, n, ldc)]));
    }
  T *dA = to_device(A), *dB = to_device(B), *dC = to_device(C), *dD = to_device(C);
  typename Gemm::Arguments args({M, N, K}, {dA, lda}, {dB, ldb}, {dC, ldc}, {dD, ldc}, {alpha, beta}, slices);
  Gemm gemm;
  void* ws = nullptr;
  size_t need = Gemm::get_workspace_size(args);
  if (need) CHECK_CUDA(cudaMalloc(&ws, need));
  cutlass::Status st = gemm(args, ws);
  CHECK_CUDA(cudaDeviceSynchronize());
  std::vector<T> got(C.size());
  CHECK_CUDA(cudaMemcpy(got.data(), dD, got.size() * sizeof(T), cudaMemcpyDeviceToHost));
  cudaFree(dA); cudaFree(dB); cudaFree(dC); cudaFree(dD); cudaFree(ws);
  const bool ok = st == cutlass::Status::kSuccess && got == want;     // padding elements included: they must stay
  if (!ok) std::printf("FAILED %s %dx%dx%d slices=%d status=%d\n", what, M, N, K, slices, static_cast<int>(st));
  return ok ? 0 : 1;
}

template <typename Gemm>
static int grid(std::mt19937_64& rng, const char* what, int slices = 1) {
  int bad = 0;
  for (int M : {1, 509})
    for (int N : {1, 510})
      for (int K : {1, 23}) bad += one_case<Gemm>(M, N, K, slices, rng, what);
  bad += one_case<Gemm>(130, 70, 300, slices, rng, what);            // several K stages, several tiles
  return bad;
}

template <typename Add, typename Mul, typename T>
static int all_layouts(std::mt19937_64& rng, const char* what) {
  using namespace cuasr::gemm::device;
  int bad = 0;
  bad += grid<Srgemm<Add, Mul, T, ColumnMajor, T, ColumnMajor, T, ColumnMajor>>(rng, what);
  bad += grid<Srgemm<Add, Mul, T, ColumnMajor, T, ColumnMajor, T, RowMajor>>(rng, what);
  bad += grid<Srgemm<Add, Mul, T, ColumnMajor, T, RowMajor, T, ColumnMajor>>(rng, what);
  bad += grid<Srgemm<Add, Mul, T, ColumnMajor, T, RowMajor, T, RowMajor>>(rng, what);
  bad += grid<Srgemm<Add, Mul, T, RowMajor, T, ColumnMajor, T, ColumnMajor>>(rng, what);
  bad += grid<Srgemm<Add, Mul, T, RowMajor, T, ColumnMajor, T, RowMajor>>(rng, what);
  bad += grid<Srgemm<Add, Mul, T, RowMajor, T, RowMajor, T, ColumnMajor>>(rng, what);
  bad += grid<Srgemm<Add, Mul, T, RowMajor, T, RowMajor, T, RowMajor>>(rng, what);
  std::printf("%s: %s\n", what, bad == 0 ? "ok" : "FAILED");
  return bad;
}

int main() {
  int failures = 0;
  std::mt19937_64 rng(2080);
  // the probe must not take the saturating sum for plus, and must still recognise the hand-written minimum
  bool probe_ok = cuasr::OpCodeOf<saturating_plus<float>, float>::get() == -1 &&
                  cuasr::OpCodeOf<saturating_plus<int>, int>::get() == -1 &&
                  cuasr::OpCodeOf<left_shifted_sum<int>, int>::get() == -1 &&
                  cuasr::OpCodeOf<user_minimum<float>, float>::get() == CUASR_OP_MINIMUM;
  std::printf("operator probe: %s\n", probe_ok ? "ok" : "FAILED");
  failures += !probe_ok;
  // a library functor paired with a user functor, two user functors, and a non-commutative (x)
  failures += all_layouts<cuasr::minimum<float>, saturating_plus<float>, float>(rng, "minimum / saturating_plus float");
  failures += all_layouts<user_minimum<double>, saturating_plus<double>, double>(rng, "user_minimum / saturating_plus double");
  failures += all_layouts<user_minimum<int>, saturating_plus<int>, int>(rng, "user_minimum / saturating_plus int");
  failures += all_layouts<cuasr::maximum<int>, left_shifted_sum<int>, int>(rng, "maximum / left_shifted_sum int");
  {  // the split-K template with the same functors: slice counts are accepted, the result is the single-pass one
    using namespace cuasr::gemm::device;
    int bad = grid<SrgemmSplitKParallel<cuasr::minimum<float>, saturating_plus<float>, float, RowMajor, float, ColumnMajor,
                                        float, RowMajor>>(rng, "split-K minimum / saturating_plus", 4);
    std::printf("split-K minimum / saturating_plus float: %s\n", bad == 0 ? "ok" : "FAILED");
    failures += bad;
  }
  std::printf("%s\n", failures == 0 ? "ALL OK" : "FAILURES");
  return failures == 0 ? 0 : 1;
}
