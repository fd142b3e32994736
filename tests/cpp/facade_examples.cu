// The three BLAS-style wrappers of the reference's examples, written against this library's drop-in headers
// and checked against naive host loops:
//   examples/00_minplus_srgemm/minplus_srgemm.cu:9-81           cuasr_minplus_srsgemm_nt_n (C aliases D)
//   examples/01_userdefined_semiring/userdefined_semiring.cu:104-192   GF(2) SRGEMM with a user-defined xor functor
//   examples/02_splitk_srgemm/splitk_srgemm.cu:17-103           cuasr_splitk_minplus_srsgemm_tn_t
// plus an all-pairs-shortest-paths solve through the C entry points of cuasr_b200_apsp.h, from C++ alone.
// Exit code 0 = every check passed.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <limits>
#include <random>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "cuasr_b200_apsp.h"
#include "cuasr/functional.h"
#include "cuasr/gemm/device/default_srgemm_configuration.h"
#include "cuasr/gemm/device/srgemm.h"
#include "cuasr/gemm/device/srgemm_splitk_parallel.h"

using ColumnMajor = cutlass::layout::ColumnMajor;
using RowMajor = cutlass::layout::RowMajor;

#define CHECK_CUDA(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::printf("CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__); std::exit(2); } } while (0)

// ---- example 00: min-plus, A column-major, B row-major, C/D column-major -------------------------------
int cuasr_minplus_srsgemm_nt_n(int M, int N, int K, float const* A, int lda, float const* B, int ldb, float* C,
                               int ldc, float* D, bool do_epilogue_min, cudaStream_t stream = nullptr) {
  using AdditionOp = cuasr::minimum<float>;
  using MultiplicationOp = cuasr::plus<float>;
  using Gemm = cuasr::gemm::device::Srgemm<AdditionOp, MultiplicationOp, float, ColumnMajor, float, RowMajor, float,
                                           ColumnMajor, float>;
  float alpha = MultiplicationOp::Identity;
  float beta = do_epilogue_min ? MultiplicationOp::Identity : MultiplicationOp::Annihilator;
  Gemm::Arguments args({M, N, K}, {A, lda}, {B, ldb}, {C, ldc}, {D, ldc}, {alpha, beta});
  Gemm gemm;
  return static_cast<int>(gemm(args, nullptr, stream));
}

// ---- example 01: a user-defined functor joins the library by naming its operator code ------------------
namespace {
template <typename T, int N = 1>
struct binary_xor {
  static T constexpr Identity = static_cast<T>(false);
  T operator()(T lhs, T const& rhs) const { return lhs ^ rhs; }
};
}  // namespace
namespace cuasr {
template <typename T, int N>
struct OpCode<binary_xor<T, N>, void> { static constexpr int value = CUASR_OP_BIT_XOR; };
}  // namespace cuasr

int cuasr_gf_srgemm_nnn(int M, int N, int K, int const* A, int lda, int const* B, int ldb, int* C, int ldc, int* D,
                        bool do_epilogue_xor, cudaStream_t stream = nullptr) {
  using AdditionOp = binary_xor<int>;
  using MultiplicationOp = cuasr::binary_and<int>;
  using EpilogueOutputOp = cuasr::epilogue::thread::SemiringLinearCombination<AdditionOp, MultiplicationOp, int, 1>;
  using Gemm = cuasr::gemm::device::Srgemm<AdditionOp, MultiplicationOp, int, RowMajor, int, RowMajor, int, RowMajor,
                                           int, cutlass::arch::OpClassSimt, cutlass::arch::Sm50,
                                           cutlass::gemm::GemmShape<64, 128, 8>, cutlass::gemm::GemmShape<32, 64, 8>,
                                           cutlass::gemm::GemmShape<1, 1, 1>, EpilogueOutputOp>;
  int alpha = MultiplicationOp::Identity;
  int beta = do_epilogue_xor ? MultiplicationOp::Identity : MultiplicationOp::Annihilator;
  Gemm::Arguments args({M, N, K}, {A, lda}, {B, ldb}, {C, ldc}, {D, ldc}, {alpha, beta});
  Gemm gemm;
  return static_cast<int>(gemm(args, nullptr, stream));
}

// ---- example 02: parallel split-K, A row-major, B column-major, C/D row-major ---------------------------
int cuasr_splitk_minplus_srsgemm_tn_t(int M, int N, int K, float const* A, int lda, float const* B, int ldb, float* C,
                                      int ldc, float* D, bool do_epilogue_min, int split_k_slices,
                                      cudaStream_t stream = nullptr) {
  using AdditionOp = cuasr::minimum<float>;
  using MultiplicationOp = cuasr::plus<float>;
  using Gemm = cuasr::gemm::device::SrgemmSplitKParallel<AdditionOp, MultiplicationOp, float, RowMajor, float,
                                                         ColumnMajor, float, RowMajor>;
  float alpha = MultiplicationOp::Identity;
  float beta = do_epilogue_min ? MultiplicationOp::Identity : MultiplicationOp::Annihilator;
  Gemm::Arguments args({M, N, K}, {A, lda}, {B, ldb}, {C, ldc}, {D, ldc}, {alpha, beta}, split_k_slices);
  size_t workspace_size = Gemm::get_workspace_size(args);
  void* workspace = nullptr;
  CHECK_CUDA(cudaMalloc(&workspace, workspace_size));
  Gemm gemm;
  cutlass::Status status = gemm.initialize(args, workspace);
  if (status == cutlass::Status::kSuccess) status = gemm(stream);
  CHECK_CUDA(cudaDeviceSynchronize());
  CHECK_CUDA(cudaFree(workspace));
  return static_cast<int>(status);
}

template <typename T>
T* to_device(std::vector<T> const& h) {
  T* d = nullptr;
  CHECK_CUDA(cudaMalloc(&d, h.size() * sizeof(T)));
  CHECK_CUDA(cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice));
  return d;
}

int main() {
  int failures = 0;
  std::mt19937_64 rng(3090);
  {  // example 00 at 300 x 260 x 190, C aliases D, with and without the epilogue min
    int M = 300, N = 260, K = 190;
    std::uniform_real_distribution<float> dist(0.5f, 1.5f);
    std::vector<float> A(M * K), B(K * N), C(M * N);
    for (auto& v : A) v = dist(rng);
    for (auto& v : B) v = dist(rng);
    for (auto& v : C) v = dist(rng) + 0.6f;
    for (int with_c = 0; with_c < 2; ++with_c) {
      std::vector<float> want(M * N);
      for (int n = 0; n < N; ++n)
        for (int m = 0; m < M; ++m) {
          float acc = cuasr::minimum<float>::Identity;
          for (int k = 0; k < K; ++k) acc = std::min(acc, A[m + k * M] + B[k * N + n]);
          want[m + n * M] = with_c ? std::min(acc, C[m + n * M]) : acc;
        }
      float *dA = to_device(A), *dB = to_device(B), *dC = to_device(C);
      int st = cuasr_minplus_srsgemm_nt_n(M, N, K, dA, M, dB, N, dC, M, dC, with_c != 0);
      CHECK_CUDA(cudaDeviceSynchronize());
      std::vector<float> got(M * N);
      CHECK_CUDA(cudaMemcpy(got.data(), dC, got.size() * sizeof(float), cudaMemcpyDeviceToHost));
      bool ok = st == 0 && got == want;
      std::printf("minplus_srsgemm_nt_n epilogue_min=%d: %s\n", with_c, ok ? "ok" : "FAILED");
      failures += !ok;
      cudaFree(dA); cudaFree(dB); cudaFree(dC);
    }
  }
  {  // example 01: GF(2) on Bernoulli(0.025) bits, 512^3 like the reference's self-check
    int M = 512, N = 512, K = 512;
    std::bernoulli_distribution bit(0.025);
    std::vector<int> A(M * K), B(K * N), C(M * N);
    for (auto& v : A) v = bit(rng);
    for (auto& v : B) v = bit(rng);
    for (auto& v : C) v = bit(rng);
    std::vector<int> want(M * N);
    for (int m = 0; m < M; ++m)
      for (int n = 0; n < N; ++n) {
        int acc = 0;
        for (int k = 0; k < K; ++k) acc ^= (A[m * K + k] && B[k * N + n]);
        want[m * N + n] = acc ^ C[m * N + n];
      }
    int *dA = to_device(A), *dB = to_device(B), *dC = to_device(C), *dD = to_device(C);
    int st = cuasr_gf_srgemm_nnn(M, N, K, dA, K, dB, N, dC, N, dD, true);
    CHECK_CUDA(cudaDeviceSynchronize());
    std::vector<int> got(M * N);
    CHECK_CUDA(cudaMemcpy(got.data(), dD, got.size() * sizeof(int), cudaMemcpyDeviceToHost));
    bool ok = st == 0 && got == want;
    std::printf("gf_srgemm_nnn: %s\n", ok ? "ok" : "FAILED");
    failures += !ok;
  }
  {  // example 02: split-K equals the single-pass result and the host loop
    int M = 128, N = 128, K = 128 * 64;
    std::uniform_real_distribution<float> dist(0.5f, 1.5f);
    std::vector<float> A(M * K), B(K * N), C(M * N);
    for (auto& v : A) v = dist(rng);
    for (auto& v : B) v = dist(rng);
    for (auto& v : C) v = dist(rng) + 0.7f;
    std::vector<float> want(M * N);
    for (int m = 0; m < M; ++m)
      for (int n = 0; n < N; ++n) {
        float acc = cuasr::minimum<float>::Identity;
        for (int k = 0; k < K; ++k) acc = std::min(acc, A[m * K + k] + B[n * K + k]);
        want[m * N + n] = std::min(acc, C[m * N + n]);
      }
    for (int slices : {1, 4, 16}) {
      float *dA = to_device(A), *dB = to_device(B), *dC = to_device(C), *dD = to_device(C);
      int st = cuasr_splitk_minplus_srsgemm_tn_t(M, N, K, dA, K, dB, K, dC, N, dD, true, slices);
      std::vector<float> got(M * N);
      CHECK_CUDA(cudaMemcpy(got.data(), dD, got.size() * sizeof(float), cudaMemcpyDeviceToHost));
      bool ok = st == 0 && got == want;
      std::printf("splitk_minplus_srsgemm_tn_t slices=%d: %s\n", slices, ok ? "ok" : "FAILED");
      failures += !ok;
      cudaFree(dA); cudaFree(dB); cudaFree(dC); cudaFree(dD);
    }
  }
  {  // the optional workspace through the facade: same bits, the launch that uses it is reported by the library
    using Gemm = cuasr::gemm::device::Srgemm<cuasr::minimum<float>, cuasr::plus<float>, float, ColumnMajor, float,
                                             ColumnMajor, float, ColumnMajor>;
    int M = 512, N = 384, K = 512;
    std::uniform_real_distribution<float> dist(0.0f, 100.0f);
    std::vector<float> A(M * K), B(K * N), C(M * N);
    for (auto& v : A) v = dist(rng);
    for (auto& v : B) v = dist(rng);
    for (auto& v : C) v = dist(rng) + 50.0f;
    float *dA = to_device(A), *dB = to_device(B), *dC = to_device(C), *dD0 = to_device(C), *dD1 = to_device(C);
    Gemm::Arguments a0({M, N, K}, {dA, M}, {dB, K}, {dC, M}, {dD0, M}, {0.0f, 0.0f});
    Gemm::Arguments a1({M, N, K}, {dA, M}, {dB, K}, {dC, M}, {dD1, M}, {0.0f, 0.0f});
    Gemm plain, fast;
    bool ok = plain(a0) == cutlass::Status::kSuccess;
    const size_t bytes = Gemm::get_optional_workspace_size(a1);
    void* ws = nullptr;
    ok = ok && Gemm::get_workspace_size(a1) == 0 && bytes > 0;
    CHECK_CUDA(cudaMalloc(&ws, bytes));
    ok = ok && fast(a1, ws, nullptr, bytes) == cutlass::Status::kSuccess;
    const bool used = std::string(cuasr_b200_last_kernel()) != "tma";       // "tma_balanced" / "tma_repacked"
    CHECK_CUDA(cudaDeviceSynchronize());
    std::vector<float> g0(M * N), g1(M * N);
    CHECK_CUDA(cudaMemcpy(g0.data(), dD0, g0.size() * sizeof(float), cudaMemcpyDeviceToHost));
    CHECK_CUDA(cudaMemcpy(g1.data(), dD1, g1.size() * sizeof(float), cudaMemcpyDeviceToHost));
    ok = ok && used && g0 == g1;
    std::printf("optional workspace through the templates: %s\n", ok ? "ok" : "FAILED");
    failures += !ok;
    cudaFree(dA); cudaFree(dB); cudaFree(dC); cudaFree(dD0); cudaFree(dD1); cudaFree(ws);
  }
  {  // status codes through the facade
    using Gemm = cuasr::gemm::device::Srgemm<cuasr::minimum<float>, cuasr::plus<float>, float, ColumnMajor, float,
                                             ColumnMajor, float, ColumnMajor>;
    float* x = nullptr;
    CHECK_CUDA(cudaMalloc(&x, 64 * 64 * sizeof(float)));
    Gemm::Arguments split({64, 64, 64}, {x, 64}, {x, 64}, {x, 64}, {x, 64}, {0.f, 0.f}, 2);
    bool ok = Gemm::can_implement(split) == cutlass::Status::kErrorInvalidProblem;   // not a split-K-serial operator
    Gemm::Arguments empty({0, 64, 64}, {x, 64}, {x, 64}, {x, 64}, {x, 64});
    ok = ok && Gemm::can_implement(empty) == cutlass::Status::kErrorInvalidProblem;
    Gemm gemm;
    ok = ok && gemm.run() == cutlass::Status::kErrorInternal;                         // run before initialize
    std::printf("status codes: %s\n", ok ? "ok" : "FAILED");
    failures += !ok;
  }
  {  // all-pairs shortest paths from C++ through the C entry points: both algorithms against a host Floyd-Warshall
    const int n = 300, ld = 304;
    std::bernoulli_distribution edge(0.03);
    std::uniform_int_distribution<int> weight(1, 100);
    const float inf = std::numeric_limits<float>::infinity();
    std::vector<float> G(static_cast<size_t>(ld) * n, -1.0f);          // padding rows hold -1 and must stay
    for (int j = 0; j < n; ++j)
      for (int i = 0; i < n; ++i) G[i + static_cast<size_t>(j) * ld] = i == j ? 0.0f : edge(rng) ? float(weight(rng)) : inf;
    std::vector<float> want = G;
    for (int k = 0; k < n; ++k)
      for (int j = 0; j < n; ++j)
        for (int i = 0; i < n; ++i)
          want[i + static_cast<size_t>(j) * ld] =
              std::min(want[i + static_cast<size_t>(j) * ld], want[i + static_cast<size_t>(k) * ld] + want[k + static_cast<size_t>(j) * ld]);
    for (int algorithm : {CUASR_APSP_REPEATED_SQUARING, CUASR_APSP_BLOCKED_FLOYD_WARSHALL}) {
      float* dD = to_device(G);
      cuasr_b200_apsp_args_t a{};
      a.dtype = CUASR_F32; a.algorithm = algorithm; a.n = n; a.block = 64; a.D = dD; a.ldd = ld;
      a.workspace_bytes = cuasr_b200_apsp_workspace_size(&a);
      CHECK_CUDA(cudaMalloc(&a.workspace, a.workspace_bytes));
      int st = cuasr_b200_apsp(&a);
      CHECK_CUDA(cudaDeviceSynchronize());
      std::vector<float> got(G.size());
      CHECK_CUDA(cudaMemcpy(got.data(), dD, got.size() * sizeof(float), cudaMemcpyDeviceToHost));
      bool ok = st == 0 && got == want && cuasr_b200_device_status(nullptr) == 0;
      std::printf("cuasr_b200_apsp algorithm=%d: %s\n", algorithm, ok ? "ok" : "FAILED");
      failures += !ok;
      cudaFree(dD); cudaFree(a.workspace);
    }
  }
  std::printf("%s\n", failures == 0 ? "ALL OK" : "FAILURES");
  return failures == 0 ? 0 : 1;
}
