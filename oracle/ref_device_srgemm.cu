// Builds the REFERENCE's own device SRGEMM (its SIMT kernels, unmodified, recompiled for sm_100a) into a shared
// library, to answer one question on the same GPU: how fast is the reference as it stands, and does the new
// kernel return the same bits.
//
// This translation unit contains no algorithm.  It includes, from where they lie in the reference checkout
// (passed to the compiler with -I), the reference's
//   include/cuasr/functional.h
//   include/cuasr/gemm/device/default_srgemm_configuration.h
//   include/cuasr/gemm/device/srgemm.h
// instantiates cuasr::gemm::device::Srgemm with its default configuration for the rings and element types of
// the benchmark configurations (column-major operands and output), and exports one C entry point.  The output of
// the build goes to oracle/_ref/, which is not committed.
//
// TEST AND MEASUREMENT INFRASTRUCTURE ONLY: nothing that ships may link or load the library built from this file.
#include <cuda_runtime.h>

#include "cuasr/functional.h"
#include "cuasr/gemm/device/default_srgemm_configuration.h"
#include "cuasr/gemm/device/srgemm.h"

#include "../include/cuasr_b200_types.h"

namespace {

template <template <typename, int> class Add, template <typename, int> class Mul, typename T>
int run(int m, int n, int k, void const *A, int lda, void const *B, int ldb, void const *C, int ldc, void *D, int ldd,
        void const *alpha, void const *beta, cudaStream_t stream) {
  using ColumnMajor = cutlass::layout::ColumnMajor;
  using Op = cuasr::gemm::device::Srgemm<Add<T, 1>, Mul<T, 1>, T, ColumnMajor, T, ColumnMajor, T, ColumnMajor, T>;
  typename Op::Arguments args({m, n, k}, {static_cast<T const *>(A), lda}, {static_cast<T const *>(B), ldb},
                              {static_cast<T const *>(C), ldc}, {static_cast<T *>(D), ldd},
                              {*static_cast<T const *>(alpha), *static_cast<T const *>(beta)});
  Op op;
  return static_cast<int>(op(args, nullptr, stream));
}

}  // namespace

// Returns the reference's cutlass::Status as an int (0 = success), or -1 when the (ring, type) pair was not built.
extern "C" __attribute__((visibility("default"))) int cuasr_refdev_srgemm(
    int add_op, int mul_op, int dtype, int m, int n, int k, void const *A, int lda, void const *B, int ldb,
    void const *C, int ldc, void *D, int ldd, void const *alpha, void const *beta, void *stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define CASE(ADD, MUL, DT, AddF, MulF, T)                                                           \
  if (add_op == ADD && mul_op == MUL && dtype == DT)                                                \
    return run<cuasr::AddF, cuasr::MulF, T>(m, n, k, A, lda, B, ldb, C, ldc, D, ldd, alpha, beta, s);
  CASE(CUASR_OP_MINIMUM, CUASR_OP_PLUS, CUASR_F32, minimum, plus, float)
  CASE(CUASR_OP_MINIMUM, CUASR_OP_PLUS, CUASR_F64, minimum, plus, double)
  CASE(CUASR_OP_MAXIMUM, CUASR_OP_PLUS, CUASR_F64, maximum, plus, double)
  CASE(CUASR_OP_MAXIMUM, CUASR_OP_MINIMUM, CUASR_F32, maximum, minimum, float)
  CASE(CUASR_OP_PLUS, CUASR_OP_MULTIPLIES, CUASR_F64, plus, multiplies, double)
#undef CASE
  return -1;
}
