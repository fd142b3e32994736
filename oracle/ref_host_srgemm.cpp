// Builds the REFERENCE's own host SRGEMM into a shared library, for use as a checker only.
//
// This translation unit contains no algorithm.  It includes, unmodified and from where they lie in the
// reference checkout (passed to the compiler with -I), the reference's
//   tools/include/cuasr/reference/srgemm/host_srgemm.h      (the host SRGEMM)
//   include/cuasr/functional.h                              (the ring functors)
//   include/cuasr/gemm/epilogue/thread/semiring_linear_combination.h
// instantiates them for every (ring, element type, layout) the tests use, and exports one C entry
// point with the same signature as the C restatement in srgemm_oracle.c.  The output of the build goes
// to oracle/_ref/, which is not committed.
//
// TEST INFRASTRUCTURE ONLY: nothing that ships may link or load the library built from this file.
#include <cstdint>
#include <cstring>

// host_srgemm.h:47-49 names `do_epilogue_add` in an OpenMP firstprivate clause without declaring it;
// a namespace-scope variable of that name lets the header compile unchanged when OpenMP is enabled.
static int do_epilogue_add = 0;

#include "cuasr/functional.h"
#include "cuasr/gemm/epilogue/thread/semiring_linear_combination.h"
#include "cuasr/reference/srgemm/host_srgemm.h"

#ifdef _OPENMP
#include <omp.h>
#endif

#include "../include/cuasr_b200_types.h"

namespace {

// Bitwise functors in the shape of the user-defined functor of
// examples/01_userdefined_semiring/userdefined_semiring.cu:56-99 (scalar operator + Identity).
template <typename T, int N = 1>
struct bit_xor {
  static T constexpr Identity = static_cast<T>(0);
  T operator()(T lhs, T const &rhs) const { return lhs ^ rhs; }
  cutlass::Array<T, N> operator()(cutlass::Array<T, N> const &l, cutlass::Array<T, N> const &r) const {
    cutlass::Array<T, N> o;
    for (int i = 0; i < N; ++i) o[i] = (*this)(l[i], r[i]);
    return o;
  }
  cutlass::Array<T, N> operator()(T const &s, cutlass::Array<T, N> const &r) const {
    cutlass::Array<T, N> o;
    for (int i = 0; i < N; ++i) o[i] = (*this)(s, r[i]);
    return o;
  }
};
template <typename T, int N = 1>
struct bit_or {
  static T constexpr Identity = static_cast<T>(0);
  T operator()(T lhs, T const &rhs) const { return lhs | rhs; }
  cutlass::Array<T, N> operator()(cutlass::Array<T, N> const &l, cutlass::Array<T, N> const &r) const {
    cutlass::Array<T, N> o;
    for (int i = 0; i < N; ++i) o[i] = (*this)(l[i], r[i]);
    return o;
  }
  cutlass::Array<T, N> operator()(T const &s, cutlass::Array<T, N> const &r) const {
    cutlass::Array<T, N> o;
    for (int i = 0; i < N; ++i) o[i] = (*this)(s, r[i]);
    return o;
  }
};
template <typename T, int N = 1>
struct bit_and {
  static T constexpr Identity    = static_cast<T>(~T(0));
  static T constexpr Annihilator = static_cast<T>(0);
  T operator()(T lhs, T const &rhs) const { return lhs & rhs; }
  cutlass::Array<T, N> operator()(cutlass::Array<T, N> const &l, cutlass::Array<T, N> const &r) const {
    cutlass::Array<T, N> o;
    for (int i = 0; i < N; ++i) o[i] = (*this)(l[i], r[i]);
    return o;
  }
  cutlass::Array<T, N> operator()(T const &s, cutlass::Array<T, N> const &r) const {
    cutlass::Array<T, N> o;
    for (int i = 0; i < N; ++i) o[i] = (*this)(s, r[i]);
    return o;
  }
};

using RowMajor = cutlass::layout::RowMajor;
using ColMajor = cutlass::layout::ColumnMajor;

template <typename Add, typename Mul, typename T, typename LA, typename LB, typename LC>
void run(int M, int N, int K, T alpha, const T *A, int lda, const T *B, int ldb, T beta, const T *C,
         int ldc, T *D, int ldd, T add_identity) {
  using Epilogue = cuasr::epilogue::thread::SemiringLinearCombination<Add, Mul, T, 1>;
  // same instantiation as test/device/testbed.h:204-214
  cuasr::reference::host::Srgemm<Add, Mul, T, LA, T, LB, T, LC, typename Epilogue::ElementCompute,
                                 typename Epilogue::ElementAccumulator, Epilogue>
      srgemm;
  srgemm({M, N, K}, alpha, {const_cast<T *>(A), lda}, {const_cast<T *>(B), ldb}, beta,
         {const_cast<T *>(C), ldc}, {D, ldd}, add_identity);
}

template <typename Add, typename Mul, typename T>
int by_layout(int la, int lb, int lc, int M, int N, int K, const void *alpha, const void *A, int lda,
              const void *B, int ldb, const void *beta, const void *C, int ldc, void *D, int ldd,
              const void *add_identity) {
  T al, be, id;
  std::memcpy(&al, alpha, sizeof(T));
  std::memcpy(&be, beta, sizeof(T));
  std::memcpy(&id, add_identity, sizeof(T));
  auto a = static_cast<const T *>(A);
  auto b = static_cast<const T *>(B);
  auto c = static_cast<const T *>(C);
  auto d = static_cast<T *>(D);
#define GO(LA, LB, LC) run<Add, Mul, T, LA, LB, LC>(M, N, K, al, a, lda, b, ldb, be, c, ldc, d, ldd, id)
  switch (la * 4 + lb * 2 + lc) {
    case 0: GO(ColMajor, ColMajor, ColMajor); break;
    case 1: GO(ColMajor, ColMajor, RowMajor); break;
    case 2: GO(ColMajor, RowMajor, ColMajor); break;
    case 3: GO(ColMajor, RowMajor, RowMajor); break;
    case 4: GO(RowMajor, ColMajor, ColMajor); break;
    case 5: GO(RowMajor, ColMajor, RowMajor); break;
    case 6: GO(RowMajor, RowMajor, ColMajor); break;
    case 7: GO(RowMajor, RowMajor, RowMajor); break;
    default: return CUASR_STATUS_ERROR_INVALID_LAYOUT;
  }
#undef GO
  return CUASR_STATUS_SUCCESS;
}

#define ARGS la, lb, lc, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, D, ldd, add_identity

template <template <typename, int> class Add, template <typename, int> class Mul>
int by_type(int dtype, int la, int lb, int lc, int M, int N, int K, const void *alpha, const void *A,
            int lda, const void *B, int ldb, const void *beta, const void *C, int ldc, void *D,
            int ldd, const void *add_identity) {
  switch (dtype) {
    case CUASR_F32: return by_layout<Add<float, 1>, Mul<float, 1>, float>(ARGS);
    case CUASR_F64: return by_layout<Add<double, 1>, Mul<double, 1>, double>(ARGS);
    case CUASR_S32: return by_layout<Add<int32_t, 1>, Mul<int32_t, 1>, int32_t>(ARGS);
    case CUASR_U32: return by_layout<Add<uint32_t, 1>, Mul<uint32_t, 1>, uint32_t>(ARGS);
    default: return CUASR_STATUS_ERROR_INVALID_DATA_TYPE;
  }
}
template <template <typename, int> class Add, template <typename, int> class Mul>
int by_int_type(int dtype, int la, int lb, int lc, int M, int N, int K, const void *alpha,
                const void *A, int lda, const void *B, int ldb, const void *beta, const void *C,
                int ldc, void *D, int ldd, const void *add_identity) {
  switch (dtype) {
    case CUASR_S32: return by_layout<Add<int32_t, 1>, Mul<int32_t, 1>, int32_t>(ARGS);
    case CUASR_U32: return by_layout<Add<uint32_t, 1>, Mul<uint32_t, 1>, uint32_t>(ARGS);
    default: return CUASR_STATUS_ERROR_INVALID_DATA_TYPE;
  }
}

} // namespace

extern "C" int cuasr_ref_srgemm(int add_op, int mul_op, int dtype, int la, int lb, int lc, int M, int N,
                                int K, const void *alpha, const void *A, int lda, const void *B,
                                int ldb, const void *beta, const void *C, int ldc, void *D, int ldd,
                                const void *add_identity, int nthreads) {
#ifdef _OPENMP
  if (nthreads > 0) omp_set_num_threads(nthreads);
#else
  (void)nthreads;
#endif
#define RING(a, m) ((a)*16 + (m))
  switch (RING(add_op, mul_op)) {
    case RING(CUASR_OP_PLUS, CUASR_OP_MULTIPLIES): return by_type<cuasr::plus, cuasr::multiplies>(dtype, ARGS);
    case RING(CUASR_OP_MINIMUM, CUASR_OP_PLUS): return by_type<cuasr::minimum, cuasr::plus>(dtype, ARGS);
    case RING(CUASR_OP_MAXIMUM, CUASR_OP_PLUS): return by_type<cuasr::maximum, cuasr::plus>(dtype, ARGS);
    case RING(CUASR_OP_MINIMUM, CUASR_OP_MAXIMUM): return by_type<cuasr::minimum, cuasr::maximum>(dtype, ARGS);
    case RING(CUASR_OP_MAXIMUM, CUASR_OP_MINIMUM): return by_type<cuasr::maximum, cuasr::minimum>(dtype, ARGS);
    case RING(CUASR_OP_MINIMUM, CUASR_OP_MULTIPLIES): return by_type<cuasr::minimum, cuasr::multiplies>(dtype, ARGS);
    case RING(CUASR_OP_MAXIMUM, CUASR_OP_MULTIPLIES): return by_type<cuasr::maximum, cuasr::multiplies>(dtype, ARGS);
    case RING(CUASR_OP_BINARY_OR, CUASR_OP_BINARY_AND): return by_type<cuasr::binary_or, cuasr::binary_and>(dtype, ARGS);
    case RING(CUASR_OP_BIT_XOR, CUASR_OP_BIT_AND): return by_int_type<bit_xor, bit_and>(dtype, ARGS);
    case RING(CUASR_OP_BIT_OR, CUASR_OP_BIT_AND): return by_int_type<bit_or, bit_and>(dtype, ARGS);
    case RING(CUASR_OP_BIT_XOR, CUASR_OP_BINARY_AND): return by_int_type<bit_xor, cuasr::binary_and>(dtype, ARGS);
    default: return CUASR_STATUS_ERROR_NOT_SUPPORTED;
  }
}

extern "C" int cuasr_ref_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
