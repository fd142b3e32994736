/*
 * CPU oracle for semiring GEMM.  TEST INFRASTRUCTURE ONLY: nothing that ships (the CUDA library, its
 * host API) may call into this file; it exists so that tests, the smoke check and the CPU-baseline leg
 * of the benchmark can state what the right answer is.
 *
 * It is a plain-C restatement of the reference's host SRGEMM,
 *   tools/include/cuasr/reference/srgemm/host_srgemm.h:33-113
 * using the reference's functor definitions,
 *   include/cuasr/functional.h:39-283
 * and the reference's epilogue formula,
 *   include/cuasr/gemm/epilogue/thread/semiring_linear_combination.h:139-162.
 *
 * Parity status: PINNED.  The restatement is checked (tests/test_oracle.py) against
 *   - the hand-written 4x4x2 min-plus known answer of test/regress/Srgemm_test.cu:15-62,
 *   - outputs of the reference's own host_srgemm.h, compiled unmodified (oracle/ref_host_srgemm.cpp)
 *     and run on seeded inputs; those outputs are committed as fixtures under tests/golden/.
 *
 * What is restated, step by step (host_srgemm.h line numbers):
 *   :56-57   output is processed in 32 x 32 blocks
 *   :67-72   every accumulator starts at add_identity
 *   :75-91   for k = 0 .. K-1 in order:  accum = add(mult(a, b), accum)      (product is the LEFT operand)
 *   :94-109  D = add(mult(alpha, accum), mult(beta, C))                        (C is always read)
 * Each mult/add is rounded once, in the element type; build with -ffp-contract=off so that the
 * plus-times semiring is not fused into FMAs.
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#include "../include/cuasr_b200_types.h"

#ifdef _OPENMP
#include <omp.h>
#endif

#define MBLOCK 32
#define NBLOCK 32

/* functional.h:125-163 / :165-203 — note which operand wins a tie or a NaN comparison. */
#define OP_PLUS(l, r)       ((l) + (r))
#define OP_MULTIPLIES(l, r) ((l) * (r))
#define OP_MINIMUM(l, r)    ((r) < (l) ? (r) : (l))
#define OP_MAXIMUM(l, r)    ((l) < (r) ? (r) : (l))
#define OP_BINARY_AND(l, r) ((l) && (r))
#define OP_BINARY_OR(l, r)  ((l) || (r))
#define OP_BIT_AND(l, r)    ((l) & (r))
#define OP_BIT_OR(l, r)     ((l) | (r))
#define OP_BIT_XOR(l, r)    ((l) ^ (r))

/* Element (i, j) of a matrix with leading dimension ld: column-major i + j*ld, row-major i*ld + j. */
#define AT(p, row_major, ld, i, j) \
  ((p)[(row_major) ? ((size_t)(i) * (size_t)(ld) + (size_t)(j)) : ((size_t)(i) + (size_t)(j) * (size_t)(ld))])

#define DEFINE_SRGEMM(NAME, T, ADD, MUL)                                                              \
  static void NAME(int M, int N, int K, T alpha, const T *A, int rmA, int lda, const T *B, int rmB,  \
                   int ldb, T beta, const T *C, int rmC, int ldc, T *D, int ldd, T add_identity,     \
                   int nthreads) {                                                                   \
    int mblocks = (M + MBLOCK - 1) / MBLOCK, nblocks = (N + NBLOCK - 1) / NBLOCK;                    \
    long nb = (long)mblocks * nblocks;                                                               \
    (void)nthreads;                                                                                  \
    _Pragma("omp parallel for schedule(static) num_threads(nthreads)")                               \
    for (long blk = 0; blk < nb; ++blk) {                                                            \
      int row_block = (int)(blk / nblocks) * MBLOCK, col_block = (int)(blk % nblocks) * NBLOCK;      \
      T accum[MBLOCK][NBLOCK];                                                                       \
      for (int j = 0; j < NBLOCK; j++)                                                               \
        for (int i = 0; i < MBLOCK; i++) accum[i][j] = add_identity;                                 \
      for (int k = 0; k < K; ++k) {                                                                  \
        for (int j = 0; j < NBLOCK; j++) {                                                           \
          int col = col_block + j;                                                                   \
          if (col >= N) break;                                                                       \
          T b = AT(B, rmB, ldb, k, col);                                                             \
          for (int i = 0; i < MBLOCK; i++) {                                                         \
            int row = row_block + i;                                                                 \
            if (row >= M) break;                                                                     \
            T a = AT(A, rmA, lda, row, k);                                                           \
            T prod = (T)MUL(a, b);                                                                   \
            accum[i][j] = (T)ADD(prod, accum[i][j]);                                                 \
          }                                                                                          \
        }                                                                                            \
      }                                                                                              \
      for (int j = 0; j < NBLOCK; j++) {                                                             \
        for (int i = 0; i < MBLOCK; i++) {                                                           \
          int row = row_block + i, col = col_block + j;                                              \
          if (row < M && col < N) {                                                                  \
            T c = AT(C, rmC, ldc, row, col);                                                         \
            T lhs = (T)MUL(alpha, accum[i][j]);                                                      \
            T rhs = (T)MUL(beta, c);                                                                 \
            AT(D, rmC, ldd, row, col) = (T)ADD(lhs, rhs);                                            \
          }                                                                                          \
        }                                                                                            \
      }                                                                                              \
    }                                                                                                \
  }

/* The eight pre-configured semirings of the reference
 * (include/cuasr/gemm/device/default_srgemm_configuration.h:48-275) for every element type ... */
#define DEFINE_RINGS(SUF, T)                                              \
  DEFINE_SRGEMM(srgemm_plus_multiplies_##SUF, T, OP_PLUS, OP_MULTIPLIES) \
  DEFINE_SRGEMM(srgemm_minimum_plus_##SUF, T, OP_MINIMUM, OP_PLUS)       \
  DEFINE_SRGEMM(srgemm_maximum_plus_##SUF, T, OP_MAXIMUM, OP_PLUS)       \
  DEFINE_SRGEMM(srgemm_minimum_maximum_##SUF, T, OP_MINIMUM, OP_MAXIMUM) \
  DEFINE_SRGEMM(srgemm_maximum_minimum_##SUF, T, OP_MAXIMUM, OP_MINIMUM) \
  DEFINE_SRGEMM(srgemm_minimum_multiplies_##SUF, T, OP_MINIMUM, OP_MULTIPLIES) \
  DEFINE_SRGEMM(srgemm_maximum_multiplies_##SUF, T, OP_MAXIMUM, OP_MULTIPLIES) \
  DEFINE_SRGEMM(srgemm_binary_or_binary_and_##SUF, T, OP_BINARY_OR, OP_BINARY_AND)

DEFINE_RINGS(f32, float)
DEFINE_RINGS(f64, double)
DEFINE_RINGS(s32, int32_t)
DEFINE_RINGS(u32, uint32_t)
/* ... and the bitwise rings over integers (GF(2) xor-and, or-and), user-defined in the reference. */
DEFINE_SRGEMM(srgemm_bit_xor_bit_and_s32, int32_t, OP_BIT_XOR, OP_BIT_AND)
DEFINE_SRGEMM(srgemm_bit_xor_bit_and_u32, uint32_t, OP_BIT_XOR, OP_BIT_AND)
DEFINE_SRGEMM(srgemm_bit_or_bit_and_s32, int32_t, OP_BIT_OR, OP_BIT_AND)
DEFINE_SRGEMM(srgemm_bit_or_bit_and_u32, uint32_t, OP_BIT_OR, OP_BIT_AND)
/* GF(2) exactly as examples/01_userdefined_semiring/userdefined_semiring.cu:104-123 builds it:
 * a bitwise xor paired with the reference's logical binary_and, on 0/1 data. */
DEFINE_SRGEMM(srgemm_bit_xor_binary_and_s32, int32_t, OP_BIT_XOR, OP_BINARY_AND)
DEFINE_SRGEMM(srgemm_bit_xor_binary_and_u32, uint32_t, OP_BIT_XOR, OP_BINARY_AND)

#define CALL(FN, T)                                                                                  \
  do {                                                                                               \
    T al, be, id;                                                                                    \
    memcpy(&al, alpha, sizeof(T));                                                                   \
    memcpy(&be, beta, sizeof(T));                                                                    \
    memcpy(&id, add_identity, sizeof(T));                                                            \
    FN(M, N, K, al, (const T *)A, layoutA == CUASR_ROW_MAJOR, lda, (const T *)B,                     \
       layoutB == CUASR_ROW_MAJOR, ldb, be, (const T *)C, layoutC == CUASR_ROW_MAJOR, ldc, (T *)D,   \
       ldd, id, nthreads);                                                                           \
    return CUASR_STATUS_SUCCESS;                                                                     \
  } while (0)

#define DISPATCH_TYPE(RING)                                \
  switch (dtype) {                                         \
    case CUASR_F32: CALL(srgemm_##RING##_f32, float);      \
    case CUASR_F64: CALL(srgemm_##RING##_f64, double);     \
    case CUASR_S32: CALL(srgemm_##RING##_s32, int32_t);    \
    case CUASR_U32: CALL(srgemm_##RING##_u32, uint32_t);   \
    default: return CUASR_STATUS_ERROR_INVALID_DATA_TYPE;  \
  }

#define DISPATCH_INT(RING)                                 \
  switch (dtype) {                                         \
    case CUASR_S32: CALL(srgemm_##RING##_s32, int32_t);    \
    case CUASR_U32: CALL(srgemm_##RING##_u32, uint32_t);   \
    default: return CUASR_STATUS_ERROR_INVALID_DATA_TYPE;  \
  }

/*
 * D = add(mult(alpha, A (x)(+) B), mult(beta, C)) on the CPU.
 *
 * alpha, beta and add_identity point at one element of `dtype`.  C and D share layoutC; D has its
 * own leading dimension.  nthreads <= 0 means "all cores OpenMP reports".  Returns a cuasr_status_t.
 */
int cuasr_oracle_srgemm(int add_op, int mul_op, int dtype, int layoutA, int layoutB, int layoutC,
                        int M, int N, int K, const void *alpha, const void *A, int lda,
                        const void *B, int ldb, const void *beta, const void *C, int ldc, void *D,
                        int ldd, const void *add_identity, int nthreads) {
  if (M < 0 || N < 0 || K < 0) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
#ifdef _OPENMP
  if (nthreads <= 0) nthreads = omp_get_max_threads();
#else
  nthreads = 1;
#endif
  int ring = add_op * 16 + mul_op;
  switch (ring) {
    case CUASR_OP_PLUS * 16 + CUASR_OP_MULTIPLIES: DISPATCH_TYPE(plus_multiplies)
    case CUASR_OP_MINIMUM * 16 + CUASR_OP_PLUS: DISPATCH_TYPE(minimum_plus)
    case CUASR_OP_MAXIMUM * 16 + CUASR_OP_PLUS: DISPATCH_TYPE(maximum_plus)
    case CUASR_OP_MINIMUM * 16 + CUASR_OP_MAXIMUM: DISPATCH_TYPE(minimum_maximum)
    case CUASR_OP_MAXIMUM * 16 + CUASR_OP_MINIMUM: DISPATCH_TYPE(maximum_minimum)
    case CUASR_OP_MINIMUM * 16 + CUASR_OP_MULTIPLIES: DISPATCH_TYPE(minimum_multiplies)
    case CUASR_OP_MAXIMUM * 16 + CUASR_OP_MULTIPLIES: DISPATCH_TYPE(maximum_multiplies)
    case CUASR_OP_BINARY_OR * 16 + CUASR_OP_BINARY_AND: DISPATCH_TYPE(binary_or_binary_and)
    case CUASR_OP_BIT_XOR * 16 + CUASR_OP_BIT_AND: DISPATCH_INT(bit_xor_bit_and)
    case CUASR_OP_BIT_OR * 16 + CUASR_OP_BIT_AND: DISPATCH_INT(bit_or_bit_and)
    case CUASR_OP_BIT_XOR * 16 + CUASR_OP_BINARY_AND: DISPATCH_INT(bit_xor_binary_and)
    default: return CUASR_STATUS_ERROR_NOT_SUPPORTED;
  }
}

/* Number of worker threads cuasr_oracle_srgemm uses when asked for "all". */
int cuasr_oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/*
 * Path-tracking tropical product: restatement of the reference's legacy CPU routine
 *   test/regress/include/fwgpu/cpu_srgemm.hpp:20-48  (cpu_fwgemm_naive)
 * for every (row, col): the running distance starts at dist[row, col], the running parent at parent[row, col];
 * for k ascending, a product A[row, k] + B[k, col] that is STRICTLY better replaces the distance and sets the
 * parent to k (so ties keep the earlier k, and an entry that is never improved keeps its old parent).
 * Generalised from the reference's square, column-major, min-only form to M x N x K, both layouts, and max-plus;
 * k_offset is added to the recorded index (for callers that work on a K-block of a larger product).
 * Parity status: PINNED.  The reference holds no test or fixture for this routine (it is never called there), so
 * the routine itself is the anchor: compiled unmodified (oracle/ref_path.cpp -> oracle/_ref/libcuasr_ref_path.so),
 * its distances and parents on square column-major inputs full of ties are committed as
 * tests/golden/fwgemm_outputs.npz and this restatement must reproduce them; the generalisations (M x N x K, row-major,
 * max-plus, k_offset) have no reference counterpart and are checked against the SRGEMM oracle's distances.
 */
#define DEFINE_PATH(NAME, T)                                                                            \
  static void NAME(int M, int N, int K, const T *A, int rmA, int lda, const T *B, int rmB, int ldb,     \
                   T *dist, int rmC, int lddist, int32_t *parent, int ldparent, int k_offset, int maximize) { \
    for (int row = 0; row < M; ++row) {                                                                 \
      for (int col = 0; col < N; ++col) {                                                               \
        T cur = AT(dist, rmC, lddist, row, col);                                                        \
        int32_t par = AT(parent, rmC, ldparent, row, col);                                              \
        for (int k = 0; k < K; ++k) {                                                                   \
          T prod = (T)(AT(A, rmA, lda, row, k) + AT(B, rmB, ldb, k, col));                              \
          if (maximize ? (cur < prod) : (prod < cur)) {                                                 \
            cur = prod;                                                                                 \
            par = k + k_offset;                                                                         \
          }                                                                                             \
        }                                                                                               \
        AT(dist, rmC, lddist, row, col) = cur;                                                          \
        AT(parent, rmC, ldparent, row, col) = par;                                                      \
      }                                                                                                 \
    }                                                                                                   \
  }
DEFINE_PATH(path_f32, float)
DEFINE_PATH(path_f64, double)

int cuasr_oracle_srgemm_path(int dtype, int layoutA, int layoutB, int layoutC, int M, int N, int K, const void *A,
                             int lda, const void *B, int ldb, void *dist, int lddist, int32_t *parent,
                             int ldparent, int k_offset, int maximize) {
  if (M < 0 || N < 0 || K < 0) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  int ra = layoutA == CUASR_ROW_MAJOR, rb = layoutB == CUASR_ROW_MAJOR, rc = layoutC == CUASR_ROW_MAJOR;
  if (dtype == CUASR_F32)
    path_f32(M, N, K, (const float *)A, ra, lda, (const float *)B, rb, ldb, (float *)dist, rc, lddist, parent,
             ldparent, k_offset, maximize);
  else if (dtype == CUASR_F64)
    path_f64(M, N, K, (const double *)A, ra, lda, (const double *)B, rb, ldb, (double *)dist, rc, lddist, parent,
             ldparent, k_offset, maximize);
  else
    return CUASR_STATUS_ERROR_INVALID_DATA_TYPE;
  return CUASR_STATUS_SUCCESS;
}
