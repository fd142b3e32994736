/*
 * Enumerations shared by the C ABI of the B200 semiring-GEMM library and by its CPU oracle.
 *
 * The numbering of operator codes follows the order in which the reference declares its functors
 * (include/cuasr/functional.h:39-283: plus, multiplies, minimum, maximum, binary_and, binary_or),
 * followed by the bitwise functors a user defines in the style of
 * examples/01_userdefined_semiring/userdefined_semiring.cu:56-99.
 */
#ifndef CUASR_B200_TYPES_H
#define CUASR_B200_TYPES_H

#ifdef __cplusplus
extern "C" {
#endif

/* Ring operators. A semiring is a pair (add_op, mul_op). */
typedef enum cuasr_op {
  CUASR_OP_PLUS       = 0, /* lhs + rhs                 functional.h:39-80   */
  CUASR_OP_MULTIPLIES = 1, /* lhs * rhs                 functional.h:82-123 */
  CUASR_OP_MINIMUM    = 2, /* rhs < lhs ? rhs : lhs     functional.h:125-163 */
  CUASR_OP_MAXIMUM    = 3, /* lhs < rhs ? rhs : lhs     functional.h:165-203 */
  CUASR_OP_BINARY_AND = 4, /* lhs && rhs (logical)      functional.h:205-243 */
  CUASR_OP_BINARY_OR  = 5, /* lhs || rhs (logical)      functional.h:245-283 */
  CUASR_OP_BIT_AND    = 6, /* lhs & rhs  (integers only; user-defined in the reference) */
  CUASR_OP_BIT_OR     = 7, /* lhs | rhs  (integers only; user-defined in the reference) */
  CUASR_OP_BIT_XOR    = 8  /* lhs ^ rhs  (integers only; examples/01…:56-99)            */
} cuasr_op_t;

/* Element type of A, B, C, D, the accumulator and the scalars (the reference's tests and examples
 * always use one type for all of them: test/device/simt_sm50.py:27-33). */
typedef enum cuasr_dtype {
  CUASR_F32 = 0,
  CUASR_F64 = 1,
  CUASR_S32 = 2,
  CUASR_U32 = 3
} cuasr_dtype_t;

/* cutlass::layout::{ColumnMajor,RowMajor}; one leading dimension in elements. */
typedef enum cuasr_layout {
  CUASR_COLUMN_MAJOR = 0,
  CUASR_ROW_MAJOR    = 1
} cuasr_layout_t;

/* Same numbering as cutlass::Status, which the reference returns from every host entry point
 * (include/cuasr/gemm/device/srgemm.h:196-356). */
typedef enum cuasr_status {
  CUASR_STATUS_SUCCESS                   = 0,
  CUASR_STATUS_ERROR_MISALIGNED_OPERAND  = 1,
  CUASR_STATUS_ERROR_INVALID_DATA_TYPE   = 2,
  CUASR_STATUS_ERROR_INVALID_LAYOUT      = 3,
  CUASR_STATUS_ERROR_INVALID_PROBLEM     = 4,
  CUASR_STATUS_ERROR_NOT_SUPPORTED       = 5,
  CUASR_STATUS_ERROR_WORKSPACE_NULL      = 6,
  CUASR_STATUS_ERROR_INTERNAL            = 7,
  /* Not a cutlass::Status value: the problem needs more scratch than the library's built-in static
   * scratch array holds (only returned by cuasr_b200_srgemm_splitk_static). */
  CUASR_STATUS_ERROR_STATIC_SCRATCH_TOO_SMALL = 64
} cuasr_status_t;

#ifdef __cplusplus
}
#endif
#endif /* CUASR_B200_TYPES_H */
