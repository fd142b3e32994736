// Ring operators on the device: the arithmetic of the reference's functors
// (include/cuasr/functional.h:39-283) selected by operator code, plus the fused forms the B200
// kernels use (three-input min/max, packed fp32 pairs).
//
// Floating-point minimum/maximum map to the PTX min/max instructions.  For every input without NaN
// they return a value equal (operator==) to what the reference's `rhs < lhs ? rhs : lhs` returns; they
// differ only in which zero is returned for a +0/-0 tie and in ignoring a NaN operand.
#pragma once

#include <cstdint>
#include <type_traits>

#include "../../include/cuasr_b200_types.h"
#include "ptx.cuh"

namespace cuasr_b200 {

template <int OP, typename T>
struct Op;

template <typename T>
struct Op<CUASR_OP_PLUS, T> {
  static __device__ __forceinline__ T apply(T l, T r) { return l + r; }
};
template <typename T>
struct Op<CUASR_OP_MULTIPLIES, T> {
  static __device__ __forceinline__ T apply(T l, T r) { return l * r; }
};
// minimum / maximum are written so that a NaN in the LEFT operand (the product, in the contraction) is
// never selected; the kernels rely on this when they pad a ragged K tail with NaN.
template <typename T>
struct Op<CUASR_OP_MINIMUM, T> {
  static __device__ __forceinline__ T apply(T l, T r) { return l < r ? l : r; }
};
template <>
struct Op<CUASR_OP_MINIMUM, float> {
  static __device__ __forceinline__ float apply(float l, float r) { return fminf(l, r); }
};
template <typename T>
struct Op<CUASR_OP_MAXIMUM, T> {
  static __device__ __forceinline__ T apply(T l, T r) { return r < l ? l : r; }
};
template <>
struct Op<CUASR_OP_MAXIMUM, float> {
  static __device__ __forceinline__ float apply(float l, float r) { return fmaxf(l, r); }
};
template <typename T>
struct Op<CUASR_OP_BINARY_AND, T> {
  static __device__ __forceinline__ T apply(T l, T r) { return static_cast<T>(l && r); }
};
template <typename T>
struct Op<CUASR_OP_BINARY_OR, T> {
  static __device__ __forceinline__ T apply(T l, T r) { return static_cast<T>(l || r); }
};
template <typename T>
struct Op<CUASR_OP_BIT_AND, T> {
  static __device__ __forceinline__ T apply(T l, T r) { return l & r; }
};
template <typename T>
struct Op<CUASR_OP_BIT_OR, T> {
  static __device__ __forceinline__ T apply(T l, T r) { return l | r; }
};
template <typename T>
struct Op<CUASR_OP_BIT_XOR, T> {
  static __device__ __forceinline__ T apply(T l, T r) { return l ^ r; }
};

// A semiring: (+) = ADD, (x) = MUL over element type T.
template <int ADD, int MUL, typename T>
struct Ring {
  using Element = T;
  static constexpr int kAdd = ADD;
  static constexpr int kMul = MUL;

  static __device__ __forceinline__ T mul(T a, T b) { return Op<MUL, T>::apply(a, b); }
  // the reference always calls add_op(product, accumulator): arch/srmma.h:84-91 via host_srgemm.h:87
  static __device__ __forceinline__ T add(T prod, T acc) { return Op<ADD, T>::apply(prod, acc); }

  // acc (+) (a0 (x) b0) (+) (a1 (x) b1): two steps of the contraction.
  static __device__ __forceinline__ T mac2(T acc, T a0, T b0, T a1, T b1) {
    if constexpr (std::is_same<T, float>::value && ADD == CUASR_OP_MINIMUM) {
      return min3(acc, mul(a0, b0), mul(a1, b1));
    } else if constexpr (std::is_same<T, float>::value && ADD == CUASR_OP_MAXIMUM) {
      return max3(acc, mul(a0, b0), mul(a1, b1));
    } else if constexpr (std::is_same<T, int32_t>::value && MUL == CUASR_OP_PLUS && ADD == CUASR_OP_MINIMUM) {
      // 32-bit integer tropical rings: one fused add-then-min/max instruction per product (the DPX family of
      // sm_90 and later); the sum wraps like the reference's plain `a + b`
      return __viaddmin_s32(a1, b1, __viaddmin_s32(a0, b0, acc));
    } else if constexpr (std::is_same<T, int32_t>::value && MUL == CUASR_OP_PLUS && ADD == CUASR_OP_MAXIMUM) {
      return __viaddmax_s32(a1, b1, __viaddmax_s32(a0, b0, acc));
    } else if constexpr (std::is_same<T, uint32_t>::value && MUL == CUASR_OP_PLUS && ADD == CUASR_OP_MINIMUM) {
      return __viaddmin_u32(a1, b1, __viaddmin_u32(a0, b0, acc));
    } else if constexpr (std::is_same<T, uint32_t>::value && MUL == CUASR_OP_PLUS && ADD == CUASR_OP_MAXIMUM) {
      return __viaddmax_u32(a1, b1, __viaddmax_u32(a0, b0, acc));
    } else {
      return add(mul(a1, b1), add(mul(a0, b0), acc));
    }
  }

  // fp32 rings whose two steps map onto ONE packed fp32x2 add/multiply and ONE three-input min/max.  Used where
  // both operands deliver (k, k+1) pairs in adjacent registers (both K-contiguous in shared memory).
  static constexpr bool kPackedPairs = std::is_same<T, float>::value &&
                                       (ADD == CUASR_OP_MINIMUM || ADD == CUASR_OP_MAXIMUM) &&
                                       (MUL == CUASR_OP_PLUS || MUL == CUASR_OP_MULTIPLIES);
  static __device__ __forceinline__ float mac_packed(float acc, uint64_t a, uint64_t b) {
    float p0, p1;
    unpack2(MUL == CUASR_OP_PLUS ? add2(a, b) : mul2(a, b), p0, p1);
    return ADD == CUASR_OP_MINIMUM ? min3(acc, p0, p1) : max3(acc, p0, p1);
  }

  // True when an out-of-range operand element may be replaced by NaN (float min/max rings: the NaN
  // product is ignored by min/max) — otherwise by zero, which must then be harmless: 0 (x) 0 has to be
  // the additive identity in effect (plus-times, or-and, xor-and, or-bitand).
  static constexpr bool kNanPadding =
      (ADD == CUASR_OP_MINIMUM || ADD == CUASR_OP_MAXIMUM) && std::is_floating_point<T>::value;
  static constexpr bool kZeroPadding =
      (ADD == CUASR_OP_PLUS && MUL == CUASR_OP_MULTIPLIES) ||
      ((ADD == CUASR_OP_BINARY_OR || ADD == CUASR_OP_BIT_OR || ADD == CUASR_OP_BIT_XOR) &&
       (MUL == CUASR_OP_BINARY_AND || MUL == CUASR_OP_BIT_AND));
  // Rings for which padding K by out-of-range elements is safe inside the TMA kernel.
  static constexpr bool kPaddable = kNanPadding || kZeroPadding;
};

}  // namespace cuasr_b200
