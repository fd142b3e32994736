// Ring functors with the names, scalar behaviour and Identity / Annihilator constants of the reference
// (include/cuasr/functional.h:39-283), plus bitwise functors of the kind a user of the reference defines
// himself (examples/01_userdefined_semiring/userdefined_semiring.cu:56-99).  For these functors the device arithmetic
// lives in the library: the type only selects an operator code (OpCode below) and supplies constants.  They are
// host-device callable all the same, so that they can be paired with a user-defined functor in a kernel compiled
// by the caller (gemm/device/user_functor_srgemm.h).
//
// "+inf" / "-inf" are numeric_limits<T>::max() / ::min() like the reference (functional.h:28-36); define
// CUASR_TRUE_INFINITY to get real infinities for floating-point types.
#pragma once

#include <limits>
#include <type_traits>

#include "../cuasr_b200_types.h"

namespace cuasr {
namespace detail {
template <typename T>
constexpr T pos_inf() {
#ifdef CUASR_TRUE_INFINITY
  return std::numeric_limits<T>::has_infinity ? std::numeric_limits<T>::infinity() : std::numeric_limits<T>::max();
#else
  return std::numeric_limits<T>::max();
#endif
}
template <typename T>
constexpr T neg_inf() {
#ifdef CUASR_TRUE_INFINITY
  return std::numeric_limits<T>::has_infinity ? -std::numeric_limits<T>::infinity() : std::numeric_limits<T>::min();
#else
  return std::numeric_limits<T>::min();
#endif
}
}  // namespace detail

#if defined(__CUDACC__)
#define CUASR_B200_HOST_DEVICE __host__ __device__
#else
#define CUASR_B200_HOST_DEVICE
#endif

#define CUASR_B200_FUNCTOR(NAME, CODE, IDENTITY, ANNIHILATOR, EXPR)                                  \
  template <typename T, int N = 1>                                                                    \
  struct NAME {                                                                                       \
    static constexpr T Identity = IDENTITY;                                                           \
    static constexpr T Annihilator = ANNIHILATOR;                                                     \
    static constexpr int kOpCode = CODE;                                                              \
    CUASR_B200_HOST_DEVICE constexpr T operator()(T lhs, T const& rhs) const { return EXPR; }         \
  };

CUASR_B200_FUNCTOR(plus, CUASR_OP_PLUS, static_cast<T>(0), detail::pos_inf<T>(), lhs + rhs)
CUASR_B200_FUNCTOR(multiplies, CUASR_OP_MULTIPLIES, static_cast<T>(1), static_cast<T>(0), lhs * rhs)
CUASR_B200_FUNCTOR(minimum, CUASR_OP_MINIMUM, detail::pos_inf<T>(), detail::neg_inf<T>(), (rhs < lhs ? rhs : lhs))
CUASR_B200_FUNCTOR(maximum, CUASR_OP_MAXIMUM, detail::neg_inf<T>(), detail::pos_inf<T>(), (lhs < rhs ? rhs : lhs))
CUASR_B200_FUNCTOR(binary_and, CUASR_OP_BINARY_AND, static_cast<T>(true), static_cast<T>(false), static_cast<T>(lhs && rhs))
CUASR_B200_FUNCTOR(binary_or, CUASR_OP_BINARY_OR, static_cast<T>(false), static_cast<T>(true), static_cast<T>(lhs || rhs))
// bitwise, integer element types only
CUASR_B200_FUNCTOR(bit_and, CUASR_OP_BIT_AND, static_cast<T>(~T(0)), static_cast<T>(0), static_cast<T>(lhs & rhs))
CUASR_B200_FUNCTOR(bit_or, CUASR_OP_BIT_OR, static_cast<T>(0), static_cast<T>(~T(0)), static_cast<T>(lhs | rhs))
CUASR_B200_FUNCTOR(bit_xor, CUASR_OP_BIT_XOR, static_cast<T>(0), static_cast<T>(0), static_cast<T>(lhs ^ rhs))
#undef CUASR_B200_FUNCTOR

// Operator code of a functor type.  The functors above carry theirs; a user-defined functor joins by
// specialising this template (for instance a hand-written xor functor -> CUASR_OP_BIT_XOR).
template <typename Functor, typename = void>
struct OpCode;
template <typename Functor>
struct OpCode<Functor, decltype(void(Functor::kOpCode))> {
  static constexpr int value = Functor::kOpCode;
};

// True when the functor type declares its operator code (kOpCode or an OpCode<> specialisation).
template <typename Functor, typename = void>
struct HasOpCode {
  static constexpr bool value = false;
};
template <typename Functor>
struct HasOpCode<Functor, decltype(void(OpCode<Functor>::value))> {
  static constexpr bool value = true;
};

namespace detail {
// What built-in operator `code` computes on the host, with wrap-around (not undefined) integer overflow.
template <typename T>
inline T builtin_apply(int code, T l, T r) {
  using U = typename std::conditional<std::is_integral<T>::value, typename std::make_unsigned<
      typename std::conditional<std::is_integral<T>::value, T, int>::type>::type, T>::type;
  switch (code) {
    case CUASR_OP_PLUS:       return static_cast<T>(static_cast<U>(l) + static_cast<U>(r));
    case CUASR_OP_MULTIPLIES: return static_cast<T>(static_cast<U>(l) * static_cast<U>(r));
    case CUASR_OP_MINIMUM:    return r < l ? r : l;
    case CUASR_OP_MAXIMUM:    return l < r ? r : l;
    case CUASR_OP_BINARY_AND: return static_cast<T>(l && r);
    case CUASR_OP_BINARY_OR:  return static_cast<T>(l || r);
    default: break;
  }
  // bitwise operators: integers only (the caller never asks for them with a floating-point T)
  using I = typename std::conditional<std::is_integral<T>::value, T, long long>::type;
  const I a = static_cast<I>(l), b = static_cast<I>(r);
  switch (code) {
    case CUASR_OP_BIT_AND: return static_cast<T>(a & b);
    case CUASR_OP_BIT_OR:  return static_cast<T>(a | b);
    default:               return static_cast<T>(a ^ b);
  }
}
template <typename T>
inline bool same_value(T x, T y) { return x == y || (x != x && y != y); }
// Functor::Identity / Functor::Annihilator where the functor has them (an addition functor need not have an
// annihilator: examples/01_userdefined_semiring/userdefined_semiring.cu:56-58), else `fallback`.
template <typename Functor, typename T, typename = void>
struct IdentityOr { static T get(T fallback) { return fallback; } };
template <typename Functor, typename T>
struct IdentityOr<Functor, T, decltype(void(Functor::Identity))> { static T get(T) { return Functor::Identity; } };
template <typename Functor, typename T, typename = void>
struct AnnihilatorOr { static T get(T fallback) { return fallback; } };
template <typename Functor, typename T>
struct AnnihilatorOr<Functor, T, decltype(void(Functor::Annihilator))> { static T get(T) { return Functor::Annihilator; } };
}  // namespace detail

// A functor that neither carries kOpCode nor has an OpCode<> specialisation (for instance the hand-written
// binary_xor of examples/01_userdefined_semiring/userdefined_semiring.cu:56-99, compiled unchanged) may still be
// one of the operators the library implements.  It is accepted as operator X only if it agrees with X on every one
// of several hundred value pairs: small integers, mid-range and large magnitudes of both signs, the extremes of the
// element type, and the functor's own Identity and Annihilator.  A functor that departs from X anywhere in that set
// (a saturating add, a modular product, ...) gets -1: under a CUDA compiler the caller then compiles the functor
// itself into a kernel (gemm/device/user_functor_srgemm.h); elsewhere the call is refused as not supported.
template <typename Functor, typename T>
inline int probe_op_code() {
  Functor f;
  const int candidates[] = {CUASR_OP_PLUS,       CUASR_OP_MULTIPLIES, CUASR_OP_MINIMUM, CUASR_OP_MAXIMUM, CUASR_OP_BINARY_AND,
                            CUASR_OP_BINARY_OR,  CUASR_OP_BIT_AND,    CUASR_OP_BIT_OR,  CUASR_OP_BIT_XOR};
  const T lim_max = std::numeric_limits<T>::max(), lim_low = std::numeric_limits<T>::lowest();
  const T lim_min = std::numeric_limits<T>::min();
  const T big = std::is_integral<T>::value ? static_cast<T>(lim_max / 3) : static_cast<T>(1.0e6);
  const bool is_signed = std::numeric_limits<T>::is_signed;
  T values[40];
  int nv = 0;
  for (int v = 0; v <= 8; ++v) values[nv++] = static_cast<T>(v);
  if (is_signed) for (int v = 1; v <= 8; ++v) values[nv++] = static_cast<T>(0) - static_cast<T>(v);
  const T specials[] = {static_cast<T>(100), static_cast<T>(1000), static_cast<T>(12345), big,
                        static_cast<T>(big + static_cast<T>(7)), lim_max, lim_low, lim_min,
                        detail::IdentityOr<Functor, T>::get(static_cast<T>(2)),
                        detail::AnnihilatorOr<Functor, T>::get(static_cast<T>(3))};
  for (T v : specials) values[nv++] = v;
  if (is_signed) { values[nv++] = static_cast<T>(0) - static_cast<T>(1000); values[nv++] = static_cast<T>(0) - big; }
  for (int code : candidates) {
    const bool bitwise = code == CUASR_OP_BIT_AND || code == CUASR_OP_BIT_OR || code == CUASR_OP_BIT_XOR;
    if (bitwise && !std::is_integral<T>::value) continue;
    bool agrees = true;
    for (int i = 0; i < nv && agrees; ++i)
      for (int j = 0; j < nv && agrees; ++j)
        agrees = detail::same_value(static_cast<T>(f(values[i], values[j])),
                                    detail::builtin_apply<T>(code, values[i], values[j]));
    if (agrees) return code;
  }
  return -1;
}

// The operator code of any functor: declared (kOpCode or an OpCode<> specialisation) or, failing that, probed once.
template <typename Functor, typename T, typename = void>
struct OpCodeOf {
  static int get() {
    static const int code = probe_op_code<Functor, T>();
    return code;
  }
};
template <typename Functor, typename T>
struct OpCodeOf<Functor, T, decltype(void(OpCode<Functor>::value))> {
  static int get() { return OpCode<Functor>::value; }
};

template <typename T> struct DTypeCode;
template <> struct DTypeCode<float>    { static constexpr int value = CUASR_F32; };
template <> struct DTypeCode<double>   { static constexpr int value = CUASR_F64; };
template <> struct DTypeCode<int>      { static constexpr int value = CUASR_S32; };
template <> struct DTypeCode<unsigned> { static constexpr int value = CUASR_U32; };

}  // namespace cuasr
