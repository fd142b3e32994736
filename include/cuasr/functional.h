// Ring functors with the names, scalar behaviour and Identity / Annihilator constants of the reference
// (include/cuasr/functional.h:39-283), plus bitwise functors of the kind a user of the reference defines
// himself (examples/01_userdefined_semiring/userdefined_semiring.cu:56-99).  Host-side: the device arithmetic
// lives in the library; a functor type only selects an operator code (OpCode below) and supplies constants.
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

#define CUASR_B200_FUNCTOR(NAME, CODE, IDENTITY, ANNIHILATOR, EXPR)            \
  template <typename T, int N = 1>                                              \
  struct NAME {                                                                 \
    static constexpr T Identity = IDENTITY;                                     \
    static constexpr T Annihilator = ANNIHILATOR;                               \
    static constexpr int kOpCode = CODE;                                        \
    constexpr T operator()(T lhs, T const& rhs) const { return EXPR; }          \
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

// A functor that neither carries kOpCode nor has an OpCode<> specialisation (for instance the hand-written
// binary_xor of examples/01_userdefined_semiring/userdefined_semiring.cu:56-99, compiled unchanged) is recognised by
// what it computes: evaluated on the host on three pairs of small values, the nine operators this library implements
// all give different answers.  Returns -1 for anything else, which the library refuses as "not supported".
template <typename Functor, typename T>
inline int probe_op_code() {
  Functor f;
  const long long got[3] = {static_cast<long long>(f(T(3), T(5))), static_cast<long long>(f(T(0), T(5))),
                            static_cast<long long>(f(T(6), T(3)))};
  struct Row { int code; long long want[3]; bool integers_only; };
  const Row table[] = {{CUASR_OP_PLUS, {8, 5, 9}, false},       {CUASR_OP_MULTIPLIES, {15, 0, 18}, false},
                       {CUASR_OP_MINIMUM, {3, 0, 3}, false},    {CUASR_OP_MAXIMUM, {5, 5, 6}, false},
                       {CUASR_OP_BINARY_AND, {1, 0, 1}, false}, {CUASR_OP_BINARY_OR, {1, 1, 1}, false},
                       {CUASR_OP_BIT_AND, {1, 0, 2}, true},     {CUASR_OP_BIT_OR, {7, 5, 7}, true},
                       {CUASR_OP_BIT_XOR, {6, 5, 5}, true}};
  for (const Row& row : table)
    if ((!row.integers_only || std::is_integral<T>::value) && got[0] == row.want[0] && got[1] == row.want[1] &&
        got[2] == row.want[2])
      return row.code;
  return -1;
}

// The operator code of any functor: declared (kOpCode or an OpCode<> specialisation) or, failing that, probed.
template <typename Functor, typename T, typename = void>
struct OpCodeOf {
  static int get() { return probe_op_code<Functor, T>(); }
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
