"""Operator codes, element types and ring constants.

The constants reproduce the reference's functors (include/cuasr/functional.h:28-36, :39-283): "+inf" is
numeric_limits<T>::max() and "-inf" is numeric_limits<T>::min() -- for floating types the smallest positive
normal number, not minus infinity.  `identity(op, dtype, true_infinity=True)` gives the mathematically
intended +-inf instead; the library itself never assumes either, it is told the additive identity per call.
"""
from __future__ import annotations

import enum

import numpy as np


class Op(enum.IntEnum):
    PLUS = 0
    MULTIPLIES = 1
    MINIMUM = 2
    MAXIMUM = 3
    BINARY_AND = 4
    BINARY_OR = 5
    BIT_AND = 6
    BIT_OR = 7
    BIT_XOR = 8


class DType(enum.IntEnum):
    F32 = 0
    F64 = 1
    S32 = 2
    U32 = 3


class Layout(enum.IntEnum):
    COLUMN_MAJOR = 0
    ROW_MAJOR = 1


class Status(enum.IntEnum):
    """cutlass::Status numbering, as returned by every entry point of the reference."""
    kSuccess = 0
    kErrorMisalignedOperand = 1
    kErrorInvalidDataType = 2
    kErrorInvalidLayout = 3
    kErrorInvalidProblem = 4
    kErrorNotSupported = 5
    kErrorWorkspaceNull = 6
    kErrorInternal = 7
    kErrorStaticScratchTooSmall = 64  # this library only: see cuasr_b200_srgemm_splitk_static


NUMPY_DTYPE = {DType.F32: np.float32, DType.F64: np.float64, DType.S32: np.int32, DType.U32: np.uint32}

# (add, mul) pairs the library implements; the first eight are the reference's pre-configured rings
# (include/cuasr/gemm/device/default_srgemm_configuration.h:48-275).
RINGS = {
    "plus_multiplies": (Op.PLUS, Op.MULTIPLIES),
    "minimum_plus": (Op.MINIMUM, Op.PLUS),
    "maximum_plus": (Op.MAXIMUM, Op.PLUS),
    "minimum_maximum": (Op.MINIMUM, Op.MAXIMUM),
    "maximum_minimum": (Op.MAXIMUM, Op.MINIMUM),
    "minimum_multiplies": (Op.MINIMUM, Op.MULTIPLIES),
    "maximum_multiplies": (Op.MAXIMUM, Op.MULTIPLIES),
    "binary_or_binary_and": (Op.BINARY_OR, Op.BINARY_AND),
    # integer element types only
    "bit_xor_bit_and": (Op.BIT_XOR, Op.BIT_AND),
    "bit_or_bit_and": (Op.BIT_OR, Op.BIT_AND),
    "bit_xor_binary_and": (Op.BIT_XOR, Op.BINARY_AND),
}
INTEGER_ONLY_RINGS = ("bit_xor_bit_and", "bit_or_bit_and", "bit_xor_binary_and")


def _limits(dtype: DType):
    np_t = NUMPY_DTYPE[dtype]
    if np.issubdtype(np_t, np.floating):
        fi = np.finfo(np_t)
        return np_t(fi.max), np_t(fi.tiny)  # numeric_limits::max(), numeric_limits::min()
    ii = np.iinfo(np_t)
    return np_t(ii.max), np_t(ii.min)


def identity(op: Op, dtype: DType, true_infinity: bool = False):
    """`Functor<T>::Identity` of the reference for operator `op`."""
    np_t = NUMPY_DTYPE[dtype]
    hi, lo = _limits(dtype)
    if true_infinity and np.issubdtype(np_t, np.floating):
        hi, lo = np_t(np.inf), np_t(-np.inf)
    return {
        Op.PLUS: np_t(0), Op.MULTIPLIES: np_t(1), Op.MINIMUM: hi, Op.MAXIMUM: lo,
        Op.BINARY_AND: np_t(1), Op.BINARY_OR: np_t(0),
        Op.BIT_AND: np_t(np.iinfo(np_t).max if np_t == np.uint32 else -1) if np.issubdtype(np_t, np.integer) else np_t(1),
        Op.BIT_OR: np_t(0), Op.BIT_XOR: np_t(0),
    }[Op(op)]


def annihilator(op: Op, dtype: DType, true_infinity: bool = False):
    """`Functor<T>::Annihilator` of the reference (the default beta of the epilogue is the
    multiplication functor's annihilator: semiring_linear_combination.h:67-71)."""
    np_t = NUMPY_DTYPE[dtype]
    hi, lo = _limits(dtype)
    if true_infinity and np.issubdtype(np_t, np.floating):
        hi, lo = np_t(np.inf), np_t(-np.inf)
    return {
        Op.PLUS: hi, Op.MULTIPLIES: np_t(0), Op.MINIMUM: lo, Op.MAXIMUM: hi,
        Op.BINARY_AND: np_t(0), Op.BINARY_OR: np_t(1),
        Op.BIT_AND: np_t(0), Op.BIT_OR: np_t(np.iinfo(np_t).max if np_t == np.uint32 else -1) if np.issubdtype(np_t, np.integer) else np_t(1),
        Op.BIT_XOR: np_t(0),
    }[Op(op)]
