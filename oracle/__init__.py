"""ctypes loaders of the two CPU checkers.  TEST INFRASTRUCTURE: import only from tests/, from the smoke
check and from the CPU-baseline leg of bench.py.

`srgemm(...)`     -> oracle/libcuasr_oracle.so, the plain-C restatement (srgemm_oracle.c)
`ref_srgemm(...)` -> oracle/_ref/libcuasr_ref.so, the reference's own host_srgemm.h compiled unmodified
                     (ref_host_srgemm.cpp); present only where it was built.
Both take numpy arrays (any strides are NOT honoured: pass the buffer and its leading dimension).

`ref_device_srgemm(...)` -> oracle/_ref/libcuasr_ref_device.so, the reference's own SIMT kernels recompiled for
                     sm_100a (ref_device_srgemm.cu): device pointers in, column-major only, a few rings; used to
                     time the reference as it stands on the same GPU and to compare bits.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_PATH = os.path.join(_HERE, "libcuasr_oracle.so")
REF_PATH = os.path.join(_HERE, "_ref", "libcuasr_ref.so")
REF_DEVICE_PATH = os.path.join(_HERE, "_ref", "libcuasr_ref_device.so")
REF_PATH_PATH = os.path.join(_HERE, "_ref", "libcuasr_ref_path.so")

_ARGTYPES = [ctypes.c_int] * 9 + [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                                  ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                                  ctypes.c_void_p, ctypes.c_int]
_libs = {}


def _load(path: str, symbol: str):
    if path not in _libs:
        lib = ctypes.CDLL(path)
        fn = getattr(lib, symbol)
        fn.restype = ctypes.c_int
        fn.argtypes = _ARGTYPES
        _libs[path] = (lib, fn)
    return _libs[path]


def have_ref() -> bool:
    return os.path.exists(REF_PATH)


def have_ref_device() -> bool:
    return os.path.exists(REF_DEVICE_PATH)


def ref_device_srgemm(add_op, mul_op, dtype, mnk, A, lda, B, ldb, C, ldc, D, ldd, alpha, beta, stream=0) -> int:
    """Enqueue the reference's device SRGEMM (default configuration, column-major A, B, C, D) on `stream`.
    A, B, C, D are device addresses.  Returns the reference's status (0 = success) or -1 when the (ring, element
    type) pair is not among the ones built."""
    if REF_DEVICE_PATH not in _libs:
        lib = ctypes.CDLL(REF_DEVICE_PATH)
        fn = lib.cuasr_refdev_srgemm
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_int] * 6 + [ctypes.c_void_p, ctypes.c_int] * 4 + [ctypes.c_void_p] * 3
        _libs[REF_DEVICE_PATH] = (lib, fn)
    _, fn = _libs[REF_DEVICE_PATH]
    np_t = {0: np.float32, 1: np.float64, 2: np.int32, 3: np.uint32}[int(dtype)]
    al, be = (np.array([v], dtype=np_t) for v in (alpha, beta))
    return int(fn(int(add_op), int(mul_op), int(dtype), int(mnk[0]), int(mnk[1]), int(mnk[2]), int(A), int(lda),
                  int(B), int(ldb), int(C), int(ldc), int(D), int(ldd), al.ctypes.data, be.ctypes.data, int(stream)))


def have_ref_path() -> bool:
    return os.path.exists(REF_PATH_PATH)


def ref_fwgemm(A, B, dist, parent, n: int):
    """The reference's legacy cpu_fwgemm_naive (oracle/_ref/libcuasr_ref_path.so) on square column-major n x n
    matrices, in place: dist <- min(dist, A (x) B), parent <- index of the improving k.  float32 or float64 data,
    int32 parent; returns (dist, parent)."""
    lib = ctypes.CDLL(REF_PATH_PATH)
    fn = lib.cuasr_ref_fwgemm
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                   ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    assert parent.dtype == np.int32 and A.dtype == B.dtype == dist.dtype and dist.dtype in (np.float32, np.float64)
    for arr in (A, B, dist, parent):
        assert arr.flags["C_CONTIGUOUS"] and arr.size == n * n
    fn(int(dist.dtype == np.float64), n, A.ctypes.data, n, B.ctypes.data, n, dist.ctypes.data, n, parent.ctypes.data)
    return dist, parent


def max_threads(ref: bool = False) -> int:
    lib, _ = _load(REF_PATH, "cuasr_ref_srgemm") if ref else _load(ORACLE_PATH, "cuasr_oracle_srgemm")
    fn = lib.cuasr_ref_max_threads if ref else lib.cuasr_oracle_max_threads
    fn.restype = ctypes.c_int
    return int(fn())


def _call(fn, add_op, mul_op, dtype, layouts, mnk, alpha, A, lda, B, ldb, beta, C, ldc, D, ldd, add_identity,
          nthreads):
    np_t = D.dtype.type
    for arr in (A, B, C, D):
        assert arr.dtype == D.dtype and arr.flags["C_CONTIGUOUS"]
    al, be, ident = (np.array([v], dtype=np_t) for v in (alpha, beta, add_identity))
    st = fn(int(add_op), int(mul_op), int(dtype), int(layouts[0]), int(layouts[1]), int(layouts[2]),
            int(mnk[0]), int(mnk[1]), int(mnk[2]), al.ctypes.data, A.ctypes.data, int(lda), B.ctypes.data, int(ldb),
            be.ctypes.data, C.ctypes.data, int(ldc), D.ctypes.data, int(ldd), ident.ctypes.data, int(nthreads))
    if st != 0:
        raise RuntimeError(f"oracle returned status {st}")
    return D


def srgemm(add_op, mul_op, dtype, layouts, mnk, alpha, A, lda, B, ldb, beta, C, ldc, D, ldd, add_identity,
           nthreads: int = 0):
    """D = add(mul(alpha, A (x)(+) B), mul(beta, C)) with the C restatement; fills and returns D."""
    _, fn = _load(ORACLE_PATH, "cuasr_oracle_srgemm")
    return _call(fn, add_op, mul_op, dtype, layouts, mnk, alpha, A, lda, B, ldb, beta, C, ldc, D, ldd,
                 add_identity, nthreads)


def ref_srgemm(add_op, mul_op, dtype, layouts, mnk, alpha, A, lda, B, ldb, beta, C, ldc, D, ldd, add_identity,
               nthreads: int = 0):
    """Same call on the reference's own host SRGEMM (only where oracle/_ref has been built)."""
    _, fn = _load(REF_PATH, "cuasr_ref_srgemm")
    return _call(fn, add_op, mul_op, dtype, layouts, mnk, alpha, A, lda, B, ldb, beta, C, ldc, D, ldd,
                 add_identity, nthreads)


def srgemm_path(dtype, layouts, mnk, A, lda, B, ldb, dist, lddist, parent, ldparent, k_offset=0, maximize=False):
    """In-place path-tracking tropical product on the CPU (cuasr_oracle_srgemm_path); returns (dist, parent)."""
    lib, _ = _load(ORACLE_PATH, "cuasr_oracle_srgemm")
    fn = lib.cuasr_oracle_srgemm_path
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int] * 7 + [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                                        ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    assert parent.dtype == np.int32 and dist.flags["C_CONTIGUOUS"] and parent.flags["C_CONTIGUOUS"]
    st = fn(int(dtype), int(layouts[0]), int(layouts[1]), int(layouts[2]), int(mnk[0]), int(mnk[1]), int(mnk[2]),
            A.ctypes.data, int(lda), B.ctypes.data, int(ldb), dist.ctypes.data, int(lddist), parent.ctypes.data,
            int(ldparent), int(k_offset), int(bool(maximize)))
    if st != 0:
        raise RuntimeError(f"oracle returned status {st}")
    return dist, parent
