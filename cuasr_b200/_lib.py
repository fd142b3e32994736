"""ctypes binding of cuasr_b200/csrc/libcuasr_b200.so (the declarations of include/cuasr_b200.h).

There is no fallback: if the CUDA library has not been built, importing this module raises.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libcuasr_b200.so")


class Scalar(ctypes.Structure):
    _fields_ = [("bytes", ctypes.c_ubyte * 8)]


class Desc(ctypes.Structure):
    _fields_ = [
        ("add_op", ctypes.c_int32), ("mul_op", ctypes.c_int32), ("dtype", ctypes.c_int32),
        ("layout_a", ctypes.c_int32), ("layout_b", ctypes.c_int32), ("layout_c", ctypes.c_int32),
        ("split_k_serial", ctypes.c_int32), ("reserved", ctypes.c_int32),
    ]


class Args(ctypes.Structure):
    _fields_ = [
        ("m", ctypes.c_int32), ("n", ctypes.c_int32), ("k", ctypes.c_int32), ("split_k_slices", ctypes.c_int32),
        ("A", ctypes.c_void_p), ("lda", ctypes.c_int64),
        ("B", ctypes.c_void_p), ("ldb", ctypes.c_int64),
        ("C", ctypes.c_void_p), ("ldc", ctypes.c_int64),
        ("D", ctypes.c_void_p), ("ldd", ctypes.c_int64),
        ("alpha", Scalar), ("beta", Scalar), ("add_identity", Scalar), ("mul_identity", Scalar),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
        ("stream", ctypes.c_void_p),
    ]


class ApspArgs(ctypes.Structure):          # cuasr_b200_apsp_args_t
    _fields_ = [
        ("dtype", ctypes.c_int32), ("algorithm", ctypes.c_int32), ("n", ctypes.c_int32), ("block", ctypes.c_int32),
        ("iterations", ctypes.c_int32), ("reserved", ctypes.c_int32),
        ("D", ctypes.c_void_p), ("ldd", ctypes.c_int64),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
        ("stream", ctypes.c_void_p),
        ("parent", ctypes.c_void_p), ("ld_parent", ctypes.c_int64),
    ]


class ApspShardArgs(ctypes.Structure):     # cuasr_b200_apsp_shard_args_t
    _fields_ = [
        ("dtype", ctypes.c_int32), ("n", ctypes.c_int32), ("col0", ctypes.c_int32), ("cols", ctypes.c_int32),
        ("D_cur", ctypes.c_void_p), ("ld_cur", ctypes.c_int64),
        ("D_next", ctypes.c_void_p), ("ld_next", ctypes.c_int64),
        ("n_peers", ctypes.c_int32), ("reserved", ctypes.c_int32),
        ("peer_next", ctypes.POINTER(ctypes.c_void_p)),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
        ("stream", ctypes.c_void_p),
    ]


class ApspMultiArgs(ctypes.Structure):     # cuasr_b200_apsp_multi_args_t
    _fields_ = [
        ("dtype", ctypes.c_int32), ("algorithm", ctypes.c_int32), ("n", ctypes.c_int32), ("block", ctypes.c_int32),
        ("iterations", ctypes.c_int32), ("n_devices", ctypes.c_int32),
        ("devices", ctypes.POINTER(ctypes.c_int32)),
        ("buf0", ctypes.POINTER(ctypes.c_void_p)), ("buf1", ctypes.POINTER(ctypes.c_void_p)),
        ("ldd", ctypes.c_int64),
        ("workspace", ctypes.POINTER(ctypes.c_void_p)), ("workspace_bytes", ctypes.c_size_t),
        ("streams", ctypes.POINTER(ctypes.c_void_p)),
        ("result_buffer", ctypes.POINTER(ctypes.c_int32)), ("device_status", ctypes.POINTER(ctypes.c_int32)),
    ]


# name -> (restype, argtypes); every symbol include/*.h declares
PROTOTYPES = {
    "cuasr_b200_srgemm_can_implement": (ctypes.c_int, [ctypes.POINTER(Desc), ctypes.POINTER(Args)]),
    "cuasr_b200_srgemm_workspace_size": (ctypes.c_size_t, [ctypes.POINTER(Desc), ctypes.POINTER(Args)]),
    "cuasr_b200_srgemm": (ctypes.c_int, [ctypes.POINTER(Desc), ctypes.POINTER(Args)]),
    "cuasr_b200_srgemm_optional_workspace_size": (ctypes.c_size_t, [ctypes.POINTER(Desc), ctypes.POINTER(Args)]),
    "cuasr_b200_srgemm_push": (ctypes.c_int, [ctypes.POINTER(Desc), ctypes.POINTER(Args), ctypes.c_int,
                                              ctypes.POINTER(ctypes.c_void_p)]),
    "cuasr_b200_srgemm_path": (ctypes.c_int, [ctypes.POINTER(Desc), ctypes.POINTER(Args), ctypes.c_void_p,
                                              ctypes.c_int64, ctypes.c_int32]),
    "cuasr_b200_srgemm_splitk_can_implement": (ctypes.c_int, [ctypes.POINTER(Desc), ctypes.POINTER(Args)]),
    "cuasr_b200_srgemm_splitk_workspace_size": (ctypes.c_size_t, [ctypes.POINTER(Desc), ctypes.POINTER(Args)]),
    "cuasr_b200_srgemm_splitk": (ctypes.c_int, [ctypes.POINTER(Desc), ctypes.POINTER(Args)]),
    "cuasr_b200_srgemm_splitk_static": (ctypes.c_int, [ctypes.POINTER(Desc), ctypes.POINTER(Args)]),
    "cuasr_b200_apsp_workspace_size": (ctypes.c_size_t, [ctypes.POINTER(ApspArgs)]),
    "cuasr_b200_apsp": (ctypes.c_int, [ctypes.POINTER(ApspArgs)]),
    "cuasr_b200_apsp_shard_squaring": (ctypes.c_int, [ctypes.POINTER(ApspShardArgs)]),
    "cuasr_b200_apsp_multi": (ctypes.c_int, [ctypes.POINTER(ApspMultiArgs)]),
    "cuasr_b200_apsp_multi_workspace_size": (ctypes.c_size_t, [ctypes.POINTER(ApspMultiArgs)]),
    "cuasr_b200_apsp_multi_partition": (ctypes.c_int, [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                                       ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)]),
    "cuasr_b200_flag_raise": (ctypes.c_int, [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_uint32,
                                             ctypes.c_void_p]),
    "cuasr_b200_flag_wait": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_uint32, ctypes.c_uint32,
                                            ctypes.c_void_p]),
    "cuasr_b200_pack_k_contiguous": (ctypes.c_int, [ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32,
                                                    ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64,
                                                    ctypes.c_void_p]),
    "cuasr_b200_device_status": (ctypes.c_int, [ctypes.c_void_p]),
    "cuasr_b200_last_kernel": (ctypes.c_char_p, []),
    "cuasr_b200_launch_count": (ctypes.c_uint64, []),
    "cuasr_b200_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "cuasr_b200_version": (ctypes.c_char_p, []),
}

_lib = None


def load() -> ctypes.CDLL:
    """Loads the library once and attaches prototypes.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m cuasr_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in PROTOTYPES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib
