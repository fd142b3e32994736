"""Host-side mirror of the reference's device-level operators, over the C ABI.

`Srgemm` and `SrgemmSplitKParallel` keep the method names, argument meaning and status codes of
cuasr::gemm::device::Srgemm (include/cuasr/gemm/device/srgemm.h:139-356) and
cuasr::gemm::device::SrgemmSplitKParallel (include/cuasr/gemm/device/srgemm_splitk_parallel.h:155-378);
template parameters become constructor arguments.  Matrices are device pointers with one leading
dimension (cutlass::TensorRef); torch CUDA tensors are accepted wherever a pointer is.
"""
from __future__ import annotations

import ctypes
import dataclasses
from typing import Any, Optional, Tuple

import numpy as np

from . import _lib
from .semiring import DType, Layout, NUMPY_DTYPE, Op, Status, annihilator, identity


def _ptr(x: Any) -> Optional[int]:
    if x is None:
        return None
    if hasattr(x, "data_ptr"):
        return int(x.data_ptr())
    return int(x)


def _scalar(value, dtype: DType) -> _lib.Scalar:
    s = _lib.Scalar()
    raw = np.asarray(value).astype(NUMPY_DTYPE[dtype]).tobytes()
    for i, b in enumerate(raw):
        s.bytes[i] = b
    return s


def _stream_handle(stream) -> Optional[int]:
    if stream is None:
        return None
    if hasattr(stream, "cuda_stream"):
        return int(stream.cuda_stream)
    return int(stream)


@dataclasses.dataclass
class Arguments:
    """device::Srgemm::Arguments (device/srgemm.h:139-183)."""
    problem_size: Tuple[int, int, int]                 # (M, N, K)
    ref_A: Tuple[Any, int]                             # (pointer or tensor, leading dimension)
    ref_B: Tuple[Any, int]
    ref_C: Tuple[Any, int]
    ref_D: Tuple[Any, int]
    epilogue: Tuple[Any, ...] = ()                     # (), (alpha,), or (alpha, beta)
    split_k_slices: int = 1


class _Operator:
    _splitk_parallel = False

    def __init__(self, add_op: Op, mul_op: Op, dtype: DType = DType.F32,
                 layout_a: Layout = Layout.COLUMN_MAJOR, layout_b: Layout = Layout.COLUMN_MAJOR,
                 layout_c: Layout = Layout.COLUMN_MAJOR, split_k_serial: bool = False,
                 add_identity=None, mul_identity=None):
        self.add_op, self.mul_op, self.dtype = Op(add_op), Op(mul_op), DType(dtype)
        self.layout_a, self.layout_b, self.layout_c = Layout(layout_a), Layout(layout_b), Layout(layout_c)
        self.kSplitKSerial = bool(split_k_serial)
        # AdditionOp::Identity / MultiplicationOp::Identity of the functors the operator is "instantiated" with
        self.add_identity = identity(self.add_op, self.dtype) if add_identity is None else add_identity
        self.mul_identity = identity(self.mul_op, self.dtype) if mul_identity is None else mul_identity
        self._lib = _lib.load()
        self._desc = _lib.Desc(int(self.add_op), int(self.mul_op), int(self.dtype), int(self.layout_a),
                               int(self.layout_b), int(self.layout_c), int(self.kSplitKSerial), 0)
        self._args: Optional[_lib.Args] = None
        self._keepalive = None

    # -- helpers ---------------------------------------------------------------------------------------
    def _pack(self, args: Arguments, workspace=None, workspace_bytes: int = 0, stream=None) -> _lib.Args:
        m, n, k = args.problem_size
        epi = tuple(args.epilogue)
        # EpilogueOutputOp::Params defaults (semiring_linear_combination.h:67-85)
        alpha = epi[0] if len(epi) >= 1 else self.mul_identity
        beta = epi[1] if len(epi) >= 2 else annihilator(self.mul_op, self.dtype)
        a = _lib.Args()
        a.m, a.n, a.k, a.split_k_slices = int(m), int(n), int(k), int(args.split_k_slices)
        a.A, a.lda = _ptr(args.ref_A[0]), int(args.ref_A[1])
        a.B, a.ldb = _ptr(args.ref_B[0]), int(args.ref_B[1])
        a.C, a.ldc = _ptr(args.ref_C[0]), int(args.ref_C[1])
        a.D, a.ldd = _ptr(args.ref_D[0]), int(args.ref_D[1])
        a.alpha, a.beta = _scalar(alpha, self.dtype), _scalar(beta, self.dtype)
        a.add_identity = _scalar(self.add_identity, self.dtype)
        a.mul_identity = _scalar(self.mul_identity, self.dtype)
        a.workspace = _ptr(workspace)
        if workspace is not None and workspace_bytes == 0 and hasattr(workspace, "numel"):
            workspace_bytes = workspace.numel() * workspace.element_size()
        a.workspace_bytes = int(workspace_bytes)
        a.stream = _stream_handle(stream)
        return a

    def _fn(self, base: str):
        name = "cuasr_b200_srgemm_splitk" if self._splitk_parallel else "cuasr_b200_srgemm"
        return getattr(self._lib, name + base)

    # -- the reference's interface -----------------------------------------------------------------------
    def can_implement(self, args: Arguments) -> Status:
        return Status(self._fn("_can_implement")(ctypes.byref(self._desc), ctypes.byref(self._pack(args))))

    def get_workspace_size(self, args: Arguments) -> int:
        return int(self._fn("_workspace_size")(ctypes.byref(self._desc), ctypes.byref(self._pack(args))))

    def get_optional_workspace_size(self, args: Arguments) -> int:
        """Bytes of OPTIONAL workspace for an unsplit launch (0 = nothing to gain): it buys a balanced last wave and,
        for fp32 min/max-plus/times rings, K-contiguous copies of the operands so that packed adds can be used."""
        return int(self._lib.cuasr_b200_srgemm_optional_workspace_size(ctypes.byref(self._desc),
                                                                      ctypes.byref(self._pack(args))))

    def initialize(self, args: Arguments, workspace=None, stream=None, workspace_bytes: int = 0) -> Status:
        packed = self._pack(args, workspace, workspace_bytes, stream)
        status = Status(self._fn("_can_implement")(ctypes.byref(self._desc), ctypes.byref(packed)))
        if status != Status.kSuccess:
            return status
        need = self._fn("_workspace_size")(ctypes.byref(self._desc), ctypes.byref(packed))
        if need > 0 and packed.workspace is None:
            return Status.kErrorWorkspaceNull
        self._args = packed
        self._keepalive = (args, workspace)
        return Status.kSuccess

    def update(self, args: Arguments, workspace=None, workspace_bytes: int = 0) -> Status:
        """Refreshes pointers only (device/srgemm.h:285-300)."""
        if self._args is None:
            return Status.kErrorInternal
        stream = self._args.stream
        self._args = self._pack(args, workspace, workspace_bytes, stream)
        self._keepalive = (args, workspace)
        return Status.kSuccess

    def run(self, stream=None) -> Status:
        if self._args is None:
            return Status.kErrorInternal
        if stream is not None:
            self._args.stream = _stream_handle(stream)
        return Status(self._fn("")(ctypes.byref(self._desc), ctypes.byref(self._args)))

    def run_push(self, extra_outputs, stream=None) -> Status:
        """run(), with every element of D also stored to each matrix in `extra_outputs` (pointers or tensors
        with D's layout and leading dimension; peer-GPU memory allowed): cuasr_b200_srgemm_push."""
        if self._args is None or self._splitk_parallel:
            return Status.kErrorInternal
        if stream is not None:
            self._args.stream = _stream_handle(stream)
        ptrs = (ctypes.c_void_p * max(1, len(extra_outputs)))(*[_ptr(x) for x in extra_outputs])
        return Status(self._lib.cuasr_b200_srgemm_push(ctypes.byref(self._desc), ctypes.byref(self._args),
                                                       len(extra_outputs), ptrs))

    def __call__(self, args: Optional[Arguments] = None, workspace=None, stream=None,
                 workspace_bytes: int = 0) -> Status:
        if args is not None:
            status = self.initialize(args, workspace, stream, workspace_bytes)
            if status != Status.kSuccess:
                return status
        return self.run(stream)

    # -- extras ------------------------------------------------------------------------------------------
    def last_kernel(self) -> str:
        return self._lib.cuasr_b200_last_kernel().decode()


class Srgemm(_Operator):
    """cuasr::gemm::device::Srgemm."""


class SrgemmSplitKParallel(_Operator):
    """cuasr::gemm::device::SrgemmSplitKParallel."""
    _splitk_parallel = True


def srgemm_path(operator: _Operator, problem_size, ref_A, ref_B, ref_dist, ref_parent, k_offset: int = 0,
                stream=None) -> Status:
    """dist <- min/max(dist, A (x) B) in place with the winning contraction index recorded in `parent` (int32, same
    layout as dist): cuasr_b200_srgemm_path.  `operator` supplies ring (min-plus or max-plus), type and layouts."""
    args = Arguments(problem_size, ref_A, ref_B, ref_dist, ref_dist)
    packed = operator._pack(args, None, 0, stream)
    lib = _lib.load()
    return Status(lib.cuasr_b200_srgemm_path(ctypes.byref(operator._desc), ctypes.byref(packed), _ptr(ref_parent[0]),
                                             int(ref_parent[1]), int(k_offset)))


STATIC_SCRATCH_BYTES = 16 * 1024 * 1024 + 4096


def srgemm_splitk_static(operator: _Operator, args: Arguments, stream=None) -> Status:
    """Split-K SRGEMM on the library's built-in static scratch (cuasr_b200_srgemm_splitk_static): for callers
    that are not allowed to allocate device memory.  `operator` supplies the ring, element type and layouts;
    no workspace is passed.  Calls that overlap on the GPU share the scratch and must be serialised."""
    packed = operator._pack(args, None, 0, stream)
    lib = _lib.load()
    return Status(lib.cuasr_b200_srgemm_splitk_static(ctypes.byref(operator._desc), ctypes.byref(packed)))


def pack_k_contiguous(dtype: DType, src, ld_src: int, src_k_contiguous: bool, rows: int, k: int, dst, ld_dst: int,
                      stream=None) -> Status:
    """cuasr_b200_pack_k_contiguous: copies a rows x k operand (tensors or device addresses) into storage that is
    contiguous along k, dst[r * ld_dst + kk], from src[r + kk * ld_src] or (src_k_contiguous) src[r * ld_src + kk].
    A column-major A packed this way is passed on as a row-major A with leading dimension ld_dst."""
    return Status(_lib.load().cuasr_b200_pack_k_contiguous(int(dtype), _ptr(src), int(ld_src), int(bool(src_k_contiguous)),
                                                           int(rows), int(k), _ptr(dst), int(ld_dst),
                                                           _stream_handle(stream)))


def device_status(stream=None) -> int:
    """Synchronises `stream` and returns the device-side status word (0 = ok)."""
    return int(_lib.load().cuasr_b200_device_status(_stream_handle(stream)))


def launch_count() -> int:
    return int(_lib.load().cuasr_b200_launch_count())
