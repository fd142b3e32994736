"""Host-side logic of the C ABI that needs no GPU: argument validation, status codes and workspace sizes, called
through the library with made-up (never dereferenced) pointers."""
import numpy as np
import pytest

from cuasr_b200 import Arguments, DType, Layout, Op, Srgemm, SrgemmSplitKParallel, Status, annihilator, identity

COL, ROW = Layout.COLUMN_MAJOR, Layout.ROW_MAJOR
P = 0x10000  # a fake, 16-byte aligned device address


def args(m=256, n=256, k=256, lda=256, ldb=256, ldc=256, ldd=256, a=P, b=P, c=P, d=P, slices=1, epilogue=(0.0, 0.0)):
    return Arguments((m, n, k), (a, lda), (b, ldb), (c, ldc), (d, ldd), epilogue, slices)


def test_can_implement_follows_the_reference_rules():
    op = Srgemm(Op.MINIMUM, Op.PLUS, DType.F32, COL, COL, COL)
    assert op.can_implement(args()) == Status.kSuccess
    assert op.can_implement(args(slices=2)) == Status.kErrorInvalidProblem          # device/srgemm.h:198-200
    assert op.can_implement(args(m=0)) == Status.kErrorInvalidProblem
    # A and B are only read: a short leading dimension is an overlapping view, accepted like the reference does
    assert op.can_implement(args(lda=100)) == Status.kSuccess
    assert op.can_implement(args(lda=0)) == Status.kErrorInvalidProblem
    assert op.can_implement(args(ldd=100)) == Status.kErrorInvalidProblem           # overlapping lines of D would race
    assert op.can_implement(args(a=P + 2)) == Status.kErrorMisalignedOperand
    assert op.can_implement(args(a=None)) == Status.kErrorInvalidProblem
    serial = Srgemm(Op.MINIMUM, Op.PLUS, DType.F32, COL, COL, COL, split_k_serial=True)
    assert serial.can_implement(args(slices=8)) == Status.kSuccess
    assert SrgemmSplitKParallel(Op.MINIMUM, Op.PLUS, DType.F32, ROW, COL, ROW).can_implement(args(slices=8)) \
        == Status.kSuccess


def test_layout_decides_the_minimum_leading_dimension():
    op = Srgemm(Op.PLUS, Op.MULTIPLIES, DType.F64, ROW, COL, ROW)
    # A is 100 x 300 row-major, B is 300 x 50 column-major, C and D are 100 x 50 row-major (ld >= 50)
    ok = args(m=100, n=50, k=300, lda=300, ldb=300, ldc=50, ldd=50, epilogue=(1.0, 0.0))
    assert op.can_implement(ok) == Status.kSuccess
    assert op.can_implement(args(m=100, n=50, k=300, lda=299, ldb=300, ldc=50, ldd=50)) == Status.kSuccess
    assert op.can_implement(args(m=100, n=50, k=300, lda=300, ldb=300, ldc=49, ldd=50, epilogue=(1.0, 1.0))) \
        == Status.kErrorInvalidProblem
    assert op.can_implement(args(m=100, n=50, k=300, lda=300, ldb=300, ldc=50, ldd=49)) == Status.kErrorInvalidProblem
    assert op.can_implement(args(m=100, n=50, k=300, lda=300, ldb=300, ldc=50, ldd=50, d=P + 4)) \
        == Status.kErrorMisalignedOperand                                              # 8-byte elements


def test_unsupported_combinations():
    assert Srgemm(Op.BIT_XOR, Op.BIT_AND, DType.F32, COL, COL, COL).can_implement(args()) == Status.kErrorNotSupported
    assert Srgemm(Op.PLUS, Op.PLUS, DType.F32, COL, COL, COL).can_implement(args()) == Status.kErrorNotSupported
    assert Srgemm(Op.BIT_XOR, Op.BIT_AND, DType.U32, COL, COL, COL).can_implement(args()) == Status.kSuccess


def test_workspace_sizes():
    unsplit = Srgemm(Op.MINIMUM, Op.PLUS, DType.F32, COL, COL, COL)
    assert unsplit.get_workspace_size(args()) == 0                                      # device/srgemm.h:218-234
    par = SrgemmSplitKParallel(Op.MINIMUM, Op.PLUS, DType.F32, ROW, COL, ROW)
    a16 = args(m=256, n=256, k=1 << 20, lda=1 << 20, ldb=1 << 20, slices=16)
    need = par.get_workspace_size(a16)
    # at least what the reference asks for: sizeof(element) * M * N * slices (device/srgemm_splitk_parallel.h:226-235)
    assert need >= 4 * 256 * 256 * 16
    # no more than that where no GPU is visible; with a GPU each slice may be cut further to fill its SMs
    gpu_visible = par._lib.cuasr_b200_device_status(None) >= 0
    assert need <= (4 * 256 * 256 * 16 + 4096) * (8 if gpu_visible else 1)
    assert par.get_workspace_size(args(m=256, n=256, k=1 << 20, lda=1 << 20, ldb=1 << 20, slices=32)) >= need
    f64 = SrgemmSplitKParallel(Op.MINIMUM, Op.PLUS, DType.F64, ROW, COL, ROW)
    assert f64.get_workspace_size(a16) >= 2 * (need - 4096)
    # ragged shapes are padded to whole 128 x 128 tiles
    assert par.get_workspace_size(args(m=130, n=70, k=1000, lda=1000, ldb=1000, ldc=70, ldd=70, slices=3)) \
        >= 4 * 2 * 1 * 128 * 128 * 3


def test_reference_constants():
    """functional.h:28-36: '+inf' is numeric_limits::max(), '-inf' is numeric_limits::min()."""
    assert identity(Op.MINIMUM, DType.F32) == np.finfo(np.float32).max
    assert identity(Op.MAXIMUM, DType.F32) == np.finfo(np.float32).tiny
    assert identity(Op.MAXIMUM, DType.S32) == np.iinfo(np.int32).min
    assert annihilator(Op.PLUS, DType.F64) == np.finfo(np.float64).max
    assert identity(Op.MINIMUM, DType.F32, true_infinity=True) == np.inf
    assert identity(Op.BIT_AND, DType.U32) == 0xFFFFFFFF and identity(Op.BIT_XOR, DType.U32) == 0
    assert annihilator(Op.MULTIPLIES, DType.F32) == 0 and identity(Op.MULTIPLIES, DType.F32) == 1


def test_run_before_initialize_and_update():
    op = Srgemm(Op.MINIMUM, Op.PLUS, DType.F32, COL, COL, COL)
    assert op.run() == Status.kErrorInternal
    assert op.update(args()) == Status.kErrorInternal
    assert op.initialize(args(slices=2)) == Status.kErrorInvalidProblem
    assert op.initialize(args()) == Status.kSuccess
    assert op.update(args(a=P + 4096)) == Status.kSuccess


def test_shares_of_the_shared_operand_tile_it_exactly_once():
    """Sharded host-buffer SRGEMM: every rank brings 1/world of every K piece of the operand all ranks need; together
    the shares must cover the operand once, piece by piece, and a rank's host tensor holds its ranges back to back."""
    from cuasr_b200.host_pipeline import share_ranges
    for elems, pieces, world in ((8192 * 8192, 4, 8), (1024 * 640, 4, 2), (4096, 1, 4), (96, 4, 3)):
        covered = np.zeros(elems, dtype=np.int32)
        for rank in range(world):
            ranges = share_ranges(elems, pieces, rank, world)
            assert len(ranges) == pieces
            assert all(b - a == elems // (pieces * world) for a, b in ranges)
            # piece p of this rank lies inside piece p of the operand
            assert all(p * (elems // pieces) <= a and b <= (p + 1) * (elems // pieces) for p, (a, b) in enumerate(ranges))
            for a, b in ranges:
                covered[a:b] += 1
        assert (covered == 1).all()
    with pytest.raises(ValueError):
        share_ranges(100, 4, 0, 3)


def test_numa_local_leaves_the_process_as_it_found_it():
    """numa_local moves the process next to a GPU's host link for the length of a block and puts the CPU affinity
    back; where the system does not tell the topology (no GPU here) it does nothing at all."""
    import os
    from cuasr_b200.host_pipeline import device_numa_node, numa_local
    before = os.sched_getaffinity(0)
    node, cpus = device_numa_node(0)
    assert node is None or cpus <= before
    with numa_local(0) as where:
        inside = os.sched_getaffinity(0)
        assert inside <= before and (where.node is not None or inside == before)
    assert os.sched_getaffinity(0) == before


def test_pack_k_contiguous_checks_its_arguments_before_touching_a_device():
    from cuasr_b200 import pack_k_contiguous
    ok = dict(dtype=DType.F32, src=4096, ld_src=16, src_k_contiguous=False, rows=16, k=8, dst=8192, ld_dst=8)
    call = lambda **kw: pack_k_contiguous(**dict(ok, **kw))
    assert call(src=0) == Status.kErrorInvalidProblem
    assert call(dst=0) == Status.kErrorInvalidProblem
    assert call(rows=0) == Status.kErrorInvalidProblem
    assert call(ld_dst=7) == Status.kErrorInvalidProblem                      # shorter than a line of the copy
    assert call(ld_src=15) == Status.kErrorInvalidProblem                     # shorter than a line of the source
    assert call(src_k_contiguous=True, ld_src=7) == Status.kErrorInvalidProblem
    assert call(src=4098) == Status.kErrorMisalignedOperand
    assert call(dtype=DType.F64, dst=8196) == Status.kErrorMisalignedOperand
    import ctypes
    from cuasr_b200 import _lib
    assert _lib.load().cuasr_b200_pack_k_contiguous(99, 4096, 16, 0, 16, 8, 8192, 8, None) == int(Status.kErrorInvalidDataType)
