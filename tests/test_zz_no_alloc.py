"""The allocation-free split-K entry point (cuasr_b200_srgemm_splitk_static).

It exists for callers that must not allocate device memory when they need a split-K product -- code hosted by a
framework that owns the whole device heap, or services under a "no allocation after start-up" rule -- so its
scratch is a static device array inside the library.  The test calls it through the C ABI twice in a row (the
second call meets the first call's leftovers in the shared array) and requires exactly the result of the
ordinary split-K entry point, which is deterministic.  This file sorts last on purpose, so that a run that
stops at the first failure has already run every other test; it also passes when run alone.
"""
import numpy as np
import pytest

import util
from cuasr_b200 import (Arguments, DType, Layout, Op, STATIC_SCRATCH_BYTES, Srgemm, SrgemmSplitKParallel, Status,
                        device_status, srgemm_splitk_static)

pytestmark = pytest.mark.gpu
ROW, COL = Layout.ROW_MAJOR, Layout.COLUMN_MAJOR


def test_static_scratch_matches_workspace_split_k(cuda_device):
    import torch

    rng = np.random.default_rng(41)
    m, n, k, slices = 256, 192, 8192, 8
    A = rng.random(m * k, dtype=np.float32)
    B = rng.random(k * n, dtype=np.float32)
    C = rng.random(m * n, dtype=np.float32) * 4
    dA, dB, dC = (torch.from_numpy(x).cuda() for x in (A, B, C))
    op = SrgemmSplitKParallel(Op.MINIMUM, Op.PLUS, DType.F32, ROW, COL, ROW)

    def arguments(dD):
        return Arguments((m, n, k), (dA, k), (dB, k), (dC, n), (dD, n), (0.0, 0.0), slices)

    # the existing entry point, with a caller-allocated workspace
    want = torch.zeros(m * n, device="cuda")
    ws = torch.empty(op.get_workspace_size(arguments(want)), dtype=torch.uint8, device="cuda")
    assert op(arguments(want), ws) == Status.kSuccess
    torch.cuda.synchronize()

    # the allocation-free entry point, two calls in a row on the same static scratch
    for attempt in range(2):
        got = torch.full((m * n,), -1.0, device="cuda")
        assert srgemm_splitk_static(op, arguments(got)) == Status.kSuccess
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {attempt + 1} differs from the workspace split-K result"
    assert device_status() == 0

    # and against the CPU oracle, so that "equal to the other entry point" cannot hide a shared mistake
    ref = util.run_oracle("minimum_plus", DType.F32, (ROW, COL, ROW), (m, n, k), 0.0, A, k, B, k, 0.0, C, n)
    assert np.array_equal(want.cpu().numpy(), ref)


def test_static_scratch_with_operands_the_fast_kernel_cannot_read(cuda_device):
    """The same entry point when an operand has an odd leading dimension: the split runs on the any-alignment
    kernel and its reduction kernel, partials in the static array, and must again equal the workspace entry point
    (two calls in a row) and the host SRGEMM."""
    import torch

    rng = np.random.default_rng(43)
    m, n, k, slices = 130, 200, 1027, 4
    lda = k + 1                                           # row-major A with an odd leading dimension
    A = rng.integers(-8, 9, size=m * lda).astype(np.float32)
    B = rng.integers(-8, 9, size=k * n).astype(np.float32)
    C = rng.integers(-8, 9, size=m * n).astype(np.float32)
    dA, dB, dC = (torch.from_numpy(x).cuda() for x in (A, B, C))
    op = SrgemmSplitKParallel(Op.MINIMUM, Op.PLUS, DType.F32, ROW, COL, ROW)

    def arguments(dD):
        return Arguments((m, n, k), (dA, lda), (dB, k), (dC, n), (dD, n), (0.0, 0.0), slices)

    want = torch.zeros(m * n, device="cuda")
    ws = torch.empty(op.get_workspace_size(arguments(want)), dtype=torch.uint8, device="cuda")
    assert op(arguments(want), ws) == Status.kSuccess
    torch.cuda.synchronize()
    assert op.last_kernel() == "generic_splitk"
    for attempt in range(2):
        got = torch.full((m * n,), -1.0, device="cuda")
        assert srgemm_splitk_static(op, arguments(got)) == Status.kSuccess
        torch.cuda.synchronize()
        assert op.last_kernel() == "generic_splitk"
        assert torch.equal(got, want), f"call {attempt + 1} differs from the workspace split-K result"
    assert device_status() == 0
    ref = util.run_oracle("minimum_plus", DType.F32, (ROW, COL, ROW), (m, n, k), 0.0, A, lda, B, k, 0.0, C, n)
    assert np.array_equal(want.cpu().numpy(), ref)


def test_static_scratch_rejects_oversized_problems(cuda_device):
    import torch

    m = n = 1024
    k, slices = 256, 8          # 8 slices of a 1024 x 1024 fp32 result need 32 MiB of partials
    x = torch.zeros(m * k, device="cuda")
    y = torch.zeros(m * n, device="cuda")
    op = SrgemmSplitKParallel(Op.MINIMUM, Op.PLUS, DType.F32, ROW, COL, ROW)
    args = Arguments((m, n, k), (x, k), (x, k), (y, n), (y, n), (0.0, 0.0), slices)
    assert op.get_workspace_size(args) > STATIC_SCRATCH_BYTES
    assert srgemm_splitk_static(op, args) == Status.kErrorStaticScratchTooSmall
