"""Outputs with more than 2^31 elements: every offset in the kernels must be 64-bit.  Whole-matrix comparison is
out of reach for the host SRGEMM at this size, so storage lines at the start, across the 2^31-element offset and
at the very end are compared bit for bit, and a size-independent property covers the rest: the in-place update
D <- D (+) A (x) B is idempotent, so a second call must leave all of D unchanged."""
import numpy as np
import pytest

import util
from cuasr_b200 import Arguments, DType, Layout, RINGS, Srgemm, Status

pytestmark = pytest.mark.gpu
COL, ROW = Layout.COLUMN_MAJOR, Layout.ROW_MAJOR


@pytest.mark.parametrize("layouts,lines,contig,kernel", [
    ((ROW, COL, ROW), 70000, 40000, "tma"),        # row-major D, both operands K-contiguous
    ((COL, ROW, COL), 33000, 70001, "generic"),    # column-major D with an odd leading dimension
])
def test_output_beyond_two_to_the_31_elements(cuda_device, layouts, lines, contig, kernel):
    import torch
    free, _ = torch.cuda.mem_get_info()
    if free < 30e9:
        pytest.skip("needs 30 GB of free device memory")
    k = 8
    row_c = layouts[2] == ROW
    m, n = (lines, contig) if row_c else (contig, lines)
    assert lines * contig > 2 ** 31
    g = torch.Generator(device="cuda").manual_seed(lines)
    A = torch.randint(-8, 9, (m * k,), generator=g, device="cuda").float()
    B = torch.randint(-8, 9, (k * n,), generator=g, device="cuda").float()
    D = torch.empty(lines * contig, dtype=torch.float32, device="cuda")
    pattern = (torch.arange(contig, device="cuda") % 13 - 6).float()
    D.view(lines, contig).copy_(pattern.expand(lines, contig))
    add_op, mul_op = RINGS["minimum_plus"]
    op = Srgemm(add_op, mul_op, DType.F32, *layouts)
    lda = k if layouts[0] == ROW else m
    ldb = n if layouts[1] == ROW else k
    args = Arguments((m, n, k), (A, lda), (B, ldb), (D, contig), (D, contig), (0.0, 0.0))   # C aliases D
    assert op(args) == Status.kSuccess
    torch.cuda.synchronize()
    assert kernel in op.last_kernel()

    hA, hB, hp = A.cpu().numpy(), B.cpu().numpy(), pattern.cpu().numpy()
    straddle = 2 ** 31 // contig
    for l0 in (0, straddle - 15, lines - 32):
        # the sub-problem that produces storage lines [l0, l0 + 32) of D
        if row_c:      # lines are rows of D: rows l0.. of A (row-major, contiguous), all of B
            sub_mnk, sA, sB = (32, n, k), hA[l0 * k:(l0 + 32) * k], hB
        else:          # lines are columns of D: all of A, columns l0.. of B (row-major: same ld, shifted start)
            sub_mnk, sA, sB = (m, 32, k), hA, hB[l0:]
        C0 = np.tile(hp, 32)
        want = util.run_oracle("minimum_plus", DType.F32, layouts, sub_mnk, 0.0, sA, lda, sB, ldb, 0.0, C0, contig)
        got = D[l0 * contig:(l0 + 32) * contig].cpu().numpy()
        assert np.array_equal(got, want), f"lines {l0}..{l0 + 32}"

    before = torch.empty_like(D).copy_(D)
    assert op(args) == Status.kSuccess
    torch.cuda.synchronize()
    assert torch.equal(before, D)
