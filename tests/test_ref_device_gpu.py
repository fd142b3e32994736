"""The new kernels against the reference's own device kernels (recompiled for sm_100a into oracle/_ref), on the
GPU, bit for bit.  Skipped where that library was not built."""
import numpy as np
import pytest

import oracle
from cuasr_b200 import Arguments, DType, Layout, RINGS, Srgemm, Status

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not oracle.have_ref_device(),
                                                  reason="oracle/_ref/libcuasr_ref_device.so was not built")]
COL = Layout.COLUMN_MAJOR
CASES = [("minimum_plus", DType.F32, 0.0, 0.0), ("minimum_plus", DType.F64, 0.0, 0.0),
         ("maximum_plus", DType.F64, 0.0, 0.0), ("maximum_minimum", DType.F32, np.inf, np.inf)]


@pytest.mark.parametrize("ring,dtype,alpha,beta", CASES)
@pytest.mark.parametrize("shape", [(512, 512, 512), (509, 130, 23), (257, 384, 1000)])
def test_same_bits_as_the_reference_device_kernel(ring, dtype, alpha, beta, shape):
    import torch
    m, n, k = shape
    tdt = torch.float32 if dtype == DType.F32 else torch.float64
    g = torch.Generator(device="cuda").manual_seed(m * 7 + k)
    # integer-valued operands as in the reference's testbed: every sum is exact in both element types
    A = torch.randint(-8, 9, (m * k,), generator=g, device="cuda").to(tdt)
    B = torch.randint(-8, 9, (k * n,), generator=g, device="cuda").to(tdt)
    C = torch.randint(-8, 9, (m * n,), generator=g, device="cuda").to(tdt)
    ours, theirs = torch.zeros(m * n, dtype=tdt, device="cuda"), torch.zeros(m * n, dtype=tdt, device="cuda")
    add_op, mul_op = RINGS[ring]
    op = Srgemm(add_op, mul_op, dtype, COL, COL, COL)      # the reference's constants for the identities
    args = Arguments((m, n, k), (A, m), (B, k), (C, m), (ours, m), (alpha, beta))
    assert op(args) == Status.kSuccess
    st = oracle.ref_device_srgemm(add_op, mul_op, dtype, shape, A.data_ptr(), m, B.data_ptr(), k, C.data_ptr(), m,
                                  theirs.data_ptr(), m, alpha, beta, torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    assert torch.equal(ours, theirs)
