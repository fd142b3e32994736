"""Shared helpers of the parity tests: seeded inputs, the oracle call and the library call on the same buffers."""
from __future__ import annotations

import itertools

import numpy as np

import oracle
from cuasr_b200 import Arguments, DType, Layout, Op, RINGS, Srgemm, SrgemmSplitKParallel, Status, annihilator, identity
from cuasr_b200.semiring import INTEGER_ONLY_RINGS, NUMPY_DTYPE

ALL_LAYOUTS = list(itertools.product((Layout.COLUMN_MAJOR, Layout.ROW_MAJOR), repeat=3))
FLOAT_RINGS = [r for r in RINGS if r not in INTEGER_ONLY_RINGS]


def ring_dtype_cases(dtypes=(DType.F32, DType.F64, DType.S32, DType.U32)):
    for name in RINGS:
        for dt in dtypes:
            if name in INTEGER_ONLY_RINGS and dt in (DType.F32, DType.F64):
                continue
            yield name, dt


def extents(layout, rows, cols):
    """(contiguous extent, number of lines) of a rows x cols matrix in `layout`."""
    return (cols, rows) if layout == Layout.ROW_MAJOR else (rows, cols)


def make_matrix(rng, dtype, layout, rows, cols, ld=None, lo=-8, hi=8, values=None):
    """A flat buffer holding a rows x cols matrix with leading dimension ld (>= contiguous extent).

    Values are small integers like the reference's test bed uses (test/device/testbed.h:85-108:
    uniform in [-8, 8] with zero fractional bits), so every ring is exact in every element type.
    """
    np_t = NUMPY_DTYPE[dtype]
    contig, lines = extents(layout, rows, cols)
    ld = contig if ld is None else ld
    assert ld >= contig
    if values is None:
        if np_t == np.uint32:
            lo = max(lo, 0)
        buf = rng.integers(lo, hi + 1, size=ld * lines).astype(np_t)
    else:
        buf = values(ld * lines).astype(np_t)
    return buf, ld


def as_2d(buf, layout, rows, cols, ld):
    """View of the logical rows x cols matrix inside a flat buffer."""
    if layout == Layout.ROW_MAJOR:
        return buf[: rows * ld].reshape(rows, ld)[:, :cols]
    return buf[: cols * ld].reshape(cols, ld)[:, :rows].T


def run_oracle(ring, dtype, layouts, mnk, alpha, A, lda, B, ldb, beta, C, ldc, ldd=None, add_identity=None,
               use_ref=False, D_init=None):
    add_op, mul_op = RINGS[ring]
    m, n, k = mnk
    ldd = ldc if ldd is None else ldd
    contig, lines = extents(layouts[2], m, n)
    D = np.zeros(ldd * lines, dtype=NUMPY_DTYPE[dtype]) if D_init is None else D_init.copy()
    ident = identity(add_op, dtype) if add_identity is None else add_identity
    fn = oracle.ref_srgemm if use_ref else oracle.srgemm
    fn(add_op, mul_op, dtype, layouts, mnk, alpha, A, lda, B, ldb, beta, C, ldc, D, ldd, ident)
    return D


def run_device(ring, dtype, layouts, mnk, alpha, A, lda, B, ldb, beta, C, ldc, ldd=None, add_identity=None,
               split_k_slices=1, parallel_splitk=False, split_k_serial=False, D_init=None, alias_c=False,
               expect=Status.kSuccess):
    """Runs the library on copies of the host buffers; returns (D as numpy, name of the kernel used)."""
    import torch

    add_op, mul_op = RINGS[ring]
    m, n, k = mnk
    ldd = ldc if ldd is None else ldd
    np_t = NUMPY_DTYPE[dtype]
    contig, lines = extents(layouts[2], m, n)

    def dev(x):
        # uint32 has no torch dtype with full support: ship the bits as int32
        return torch.from_numpy(x.view(np.int32) if x.dtype == np.uint32 else x).cuda()

    dA, dB = dev(A), dev(B)
    dC = dev(C) if C is not None else None
    if alias_c:
        dD = dC
    else:
        dD = dev(np.zeros(ldd * lines, dtype=np_t) if D_init is None else D_init)
    cls = SrgemmSplitKParallel if parallel_splitk else Srgemm
    ident = identity(add_op, dtype) if add_identity is None else add_identity
    op = cls(add_op, mul_op, dtype, *layouts, split_k_serial=split_k_serial, add_identity=ident)
    args = Arguments((m, n, k), (dA, lda), (dB, ldb), (dC, ldc), (dD, ldd), (alpha, beta), split_k_slices)
    ws = None
    need = op.get_workspace_size(args)
    if need:
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    status = op(args, ws)
    assert status == expect, f"status {status!r}, expected {expect!r}"
    torch.cuda.synchronize()
    out = dD.cpu().numpy()
    return (out.view(np.uint32) if np_t == np.uint32 else out), op.last_kernel()


def default_scalars(ring, dtype):
    """alpha = mult identity, beta = mult annihilator: what TestAllGemm uses (test/device/testbed.h:324-325)."""
    add_op, mul_op = RINGS[ring]
    return identity(mul_op, dtype), annihilator(mul_op, dtype)


def annihilator_beta_is_defined(ring, dtype):
    """False where beta = mult annihilator makes the host SRGEMM's `mult(beta, C)` overflow: for integer element
    types the annihilator of `plus` is numeric_limits::max() (functional.h:42), max() + C wraps (undefined for
    signed), and the device epilogue does not even read C then (semiring_linear_combination.h:118-125).  The
    reference only tests float and double (test/device/simt_sm50.py:27-33); integer cases use beta = identity."""
    return not (dtype in (DType.S32, DType.U32) and RINGS[ring][1] == Op.PLUS)


def assert_equal(got, want, layout, m, n, ld, what=""):
    """Value equality on the logical matrix, like cutlass TensorEquals (test/device/testbed.h:159-160)."""
    g, w = as_2d(got, layout, m, n, ld), as_2d(want, layout, m, n, ld)
    bad = ~((g == w) | (np.isnan(g.astype(np.float64)) & np.isnan(w.astype(np.float64))))
    if bad.any():
        idx = np.argwhere(bad)[0]
        raise AssertionError(f"{what}: {bad.sum()} of {bad.size} differ; first at {tuple(idx)}: "
                             f"got {g[tuple(idx)]!r}, want {w[tuple(idx)]!r}")
