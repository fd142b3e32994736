"""Pins the CPU oracle (oracle/srgemm_oracle.c) to the reference: its own known-answer test, outputs of its own
host SRGEMM (committed fixtures), and -- where oracle/_ref has been built -- that host SRGEMM run live."""
import numpy as np
import pytest

import golden_io
import oracle
import util
from cuasr_b200 import DType, Layout, Op, identity
from cuasr_b200.semiring import NUMPY_DTYPE

COL = Layout.COLUMN_MAJOR


def test_known_answer_4x4x2_min_plus():
    """test/regress/Srgemm_test.cu:15-62: C = min(C, A (x) B), column-major, compared with EXPECT_FLOAT_EQ."""
    ka = golden_io.known_answer()
    a, b, c, want = (np.array(ka[k]["data"], dtype=np.float32) for k in ("a", "b", "c", "correct"))
    d = np.zeros(16, np.float32)
    oracle.srgemm(Op.MINIMUM, Op.PLUS, DType.F32, (COL, COL, COL), (4, 4, 2), 0.0, a, 4, b, 2, 0.0, c, 4, d, 4,
                  identity(Op.MINIMUM, DType.F32))
    # EXPECT_FLOAT_EQ is a 4-ulp comparison
    assert np.all(np.abs(d - want) <= 4 * np.spacing(np.abs(want)))
    # exactly one entry is improved by the product, and it is the float32 sum the definition gives
    A, B, Cm, Dm = a.reshape(2, 4).T, b.reshape(4, 2).T, c.reshape(4, 4).T, d.reshape(4, 4).T
    changed = np.argwhere(Dm != Cm)
    assert len(changed) == 1
    i, j = changed[0]
    assert Dm[i, j] == min(A[i, 0] + B[0, j], A[i, 1] + B[1, j])


def test_matches_committed_reference_outputs():
    n = 0
    for case in golden_io.host_cases():
        ring, dt, layouts, (m, nn, k) = case["ring"], case["dtype"], case["layouts"], case["mnk"]
        lda, ldb, ldc = (util.extents(layouts[0], m, k)[0], util.extents(layouts[1], k, nn)[0],
                         util.extents(layouts[2], m, nn)[0])
        alpha, beta = util.default_scalars(ring, dt)
        for tag, be in (("D_ann", beta), ("D_id", alpha)):
            got = util.run_oracle(ring, dt, layouts, (m, nn, k), alpha, case["A"], lda, case["B"], ldb, be,
                                  case["C"], ldc)
            util.assert_equal(got, case[tag], layouts[2], m, nn, ldc, what=f"{case['key']} {tag}")
            n += 1
    assert n >= 600


@pytest.mark.skipif(not oracle.have_ref(), reason="oracle/_ref (the reference's host SRGEMM) is not built here")
@pytest.mark.parametrize("ring,dt", list(util.ring_dtype_cases()))
def test_matches_live_reference(ring, dt):
    """The reference's ragged grid M in {1, 509}, N in {1, 510}, K in {1, 23} (test/device/testbed.h:313-319),
    sub-matrices with ld > extent, and a non-default additive identity."""
    rng = np.random.default_rng(hash((ring, int(dt))) & 0xFFFF)
    alpha, beta = util.default_scalars(ring, dt)
    for layouts in (util.ALL_LAYOUTS[0], util.ALL_LAYOUTS[3], util.ALL_LAYOUTS[6]):
        for (m, n, k, pad) in ((1, 1, 1, 0), (509, 510, 23, 0), (1, 510, 23, 3), (509, 1, 1, 5), (37, 41, 64, 7)):
            A, lda = util.make_matrix(rng, dt, layouts[0], m, k, util.extents(layouts[0], m, k)[0] + pad)
            B, ldb = util.make_matrix(rng, dt, layouts[1], k, n, util.extents(layouts[1], k, n)[0] + pad)
            C, ldc = util.make_matrix(rng, dt, layouts[2], m, n, util.extents(layouts[2], m, n)[0] + pad)
            for be in (beta, alpha):
                got = util.run_oracle(ring, dt, layouts, (m, n, k), alpha, A, lda, B, ldb, be, C, ldc)
                want = util.run_oracle(ring, dt, layouts, (m, n, k), alpha, A, lda, B, ldb, be, C, ldc, use_ref=True)
                util.assert_equal(got, want, layouts[2], m, n, ldc, what=f"{ring} {dt.name} {m}x{n}x{k}")
    # additive identity is an argument of the host SRGEMM (host_srgemm.h:41), not a constant
    if dt in (DType.F32, DType.F64):
        ident = NUMPY_DTYPE[dt](3)
        got = util.run_oracle(ring, dt, util.ALL_LAYOUTS[0], (5, 6, 7), alpha, A[:35], 5, B[:42], 7, beta, C[:30], 5,
                              add_identity=ident)
        want = util.run_oracle(ring, dt, util.ALL_LAYOUTS[0], (5, 6, 7), alpha, A[:35], 5, B[:42], 7, beta, C[:30], 5,
                               add_identity=ident, use_ref=True)
        util.assert_equal(got, want, COL, 5, 6, 5)


def test_min_plus_against_numpy_definition():
    """Independent restatement: D[i, j] = min(min_k A[i, k] + B[k, j], C[i, j]) in float32."""
    rng = np.random.default_rng(7)
    m, n, k = 70, 45, 33
    A = rng.random(m * k, dtype=np.float32) * 100
    B = rng.random(k * n, dtype=np.float32) * 100
    C = rng.random(m * n, dtype=np.float32) * 100
    got = util.run_oracle("minimum_plus", DType.F32, (COL, COL, COL), (m, n, k), 0.0, A, m, B, k, 0.0, C, m)
    Am, Bm, Cm = A.reshape(k, m).T, B.reshape(n, k).T, C.reshape(n, m).T
    want = np.minimum((Am[:, :, None] + Bm[None, :, :]).min(axis=1), Cm)
    assert np.array_equal(got.reshape(n, m).T, want)


def test_threads_do_not_change_the_result():
    rng = np.random.default_rng(11)
    m, n, k = 130, 97, 50
    A = rng.random(m * k) - 0.5
    B = rng.random(k * n) - 0.5
    C = np.zeros(m * n)
    outs = []
    for threads in (1, 4):
        D = np.zeros(m * n)
        oracle.srgemm(Op.PLUS, Op.MULTIPLIES, DType.F64, (COL, COL, COL), (m, n, k), 1.0, A, m, B, k, 0.0, C, m, D, m,
                      0.0, threads)
        outs.append(D)
    assert np.array_equal(outs[0], outs[1])
