"""Path-tracking tropical product (cuasr_b200_srgemm_path) against the CPU restatement of the reference's
cpu_fwgemm_naive (test/regress/include/fwgpu/cpu_srgemm.hpp:20-48)."""
import numpy as np
import pytest

import oracle
import util
from cuasr_b200 import DType, Layout, Op, Srgemm, Status, device_status, srgemm_path
from cuasr_b200.semiring import NUMPY_DTYPE

COL, ROW = Layout.COLUMN_MAJOR, Layout.ROW_MAJOR


def test_oracle_path_distances_equal_the_pinned_srgemm_oracle():
    """The distance half of the path oracle is the min-plus SRGEMM with C = the old distances."""
    rng = np.random.default_rng(3)
    m, n, k = 37, 29, 41
    A = rng.integers(0, 9, m * k).astype(np.float32)
    B = rng.integers(0, 9, k * n).astype(np.float32)
    C = rng.integers(0, 30, m * n).astype(np.float32)
    want = util.run_oracle("minimum_plus", DType.F32, (COL, COL, COL), (m, n, k), 0.0, A, m, B, k, 0.0, C, m)
    dist, parent = oracle.srgemm_path(DType.F32, (COL, COL, COL), (m, n, k), A, m, B, k, C.copy(), m,
                                      np.full(m * n, -1, np.int32), m)
    assert np.array_equal(dist, want)
    # every recorded parent reproduces its distance, and it is the FIRST k that does
    Am, Bm = A.reshape(k, m).T, B.reshape(n, k).T
    P, Dm, Cm = parent.reshape(n, m).T, dist.reshape(n, m).T, C.reshape(n, m).T
    for i in range(m):
        for j in range(n):
            if P[i, j] >= 0:
                sums = Am[i, :] + Bm[:, j]
                assert Dm[i, j] < Cm[i, j] and sums[P[i, j]] == Dm[i, j] and np.argmin(sums) == P[i, j]
            else:
                assert Dm[i, j] == Cm[i, j]


def test_oracle_path_equals_the_reference_routine_on_committed_outputs():
    """Distances AND parents of the path oracle against outputs of the reference's own cpu_fwgemm_naive
    (tests/golden/fwgemm_outputs.npz, written by tests/golden/make_golden.py): inputs full of ties."""
    import golden_io
    cases = list(golden_io.fwgemm_cases())
    assert len(cases) == 6
    for c in cases:
        n, dt = c["n"], (DType.F32 if c["dtype"] == np.float32 else DType.F64)
        dist, parent = oracle.srgemm_path(dt, (COL, COL, COL), (n, n, n), c["A"], n, c["B"], n, c["dist_in"].copy(), n,
                                          c["parent_in"].copy(), n)
        assert np.array_equal(dist, c["dist_out"]), c["key"]
        assert np.array_equal(parent, c["parent_out"]), c["key"]
        assert (parent != c["parent_in"]).any() and (parent == c["parent_in"]).any()     # both branches occur


@pytest.mark.skipif(not oracle.have_ref_path(), reason="oracle/_ref/libcuasr_ref_path.so was not built")
def test_oracle_path_equals_the_reference_routine_live():
    rng = np.random.default_rng(8)
    for np_t, dt in ((np.float32, DType.F32), (np.float64, DType.F64)):
        for n in (1, 7, 33, 96):
            A = rng.integers(0, 5, n * n).astype(np_t)
            B = rng.integers(0, 5, n * n).astype(np_t)
            d0 = rng.integers(1, 8, n * n).astype(np_t)
            p0 = np.full(n * n, -1, np.int32)
            want_d, want_p = oracle.ref_fwgemm(A, B, d0.copy(), p0.copy(), n)
            got_d, got_p = oracle.srgemm_path(dt, (COL, COL, COL), (n, n, n), A, n, B, n, d0.copy(), n, p0.copy(), n)
            assert np.array_equal(got_d, want_d) and np.array_equal(got_p, want_p), (np_t.__name__, n)


@pytest.mark.gpu
def test_path_tracking_on_committed_reference_outputs(cuda_device):
    """The device kernel against the same committed outputs of the reference's routine."""
    import golden_io
    import torch
    for c in golden_io.fwgemm_cases():
        n, dt = c["n"], (DType.F32 if c["dtype"] == np.float32 else DType.F64)
        dA, dB = torch.from_numpy(c["A"]).cuda(), torch.from_numpy(c["B"]).cuda()
        dD, dP = torch.from_numpy(c["dist_in"].copy()).cuda(), torch.from_numpy(c["parent_in"].copy()).cuda()
        op = Srgemm(Op.MINIMUM, Op.PLUS, dt, COL, COL, COL)
        assert srgemm_path(op, (n, n, n), (dA, n), (dB, n), (dD, n), (dP, n)) == Status.kSuccess
        torch.cuda.synchronize()
        assert np.array_equal(dD.cpu().numpy(), c["dist_out"]) and np.array_equal(dP.cpu().numpy(), c["parent_out"]), c["key"]
    assert device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [DType.F32, DType.F64])
@pytest.mark.parametrize("maximize", [False, True])
def test_path_tracking_matches_oracle(cuda_device, dt, maximize):
    import torch
    rng = np.random.default_rng(19)
    np_t = NUMPY_DTYPE[dt]
    add_op = Op.MAXIMUM if maximize else Op.MINIMUM
    for layouts in (util.ALL_LAYOUTS[0], util.ALL_LAYOUTS[3], util.ALL_LAYOUTS[5], util.ALL_LAYOUTS[6]):
        for (m, n, k, integers) in ((1, 1, 1, True), (130, 67, 45, True), (257, 129, 100, False), (64, 64, 300, True)):
            A, lda = util.make_matrix(rng, dt, layouts[0], m, k, util.extents(layouts[0], m, k)[0] + 3)
            B, ldb = util.make_matrix(rng, dt, layouts[1], k, n, util.extents(layouts[1], k, n)[0] + 1)
            D, ldd = util.make_matrix(rng, dt, layouts[2], m, n, util.extents(layouts[2], m, n)[0] + 2, lo=-4, hi=4)
            if not integers:   # real values: ties are unlikely; integers: ties are the rule and test "first k wins"
                A = (A + rng.random(A.size)).astype(np_t)
                B = (B + rng.random(B.size)).astype(np_t)
            parent = np.full(D.size, -7, np.int32)
            want_d, want_p = oracle.srgemm_path(dt, layouts, (m, n, k), A, lda, B, ldb, D.copy(), ldd, parent.copy(), ldd,
                                                k_offset=1000, maximize=maximize)
            dA, dB, dD, dP = (torch.from_numpy(x).cuda() for x in (A, B, D, parent))
            op = Srgemm(add_op, Op.PLUS, dt, *layouts)
            st = srgemm_path(op, (m, n, k), (dA, lda), (dB, ldb), (dD, ldd), (dP, ldd), k_offset=1000)
            assert st == Status.kSuccess
            torch.cuda.synchronize()
            assert np.array_equal(dD.cpu().numpy(), want_d), (layouts, m, n, k)
            assert np.array_equal(dP.cpu().numpy(), want_p), (layouts, m, n, k)
    assert device_status() == 0
    bad = Srgemm(Op.PLUS, Op.MULTIPLIES, dt, COL, COL, COL)
    x = torch.zeros(16, device="cuda", dtype=torch.float32 if dt == DType.F32 else torch.float64)
    p = torch.zeros(16, device="cuda", dtype=torch.int32)
    assert srgemm_path(bad, (4, 4, 4), (x, 4), (x, 4), (x, 4), (p, 4)) == Status.kErrorNotSupported


@pytest.mark.gpu
@pytest.mark.parametrize("maximize", [False, True])
def test_path_tracking_on_the_tma_pipeline(cuda_device, maximize):
    """fp32 operands TMA can describe (16-byte aligned lines) take the pipelined kernel: all eight layouts, shapes
    ragged against the 128-wide tiles and the 32-deep K step, integer data (ties everywhere: the first k must win)
    and real data, existing distances and parents that must survive where nothing improves."""
    import torch
    rng = np.random.default_rng(23)
    dt = DType.F32
    add_op = Op.MAXIMUM if maximize else Op.MINIMUM
    for layouts in util.ALL_LAYOUTS:
        for (m, n, k, integers) in ((128, 128, 64, True), (300, 260, 77, True), (200, 136, 512, False), (64, 64, 33, True)):
            pad = lambda lay, r, c: (util.extents(lay, r, c)[0] + 3) // 4 * 4      # leading dimensions: multiples of 4
            A, lda = util.make_matrix(rng, dt, layouts[0], m, k, pad(layouts[0], m, k))
            B, ldb = util.make_matrix(rng, dt, layouts[1], k, n, pad(layouts[1], k, n))
            D, ldd = util.make_matrix(rng, dt, layouts[2], m, n, util.extents(layouts[2], m, n)[0] + 1, lo=-4, hi=4)
            if not integers:
                A = (A + rng.random(A.size)).astype(np.float32)
                B = (B + rng.random(B.size)).astype(np.float32)
            parent = np.full(D.size, -7, np.int32)
            want_d, want_p = oracle.srgemm_path(dt, layouts, (m, n, k), A, lda, B, ldb, D.copy(), ldd, parent.copy(), ldd,
                                                k_offset=500, maximize=maximize)
            dA, dB, dD, dP = (torch.from_numpy(x).cuda() for x in (A, B, D, parent))
            op = Srgemm(add_op, Op.PLUS, dt, *layouts)
            assert srgemm_path(op, (m, n, k), (dA, lda), (dB, ldb), (dD, ldd), (dP, ldd), k_offset=500) == Status.kSuccess
            torch.cuda.synchronize()
            assert op.last_kernel() == "path_tma", (op.last_kernel(), layouts, m, n, k)
            assert np.array_equal(dD.cpu().numpy(), want_d), (layouts, m, n, k)
            assert np.array_equal(dP.cpu().numpy(), want_p), (layouts, m, n, k)
    assert device_status() == 0


@pytest.mark.gpu
def test_path_tracking_at_4096_sampled(cuda_device):
    """One 4096^3 path-tracking product on uniform [0, 100) operands (distances start at +inf, parents at -1):
    distances equal the plain min-plus SRGEMM everywhere; distances and parents of sampled columns equal the host
    routine."""
    import torch
    from cuasr_b200 import Arguments
    from cuasr_b200.workloads import WORKLOADS
    wl = WORKLOADS["minplus_f32_4096"]
    n = wl.n
    dev = torch.device("cuda", 0)
    A, B = wl.operand("A", dev), wl.operand("B", dev)
    D = torch.full((n * n,), float("inf"), dtype=torch.float32, device=dev)
    P = torch.full((n * n,), -1, dtype=torch.int32, device=dev)
    op = Srgemm(Op.MINIMUM, Op.PLUS, DType.F32, COL, COL, COL, add_identity=float("inf"))
    assert srgemm_path(op, (n, n, n), (A, n), (B, n), (D, n), (P, n)) == Status.kSuccess
    torch.cuda.synchronize()
    assert op.last_kernel() == "path_tma"
    plain = torch.empty_like(D)
    C = torch.full_like(D, float("inf"))
    assert op(Arguments((n, n, n), (A, n), (B, n), (C, n), (plain, n), (0.0, 0.0))) == Status.kSuccess
    torch.cuda.synchronize()
    assert torch.equal(plain, D)
    hA = A.cpu().numpy()
    for c0 in (0, 2048, n - 8):
        hB = wl.operand("B", "cpu", c0 * n, 8 * n).numpy()
        d0 = np.full(8 * n, np.inf, np.float32)
        p0 = np.full(8 * n, -1, np.int32)
        want_d, want_p = oracle.srgemm_path(DType.F32, (COL, COL, COL), (n, 8, n), hA, n, hB, n, d0, n, p0, n)
        assert np.array_equal(D[c0 * n:(c0 + 8) * n].cpu().numpy(), want_d), c0
        assert np.array_equal(P[c0 * n:(c0 + 8) * n].cpu().numpy(), want_p), c0
    assert device_status() == 0
