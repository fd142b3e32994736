"""Parity of the CUDA library (through the C ABI) with the CPU oracle.  Bit-exact (value equality, like
cutlass TensorEquals) for every ring except plus-times on non-integer data, which gets a stated tolerance."""
import numpy as np
import pytest

import golden_io
import util
from cuasr_b200 import (Arguments, DType, Layout, Op, RINGS, Srgemm, SrgemmSplitKParallel, Status, annihilator,
                        device_status, identity)
from cuasr_b200.semiring import NUMPY_DTYPE

pytestmark = pytest.mark.gpu
COL, ROW = Layout.COLUMN_MAJOR, Layout.ROW_MAJOR


def _check(ring, dt, layouts, mnk, rng, pad=0, beta_is_identity=False, expect_kernel=None, **kw):
    m, n, k = mnk
    A, lda = util.make_matrix(rng, dt, layouts[0], m, k, util.extents(layouts[0], m, k)[0] + pad)
    B, ldb = util.make_matrix(rng, dt, layouts[1], k, n, util.extents(layouts[1], k, n)[0] + pad)
    C, ldc = util.make_matrix(rng, dt, layouts[2], m, n, util.extents(layouts[2], m, n)[0] + pad)
    alpha, beta = util.default_scalars(ring, dt)
    if beta_is_identity or not util.annihilator_beta_is_defined(ring, dt):
        beta = alpha
    if ring == "maximum_plus" and dt == DType.U32 and beta == 0:
        # numeric_limits<unsigned>::min() == 0 makes maximum::Identity equal plus::Identity, so the device-side
        # rule "C is read unless mult(beta, 1x) == 0+" (semiring_linear_combination.h:118-125) drops C for
        # beta = 0 while the host SRGEMM always reads it; beta = 1 keeps both sides on the same formula
        beta = NUMPY_DTYPE[dt](1)
    canary = np.full_like(C, 77)
    want = util.run_oracle(ring, dt, layouts, mnk, alpha, A, lda, B, ldb, beta, C, ldc, D_init=canary)
    got, kernel = util.run_device(ring, dt, layouts, mnk, alpha, A, lda, B, ldb, beta, C, ldc, D_init=canary, **kw)
    what = f"{ring} {dt.name} {[int(x) for x in layouts]} {mnk} pad={pad} kernel={kernel}"
    util.assert_equal(got, want, layouts[2], m, n, ldc, what=what)
    # nothing outside the logical matrix may be written (the padding of each line keeps its canary)
    assert np.array_equal(got, want), f"{what}: bytes outside the matrix were modified"
    if expect_kernel is not None:
        assert kernel == expect_kernel, what
    return kernel


@pytest.mark.parametrize("ring,dt", list(util.ring_dtype_cases()))
def test_reference_grid(cuda_device, ring, dt):
    """TestAllGemm's grid (test/device/testbed.h:313-358): M in {1, 509}, N in {1, 510}, K in {1, 23}, all eight
    layout combinations, alpha = mult identity, beta = mult annihilator, integers in [-8, 8]."""
    rng = np.random.default_rng(2080)
    for layouts in util.ALL_LAYOUTS:
        for m in (1, 509):
            for n in (1, 510):
                for k in (1, 23):
                    _check(ring, dt, layouts, (m, n, k), rng)
    assert device_status() == 0


@pytest.mark.parametrize("ring,dt", [(r, d) for r, d in util.ring_dtype_cases() if d in (DType.F32, DType.F64, DType.U32)])
def test_tma_kernel_ragged_but_aligned(cuda_device, ring, dt):
    """16-byte aligned operands take the TMA kernel; M, N, K tails are not multiples of the tile."""
    from cuasr_b200.srgemm import _lib
    rng = np.random.default_rng(99)
    kernels = set()
    for layouts in util.ALL_LAYOUTS:
        for mnk in ((260, 392, 100), (128, 128, 32), (132, 516, 36)):
            for beta_id in (False, True):
                kernels.add(_check(ring, dt, layouts, mnk, rng, beta_is_identity=beta_id))
    assert device_status() == 0
    fast = {"minimum_plus", "maximum_plus", "minimum_maximum", "maximum_minimum", "plus_multiplies",
            "minimum_multiplies", "maximum_multiplies"}
    if dt in (DType.F32, DType.F64) and ring in fast:
        assert kernels == {"tma"}, kernels     # plus-times fp64 is the tensor-core (DMMA) variant of that kernel
    if dt == DType.U32 and ring in ("bit_xor_bit_and", "bit_or_bit_and", "bit_xor_binary_and"):
        assert kernels == {"tma"}, kernels


def test_config_minplus_f32_512_cube(cuda_device):
    """Min-plus fp32, M = N = K = 512, column-major, A and B uniform in [0, 100), C filled with the additive
    identity, alpha = beta = 0 (the multiplicative identity of min-plus): bit-exact."""
    rng = np.random.default_rng(3090)
    n = 512
    A = (rng.random(n * n, dtype=np.float32) * 100).astype(np.float32)
    B = (rng.random(n * n, dtype=np.float32) * 100).astype(np.float32)
    ident = identity(Op.MINIMUM, DType.F32)
    C = np.full(n * n, ident, np.float32)
    layouts = (COL, COL, COL)
    want = util.run_oracle("minimum_plus", DType.F32, layouts, (n, n, n), 0.0, A, n, B, n, 0.0, C, n)
    got, kernel = util.run_device("minimum_plus", DType.F32, layouts, (n, n, n), 0.0, A, n, B, n, 0.0, C, n)
    assert kernel == "tma"
    assert np.array_equal(got, want)
    # with true infinities as identity and fill the finite entries are the same
    inf = np.float32(np.inf)
    got2, _ = util.run_device("minimum_plus", DType.F32, layouts, (n, n, n), 0.0, A, n, B, n, 0.0,
                              np.full(n * n, inf, np.float32), n, add_identity=inf)
    assert np.array_equal(got2, want)
    assert device_status() == 0


def test_known_answer_on_device(cuda_device):
    """test/regress/Srgemm_test.cu:64-116 (the GPU twin of the CPU known-answer test)."""
    ka = golden_io.known_answer()
    a, b, c, want = (np.array(ka[k]["data"], dtype=np.float32) for k in ("a", "b", "c", "correct"))
    got, _ = util.run_device("minimum_plus", DType.F32, (COL, COL, COL), (4, 4, 2), 0.0, a, 4, b, 2, 0.0, c, 4)
    assert np.all(np.abs(got - want) <= 4 * np.spacing(np.abs(want)))


def test_committed_reference_outputs_on_device(cuda_device):
    """The fixtures under tests/golden/ were produced by the reference's own host SRGEMM."""
    count = 0
    for case in golden_io.host_cases():
        ring, dt, layouts, (m, n, k) = case["ring"], case["dtype"], case["layouts"], case["mnk"]
        lda, ldb, ldc = (util.extents(layouts[0], m, k)[0], util.extents(layouts[1], k, n)[0],
                         util.extents(layouts[2], m, n)[0])
        alpha, beta = util.default_scalars(ring, dt)
        for tag, be in (("D_ann", beta), ("D_id", alpha)):
            if tag == "D_ann" and not util.annihilator_beta_is_defined(ring, dt):
                continue
            got, _ = util.run_device(ring, dt, layouts, (m, n, k), alpha, case["A"], lda, case["B"], ldb, be,
                                     case["C"], ldc)
            util.assert_equal(got, case[tag], layouts[2], m, n, ldc, what=f"{case['key']} {tag}")
            count += 1
    assert count >= 550
    assert device_status() == 0


@pytest.mark.parametrize("dt", [DType.S32, DType.U32])
@pytest.mark.parametrize("ring", ["minimum_plus", "maximum_plus", "minimum_maximum", "maximum_minimum"])
def test_integer_tropical_rings_take_the_tma_kernel(cuda_device, ring, dt):
    """32-bit integer tropical and bottleneck rings run on the TMA kernel when K is a multiple of its K step (there
    is no padding value for them); min-plus and max-plus use the fused add-min / add-max instructions."""
    rng = np.random.default_rng(7)
    kernels = set()
    for layouts in util.ALL_LAYOUTS:
        for mnk in ((260, 392, 96), (132, 516, 64), (128, 128, 32)):
            kernels.add(_check(ring, dt, layouts, mnk, rng, beta_is_identity=True))
    assert device_status() == 0
    assert kernels == {"tma"}, kernels


@pytest.mark.parametrize("ring", ["minimum_plus", "maximum_minimum", "plus_multiplies"])
def test_submatrix_views(cuda_device, ring):
    """Operands that are windows of larger matrices: ld > extent and offset base pointers, as in
    test/regress/Srgemm_test.cu:253-537 (top-left / bottom-right sub-blocks) and :539-605 (odd shapes)."""
    import torch
    rng = np.random.default_rng(5)
    dt = DType.F32
    big = 160
    for (m, n, k, off) in ((64, 64, 64, 0), (64, 64, 64, 96), (17, 27, 17, 0), (7, 6, 5, 3), (128, 128, 8, 32)):
        for layouts in (util.ALL_LAYOUTS[0], util.ALL_LAYOUTS[2], util.ALL_LAYOUTS[7]):
            A, _ = util.make_matrix(rng, dt, COL, big, big)
            B, _ = util.make_matrix(rng, dt, COL, big, big)
            C, _ = util.make_matrix(rng, dt, COL, big, big)
            start = off * big + off  # element (off, off) of a big x big matrix in either layout
            alpha, beta = util.default_scalars(ring, dt)
            beta = alpha
            want = util.run_oracle(ring, dt, layouts, (m, n, k), alpha, A[start:], big, B[start:], big, beta,
                                   C[start:], big, D_init=C[start:].copy())
            dA, dB, dC = (torch.from_numpy(x).cuda() for x in (A, B, C))
            op = Srgemm(*RINGS[ring], dt, *layouts)
            es = 4
            args = Arguments((m, n, k), (dA.data_ptr() + start * es, big), (dB.data_ptr() + start * es, big),
                             (dC.data_ptr() + start * es, big), (dC.data_ptr() + start * es, big), (alpha, beta))
            assert op(args) == Status.kSuccess  # C aliases D, like examples/00_minplus_srgemm/minplus_srgemm.cu:67-81
            torch.cuda.synchronize()
            got = dC.cpu().numpy()
            assert np.array_equal(got[start:], want), (ring, m, n, k, off, layouts)
            assert np.array_equal(got[:start], C[:start])
    assert device_status() == 0


@pytest.mark.parametrize("ring,dt", [("minimum_plus", DType.F32), ("plus_multiplies", DType.F32),
                                     ("maximum_plus", DType.F64), ("bit_xor_bit_and", DType.U32),
                                     ("minimum_plus", DType.S32)])
def test_split_k_equals_single_pass(cuda_device, ring, dt):
    """Parallel split-K equals the single-pass result exactly (examples/02_splitk_srgemm/splitk_srgemm.cu:270-287)
    and the oracle; also through the kSplitKSerial flag of Srgemm."""
    rng = np.random.default_rng(17)
    layouts = (ROW, COL, ROW)  # the layout of examples/02: A row-major, B column-major, C row-major
    for (m, n, k) in ((256, 256, 4096), (130, 70, 1000)):
        A, lda = util.make_matrix(rng, dt, layouts[0], m, k)
        B, ldb = util.make_matrix(rng, dt, layouts[1], k, n)
        C, ldc = util.make_matrix(rng, dt, layouts[2], m, n)
        alpha, _ = util.default_scalars(ring, dt)
        beta = alpha
        want = util.run_oracle(ring, dt, layouts, (m, n, k), alpha, A, lda, B, ldb, beta, C, ldc)
        single, _ = util.run_device(ring, dt, layouts, (m, n, k), alpha, A, lda, B, ldb, beta, C, ldc)
        assert np.array_equal(single, want)
        for slices in (2, 3, 16):
            got, kernel = util.run_device(ring, dt, layouts, (m, n, k), alpha, A, lda, B, ldb, beta, C, ldc,
                                          split_k_slices=slices, parallel_splitk=True)
            assert np.array_equal(got, single), (ring, slices, kernel)
            got, kernel = util.run_device(ring, dt, layouts, (m, n, k), alpha, A, lda, B, ldb, beta, C, ldc,
                                          split_k_slices=slices, split_k_serial=True)
            assert np.array_equal(got, single), (ring, slices, kernel)
    assert device_status() == 0


@pytest.mark.parametrize("ring,dt", [("minimum_plus", DType.F32), ("plus_multiplies", DType.F32),
                                     ("maximum_plus", DType.F64), ("bit_xor_bit_and", DType.U32)])
def test_balanced_launch_with_optional_workspace(cuda_device, ring, dt):
    """An unsplit launch given the optional workspace cuts the tiles of its last wave along K; the result must
    not change (integer-valued data, so plus-times is exact as well)."""
    import torch
    rng = np.random.default_rng(31)
    for layouts in (util.ALL_LAYOUTS[0], util.ALL_LAYOUTS[5]):
        for (m, n, k) in ((512, 512, 512), (640, 384, 2048), (1000, 264, 520)):
            A, lda = util.make_matrix(rng, dt, layouts[0], m, k)
            B, ldb = util.make_matrix(rng, dt, layouts[1], k, n)
            C, ldc = util.make_matrix(rng, dt, layouts[2], m, n)
            alpha, _ = util.default_scalars(ring, dt)
            want = util.run_oracle(ring, dt, layouts, (m, n, k), alpha, A, lda, B, ldb, alpha, C, ldc)

            def dev(x):
                return torch.from_numpy(x.view(np.int32) if x.dtype == np.uint32 else x).cuda()
            dA, dB, dC = dev(A), dev(B), dev(C)
            dD = torch.zeros_like(dC)
            op = Srgemm(*RINGS[ring], dt, *layouts)
            args = Arguments((m, n, k), (dA, lda), (dB, ldb), (dC, ldc), (dD, ldc), (alpha, alpha))
            assert op.get_workspace_size(args) == 0
            need = op.get_optional_workspace_size(args)
            assert need > 0, (m, n, k)
            ws = torch.empty(need, dtype=torch.uint8, device="cuda")
            for _ in range(2):   # twice: the tickets must be left clean
                assert op(args, ws) == Status.kSuccess
                torch.cuda.synchronize()
                assert op.last_kernel() == "tma_balanced"
                got = dD.cpu().numpy()
                got = got.view(np.uint32) if dt == DType.U32 else got
                assert np.array_equal(got, want), (ring, layouts, m, n, k)
            # a workspace that is too small is simply not used
            small = torch.empty(256, dtype=torch.uint8, device="cuda")
            assert op(args, small) == Status.kSuccess
            torch.cuda.synchronize()
            assert op.last_kernel() == "tma"
    assert device_status() == 0


@pytest.mark.parametrize("ring,dt", [("minimum_plus", DType.F32), ("maximum_plus", DType.F64),
                                     ("plus_multiplies", DType.F64), ("bit_xor_bit_and", DType.U32)])
def test_unaligned_operands_stay_on_the_tma_kernel_with_the_workspace(cuda_device, ring, dt):
    """The reference accepts any leading dimension and element-aligned pointers
    (include/cuasr/gemm/device/default_srgemm_configuration.h:88-89, test/device/testbed.h:313-319).  TMA cannot
    describe an operand whose address or leading dimension is not a multiple of 16 bytes: without a workspace such
    a product runs on the generic kernel, with the optional workspace the operand is first copied into aligned
    scratch and the fast kernel runs.  Either way the result is the host SRGEMM's."""
    import torch
    rng = np.random.default_rng(97)
    m, n, k = 300, 260, 190
    for layouts in util.ALL_LAYOUTS:
        # odd leading dimensions for A and B, and views that start one element into their buffers
        A, lda = util.make_matrix(rng, dt, layouts[0], m, k, ld=util.extents(layouts[0], m, k)[0] + 5)
        B, ldb = util.make_matrix(rng, dt, layouts[1], k, n, ld=util.extents(layouts[1], k, n)[0] + 3)
        C, ldc = util.make_matrix(rng, dt, layouts[2], m, n)
        A, B = np.concatenate([A[:1], A]), np.concatenate([B[:1], B])
        alpha, _ = util.default_scalars(ring, dt)
        want = util.run_oracle(ring, dt, layouts, (m, n, k), alpha, A[1:].copy(), lda, B[1:].copy(), ldb, alpha, C, ldc)

        def dev(x):
            return torch.from_numpy(x.view(np.int32) if x.dtype == np.uint32 else x).cuda()
        dA, dB, dC = dev(A), dev(B), dev(C)
        dD = torch.zeros_like(dC)
        es = dA.element_size()
        op = Srgemm(*RINGS[ring], dt, *layouts)
        args = Arguments((m, n, k), (dA.data_ptr() + es, lda), (dB.data_ptr() + es, ldb), (dC, ldc), (dD, ldc),
                         (alpha, alpha))
        assert op(args) == Status.kSuccess
        torch.cuda.synchronize()
        assert op.last_kernel() == "generic"
        got = dD.cpu().numpy()
        assert np.array_equal(got.view(np.uint32) if dt == DType.U32 else got, want), (ring, layouts, "generic")
        need = op.get_optional_workspace_size(args)
        assert need > 0
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        dD.zero_()
        assert op(args, ws) == Status.kSuccess
        torch.cuda.synchronize()
        assert op.last_kernel().startswith("tma"), op.last_kernel()
        got = dD.cpu().numpy()
        assert np.array_equal(got.view(np.uint32) if dt == DType.U32 else got, want), (ring, layouts, "repacked")
    assert device_status() == 0


@pytest.mark.parametrize("ring,dt", [("minimum_plus", DType.S32), ("maximum_plus", DType.U32),
                                     ("minimum_maximum", DType.S32), ("maximum_minimum", DType.U32)])
def test_integer_rings_with_ragged_k_use_padded_copies(cuda_device, ring, dt):
    """Integer min/max rings have no value TMA could fill a ragged last K step with.  With the optional workspace
    both operands are copied with K extended to whole steps - A by the additive identity, B by the multiplicative
    one - and the TMA kernel runs; without it the generic kernel does."""
    import torch
    rng = np.random.default_rng(5)
    for layouts in (util.ALL_LAYOUTS[0], util.ALL_LAYOUTS[3], util.ALL_LAYOUTS[6]):
        for (m, n, k) in ((256, 192, 100), (130, 300, 77)):
            A, lda = util.make_matrix(rng, dt, layouts[0], m, k)
            B, ldb = util.make_matrix(rng, dt, layouts[1], k, n)
            C, ldc = util.make_matrix(rng, dt, layouts[2], m, n)
            alpha, _ = util.default_scalars(ring, dt)
            want = util.run_oracle(ring, dt, layouts, (m, n, k), alpha, A, lda, B, ldb, alpha, C, ldc)

            def dev(x):
                return torch.from_numpy(x.view(np.int32) if x.dtype == np.uint32 else x).cuda()
            dA, dB, dC = dev(A), dev(B), dev(C)
            dD = torch.zeros_like(dC)
            op = Srgemm(*RINGS[ring], dt, *layouts)
            args = Arguments((m, n, k), (dA, lda), (dB, ldb), (dC, ldc), (dD, ldc), (alpha, alpha))
            assert op(args) == Status.kSuccess
            torch.cuda.synchronize()
            assert op.last_kernel() == "generic"
            need = op.get_optional_workspace_size(args)
            assert need > 0
            ws = torch.empty(need, dtype=torch.uint8, device="cuda")
            dD.zero_()
            assert op(args, ws) == Status.kSuccess
            torch.cuda.synchronize()
            assert op.last_kernel().startswith("tma"), (op.last_kernel(), ring, layouts, m, n, k)
            got = dD.cpu().numpy()
            assert np.array_equal(got.view(np.uint32) if dt == DType.U32 else got, want), (ring, layouts, m, n, k)
    assert device_status() == 0


@pytest.mark.parametrize("layouts", [(COL, COL, COL), (ROW, COL, ROW), (ROW, ROW, ROW), (COL, ROW, COL)])
def test_host_buffer_pipeline_equals_one_shot(cuda_device, layouts):
    """HostSrgemm (pinned host operands, chunked and overlapped copies) gives exactly the one-shot result."""
    import torch
    from cuasr_b200 import HostSrgemm
    rng = np.random.default_rng(77)
    dt, ring = DType.F32, "minimum_plus"
    m, n, k = 1024, 768, 640
    A, lda = util.make_matrix(rng, dt, layouts[0], m, k)
    B, ldb = util.make_matrix(rng, dt, layouts[1], k, n)
    C, ldc = util.make_matrix(rng, dt, layouts[2], m, n)
    want = util.run_oracle(ring, dt, layouts, (m, n, k), 0.0, A, lda, B, ldb, 0.0, C, ldc)
    op = Srgemm(*RINGS[ring], dt, *layouts)
    pipe = HostSrgemm(op, m, n, k, 0.0, 0.0, cuda_device, chunks=4)
    hA, hB, hC = (torch.from_numpy(x).pin_memory() for x in (A, B, C))
    hD = torch.empty(m * n, dtype=torch.float32).pin_memory()
    for _ in range(2):
        hD.zero_()
        pipe(hA, hB, hC, hD)
        torch.cuda.synchronize()
        assert np.array_equal(hD.numpy(), want)
    chunked = layouts in ((COL, COL, COL), (ROW, COL, ROW), (ROW, ROW, ROW))
    assert pipe.chunks == (4 if chunked else 1)
    # a shared operand whose lines do not run along k is packed once for all chunks, not once per launch
    assert (pipe.packed is not None) == (layouts in ((COL, COL, COL), (ROW, ROW, ROW)))
    # the first chunk runs as K pieces where the K range of the shared operand is a run of whole storage lines
    assert pipe.k_pieces == (4 if layouts in ((COL, COL, COL), (ROW, ROW, ROW)) else 1)
    assert HostSrgemm(Srgemm(*RINGS["plus_multiplies"], dt, *layouts), m, n, k, 1.0, 1.0, cuda_device).k_pieces == 1
    assert device_status() == 0


@pytest.mark.parametrize("dt", [DType.F32, DType.F64, DType.S32])
def test_pack_k_contiguous(cuda_device, dt):
    """cuasr_b200_pack_k_contiguous: both source forms, ragged sizes, padded leading dimensions on either side; the
    padding of the destination stays as it was; a product fed the packed copy as a row-major A has the same bits."""
    import torch
    from cuasr_b200 import pack_k_contiguous
    rng = np.random.default_rng(5)
    np_t = util.NUMPY_DTYPE[dt]
    tdt = {DType.F32: torch.float32, DType.F64: torch.float64, DType.S32: torch.int32}[dt]
    for rows, k, ld_src_pad, ld_dst_pad in [(130, 67, 3, 5), (1, 9, 0, 0), (513, 1, 2, 3), (256, 256, 0, 0)]:
        x = rng.integers(-50, 50, size=(rows, k)).astype(np_t)                 # x[r, kk]
        for src_k_contiguous in (False, True):
            ld_src = (k if src_k_contiguous else rows) + ld_src_pad
            lines = rows if src_k_contiguous else k
            src = np.full((lines, ld_src), 77, dtype=np_t)
            src[:, :ld_src - ld_src_pad] = x if src_k_contiguous else x.T
            ld_dst = k + ld_dst_pad
            d_src = torch.from_numpy(src).cuda()
            d_dst = torch.full((rows, ld_dst), -9, dtype=tdt, device="cuda")
            assert pack_k_contiguous(dt, d_src, ld_src, src_k_contiguous, rows, k, d_dst, ld_dst) == Status.kSuccess
            torch.cuda.synchronize()
            got = d_dst.cpu().numpy()
            assert np.array_equal(got[:, :k], x) and np.all(got[:, k:] == -9), (rows, k, src_k_contiguous)
    assert pack_k_contiguous(dt, 0, 8, False, 8, 8, 4096, 8) == Status.kErrorInvalidProblem
    assert pack_k_contiguous(dt, 4096, 8, False, 8, 8, 8192, 7) == Status.kErrorInvalidProblem       # ld_dst < k
    assert pack_k_contiguous(dt, 4096, 7, False, 8, 8, 8192, 8) == Status.kErrorInvalidProblem       # ld_src < rows
    assert pack_k_contiguous(dt, 4098, 8, False, 8, 8, 8192, 8) == Status.kErrorMisalignedOperand
    if dt == DType.F32:
        m, n, k = 384, 256, 320
        A, lda = util.make_matrix(rng, dt, COL, m, k)
        B, ldb = util.make_matrix(rng, dt, COL, k, n)
        C, ldc = util.make_matrix(rng, dt, COL, m, n)
        dA, dB, dC = (torch.from_numpy(t).cuda() for t in (A, B, C))
        dD, dD2 = torch.empty_like(dC), torch.empty_like(dC)
        packed = torch.empty(m * k, dtype=torch.float32, device="cuda")
        assert pack_k_contiguous(dt, dA, lda, False, m, k, packed, k) == Status.kSuccess
        plain = Srgemm(*RINGS["minimum_plus"], dt, COL, COL, COL)
        assert plain(Arguments((m, n, k), (dA, lda), (dB, ldb), (dC, ldc), (dD, ldc), (0.0, 0.0))) == Status.kSuccess
        rowa = Srgemm(*RINGS["minimum_plus"], dt, ROW, COL, COL)
        assert rowa(Arguments((m, n, k), (packed, k), (dB, ldb), (dC, ldc), (dD2, ldc), (0.0, 0.0))) == Status.kSuccess
        torch.cuda.synchronize()
        assert torch.equal(dD, dD2)
    assert device_status() == 0


def test_host_buffer_pipeline_with_a_negative_factor_under_min_times(cuda_device):
    """alpha (x) min(x, y) is not min(alpha (x) x, alpha (x) y) when (x) is multiplication and alpha is negative, so
    the first chunk must not be folded from K pieces that each apply alpha; the pipeline falls back to whole chunks
    and still equals the host SRGEMM."""
    import torch
    from cuasr_b200 import HostSrgemm
    rng = np.random.default_rng(78)
    dt, ring, layouts = DType.F32, "minimum_multiplies", (COL, COL, COL)
    m, n, k = 512, 512, 640
    A, lda = util.make_matrix(rng, dt, layouts[0], m, k)
    B, ldb = util.make_matrix(rng, dt, layouts[1], k, n)
    C, ldc = util.make_matrix(rng, dt, layouts[2], m, n)
    want = util.run_oracle(ring, dt, layouts, (m, n, k), -1.0, A, lda, B, ldb, 1.0, C, ldc)
    op = Srgemm(*RINGS[ring], dt, *layouts)
    pipe = HostSrgemm(op, m, n, k, -1.0, 1.0, cuda_device, chunks=4)
    assert pipe.k_pieces == 1
    assert HostSrgemm(op, m, n, k, 2.0, 1.0, cuda_device, chunks=4).k_pieces == 4
    hA, hB, hC = (torch.from_numpy(x).pin_memory() for x in (A, B, C))
    hD = torch.empty(m * n, dtype=torch.float32).pin_memory()
    pipe(hA, hB, hC, hD)
    torch.cuda.synchronize()
    assert np.array_equal(hD.numpy(), want)
    assert device_status() == 0


def test_overlapping_operand_views(cuda_device):
    """A leading dimension shorter than the extent is an overlapping (sliding-window) view of a read-only operand;
    the reference accepts it (its examples/02 passes one) and so does this library, with the host SRGEMM's answer."""
    rng = np.random.default_rng(5)
    dt, ring = DType.F32, "minimum_plus"
    m, n, k = 96, 80, 200
    for layouts, lda, ldb in (((ROW, COL, ROW), 16, 8), ((COL, ROW, COL), 4, 12), ((ROW, COL, COL), 200, 8)):
        A = rng.integers(-8, 9, size=m * k + k).astype(np.float32)          # large enough for every view below
        B = rng.integers(-8, 9, size=n * k + k).astype(np.float32)
        C, ldc = util.make_matrix(rng, dt, layouts[2], m, n)
        want = util.run_oracle(ring, dt, layouts, (m, n, k), 0.0, A, lda, B, ldb, 0.0, C, ldc)
        got, kernel = util.run_device(ring, dt, layouts, (m, n, k), 0.0, A, lda, B, ldb, 0.0, C, ldc)
        assert np.array_equal(got, want) and kernel == "generic", (layouts, kernel)
    assert device_status() == 0


def test_plus_times_tolerance(cuda_device):
    """Plus-times on non-integer data: the device fuses multiply-add and sums in a different order, so the
    check is |got - want| <= 8 K eps (|A| |B|)_ij."""
    rng = np.random.default_rng(23)
    for dt, eps in ((DType.F32, 2.0 ** -24), (DType.F64, 2.0 ** -53)):
        np_t = NUMPY_DTYPE[dt]
        m, n, k = 256, 192, 520
        A = (rng.random(m * k) * 2 - 1).astype(np_t)
        B = (rng.random(k * n) * 2 - 1).astype(np_t)
        C = np.zeros(m * n, np_t)
        layouts = (COL, COL, COL)
        want = util.run_oracle("plus_multiplies", dt, layouts, (m, n, k), 1.0, A, m, B, k, 0.0, C, m)
        got, _ = util.run_device("plus_multiplies", dt, layouts, (m, n, k), 1.0, A, m, B, k, 0.0, C, m)
        bound = 8 * k * eps * (np.abs(A.reshape(k, m).T.astype(np.float64)) @ np.abs(B.reshape(n, k).T.astype(np.float64)))
        err = np.abs(got.reshape(n, m).T.astype(np.float64) - want.reshape(n, m).T.astype(np.float64))
        assert np.all(err <= bound)


def test_status_codes(cuda_device):
    """Error behaviour of device::Srgemm (device/srgemm.h:196-266) and SrgemmSplitKParallel (:247-249)."""
    import torch
    x = torch.zeros(64 * 64, device="cuda")
    ok = Arguments((64, 64, 64), (x, 64), (x, 64), (x, 64), (x, 64), (0.0, 0.0))
    op = Srgemm(Op.MINIMUM, Op.PLUS, DType.F32, COL, COL, COL)
    assert op.can_implement(ok) == Status.kSuccess
    assert op.get_workspace_size(ok) == 0
    # split-K on an operator that was not built with kSplitKSerial
    bad = Arguments((64, 64, 64), (x, 64), (x, 64), (x, 64), (x, 64), (0.0, 0.0), split_k_slices=2)
    assert op.can_implement(bad) == Status.kErrorInvalidProblem
    assert op(bad) == Status.kErrorInvalidProblem
    # serial split-K wants a workspace
    ser = Srgemm(Op.MINIMUM, Op.PLUS, DType.F32, COL, COL, COL, split_k_serial=True)
    assert ser.get_workspace_size(bad) > 0
    assert ser(bad, None) == Status.kErrorWorkspaceNull
    par = SrgemmSplitKParallel(Op.MINIMUM, Op.PLUS, DType.F32, COL, COL, COL)
    assert par.get_workspace_size(bad) >= 4 * 64 * 64 * 2
    assert par(bad, None) == Status.kErrorWorkspaceNull
    # a required workspace that does not start on a 16-byte boundary is refused, an optional one is left unused
    ws = torch.zeros(par.get_workspace_size(bad) + 64, dtype=torch.uint8, device="cuda")
    assert par(bad, ws.data_ptr() + 4, workspace_bytes=ws.numel() - 4) == Status.kErrorMisalignedOperand
    big = Arguments((640, 640, 4096), (torch.zeros(640 * 4096, device="cuda"), 640), (torch.zeros(4096 * 640, device="cuda"), 4096),
                    (None, 640), (torch.zeros(640 * 640, device="cuda"), 640))
    ows = torch.zeros(op.get_optional_workspace_size(big) + 64, dtype=torch.uint8, device="cuda")
    assert op(big, ows.data_ptr() + 4, workspace_bytes=ows.numel() - 4) == Status.kSuccess and op.last_kernel() == "tma"
    assert op(big, ows) == Status.kSuccess and op.last_kernel() != "tma"
    # empty problem, short leading dimension, misaligned pointer, unsupported ring
    assert op.can_implement(Arguments((0, 64, 64), (x, 64), (x, 64), (x, 64), (x, 64))) == Status.kErrorInvalidProblem
    assert op.can_implement(Arguments((64, 64, 64), (x, 64), (x, 64), (x, 64), (x, 32))) == Status.kErrorInvalidProblem
    assert op.can_implement(Arguments((8, 8, 8), (x.data_ptr() + 2, 64), (x, 64), (x, 64), (x, 64))) \
        == Status.kErrorMisalignedOperand
    weird = Srgemm(Op.BIT_XOR, Op.BIT_AND, DType.F32, COL, COL, COL)
    assert weird.can_implement(ok) == Status.kErrorNotSupported
    # the default epilogue (alpha = mult identity, beta = mult annihilator) does not read C: C may be null
    noc = Arguments((64, 64, 64), (x, 64), (x, 64), (None, 64), (x, 64))
    assert op(noc) == Status.kSuccess
    torch.cuda.synchronize()
    # ... but a beta that needs the source does
    needs = Arguments((64, 64, 64), (x, 64), (x, 64), (None, 64), (x, 64), (0.0, 0.0))
    assert op(needs) == Status.kErrorInvalidProblem
    assert device_status() == 0


def test_extents_beyond_the_grid_y_limit(cuda_device):
    """The reference accepts any extent.  A 4.3-million-row product with N = K = 1 has more 64-row tiles than the
    65535 a CUDA grid allows along y or z; tiles are numbered along x here, so it runs (on the generic kernel: a
    leading dimension of 1 is nothing TMA can describe)."""
    import torch
    m, n, k = 4_300_000, 1, 1
    g = torch.Generator(device="cuda").manual_seed(3)
    A = torch.randint(-8, 9, (m,), generator=g, device="cuda").float()
    B = torch.tensor([2.0], device="cuda")
    C = torch.randint(-8, 9, (m,), generator=g, device="cuda").float()
    D = torch.zeros(m, device="cuda")
    op = Srgemm(*RINGS["minimum_plus"], DType.F32, ROW, ROW, ROW)
    assert op(Arguments((m, n, k), (A, 1), (B, 1), (C, 1), (D, 1), (0.0, 0.0))) == Status.kSuccess
    torch.cuda.synchronize()
    assert op.last_kernel() == "generic"
    assert torch.equal(D, torch.minimum(A + 2.0, C))
    assert device_status() == 0
