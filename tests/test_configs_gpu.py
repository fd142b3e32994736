"""Every benchmark configuration at its stated size, through the C ABI, against the host SRGEMM.

The whole product is out of reach for the host at these sizes (8192^3 is about two minutes on 16 threads), so
each case runs the full-size SRGEMM on the GPU and compares three groups of 32 storage lines of D (the first,
the middle and the last) bit for bit with the host SRGEMM fed the same operands: the operand that follows D's
lines is re-made on the host from the seed, the other one is needed in full and is read back from the device
(the generators are bit-identical on both sides, tests/test_workloads_cpu.py).  Split-K cases must in addition
equal the single-pass result of the same operands exactly, as the reference's own split-K example checks itself
(examples/02_splitk_srgemm/splitk_srgemm.cu:270-287).
"""
import numpy as np
import pytest

import oracle
from cuasr_b200 import (Arguments, DType, Layout, RINGS, Srgemm, SrgemmSplitKParallel, Status, device_status,
                        identity)
from cuasr_b200.semiring import NUMPY_DTYPE
from cuasr_b200.workloads import TORCH_DTYPE, WORKLOADS

pytestmark = pytest.mark.gpu
COL, ROW = Layout.COLUMN_MAJOR, Layout.ROW_MAJOR
GROUP = 32          # the host SRGEMM works in 32 x 32 blocks (host_srgemm.h:56-57)


def _ident(wl):
    return identity(RINGS[wl.ring][0], wl.dtype) if wl.add_identity is None else wl.add_identity


def _host(t, np_t):
    a = t.cpu().numpy()
    return a.view(np.uint32) if np_t == np.uint32 else a


def _line_groups(total):
    return sorted({0, (total // 2) // GROUP * GROUP, total - GROUP})


def _host_lines(wl, l0, hA, hB, hC_lines, scale_abs=False):
    """Host SRGEMM for storage lines [l0, l0 + GROUP) of D.  hA / hB: the full operand on the side that does not
    follow D's lines, None on the side that does (it is re-made from the seed here)."""
    np_t = NUMPY_DTYPE[wl.dtype]
    add_op, mul_op = RINGS[wl.ring]
    fn = oracle.ref_srgemm if oracle.have_ref() else oracle.srgemm
    if wl.layouts[2] == COL:            # lines are columns of D: columns l0.. of a column-major B
        assert wl.layouts[1] == COL
        sub = _host(wl.operand("B", "cpu", l0 * wl.k, GROUP * wl.k), np_t)
        A, B, mnk = hA, sub, (wl.m, GROUP, wl.k)
        lda, ldb, ldc = (wl.m if wl.layouts[0] == COL else wl.k), wl.k, wl.m
    else:                               # lines are rows of D: rows l0.. of a row-major A
        assert wl.layouts[0] == ROW
        sub = _host(wl.operand("A", "cpu", l0 * wl.k, GROUP * wl.k), np_t)
        A, B, mnk = sub, hB, (GROUP, wl.n, wl.k)
        lda, ldb, ldc = wl.k, (wl.k if wl.layouts[1] == COL else wl.n), wl.n
    if scale_abs:
        A, B, hC_lines = np.abs(A), np.abs(B), np.abs(hC_lines)
    D = np.empty_like(hC_lines)
    alpha, beta = (np.asarray(v).astype(np_t) for v in (wl.alpha, wl.beta))
    fn(add_op, mul_op, wl.dtype, wl.layouts, mnk, alpha, A, lda, B, ldb, beta, hC_lines, ldc, D, ldc, _ident(wl), 0)
    return D


def _run_full(wl, with_optional_workspace=True, operands=None, c_fill=None, split_k_slices=None):
    """The full-size SRGEMM of `wl` on the GPU through the C ABI; returns (A, B, C, D, kernel name)."""
    import torch
    dev = torch.device("cuda", 0)
    tdt = TORCH_DTYPE[wl.dtype]
    ident = _ident(wl)
    A, B = operands if operands is not None else (wl.operand("A", dev), wl.operand("B", dev))
    fill = ident if c_fill is None else c_fill
    C = torch.full((wl.m * wl.n,), float(fill) if tdt.is_floating_point else int(fill), dtype=tdt, device=dev) \
        if not hasattr(fill, "numel") else fill
    D = torch.zeros(wl.m * wl.n, dtype=tdt, device=dev)
    slices = wl.split_k_slices if split_k_slices is None else split_k_slices
    add_op, mul_op = RINGS[wl.ring]
    cls = SrgemmSplitKParallel if slices > 1 else Srgemm
    op = cls(add_op, mul_op, wl.dtype, *wl.layouts, add_identity=ident)
    lda = wl.m if wl.layouts[0] == COL else wl.k
    ldb = wl.k if wl.layouts[1] == COL else wl.n
    ldc = wl.m if wl.layouts[2] == COL else wl.n
    args = Arguments((wl.m, wl.n, wl.k), (A, lda), (B, ldb), (C, ldc), (D, ldc), (wl.alpha, wl.beta), slices)
    need = op.get_workspace_size(args)
    if not need and with_optional_workspace:
        need = op.get_optional_workspace_size(args)
    ws = torch.empty(need, dtype=torch.uint8, device=dev) if need else None
    assert op(args, ws) == Status.kSuccess
    assert device_status() == 0
    return A, B, C, D, op.last_kernel()


def _check_lines(wl, A, B, C, D):
    np_t = NUMPY_DTYPE[wl.dtype]
    col_c = wl.layouts[2] == COL
    total, contig = (wl.n, wl.m) if col_c else (wl.m, wl.n)
    hA = _host(A, np_t) if col_c else None
    hB = None if col_c else _host(B, np_t)
    for l0 in _line_groups(total):
        sl = slice(l0 * contig, (l0 + GROUP) * contig)
        c_lines = _host(C[sl], np_t)
        want = _host_lines(wl, l0, hA, hB, c_lines)
        got = _host(D[sl], np_t)
        if wl.ring == "plus_multiplies" and wl.dtype in (DType.F32, DType.F64):
            # the tensor-core path accumulates in another order than the host loop: |delta| <= 8 K eps (|A| |B|)_ij
            bound = 8 * wl.k * np.finfo(np_t).eps * _host_lines(wl, l0, hA, hB, c_lines, scale_abs=True)
            err = np.abs(got - want)
            assert (err <= bound).all(), f"{wl.name}: lines {l0}..: max error {err.max()} beyond the bound"
        else:
            bad = got != want
            assert not bad.any(), (f"{wl.name}: lines {l0}..{l0 + GROUP}: {int(bad.sum())} of {bad.size} elements "
                                   f"differ, first at {int(np.argmax(bad))}")


@pytest.mark.parametrize("name", ["minplus_f32_512", "minplus_f32_8192", "minplus_f64_8192", "maxplus_f64_8192",
                                  "maxmin_f32_4096", "plustimes_f64_4096", "xorand_u32_4096"])
def test_config_at_full_size(cuda_device, name):
    wl = WORKLOADS[name]
    A, B, C, D, kernel = _run_full(wl)
    assert "tma" in kernel, kernel
    _check_lines(wl, A, B, C, D)


def test_north_star_without_workspace(cuda_device):
    """The same 8192^3 product without the optional workspace (no re-packed operands, no balanced last wave)."""
    wl = WORKLOADS["minplus_f32_8192"]
    A, B, C, D, kernel = _run_full(wl, with_optional_workspace=False)
    assert "tma" in kernel, kernel
    _check_lines(wl, A, B, C, D)


def test_splitk_config_16_32_64_slices(cuda_device):
    """Config 3: M = N = 256, K = 1 048 576 cut into 16 / 32 / 64 slices; every slicing must equal the single pass
    exactly (min is order-independent) and the host SRGEMM on sampled rows."""
    import torch
    wl = WORKLOADS["splitk_minplus_f32_s16"]
    A, B, C, single, kernel = _run_full(wl, split_k_slices=1)
    assert "tma" in kernel, kernel
    _check_lines(wl, A, B, C, single)
    for slices in (16, 32, 64):
        _, _, _, D, kernel = _run_full(wl, operands=(A, B), split_k_slices=slices)
        assert "tma" in kernel, kernel
        assert torch.equal(D, single), f"{slices} slices differ from the single pass"


def test_apsp_16384_one_squaring(cuda_device):
    """Config 4, one squaring at full size: D' = min(D, D (x) D) on the n = 16384 graph, sampled columns against the
    host SRGEMM fed the same matrix."""
    import torch
    free, _ = torch.cuda.mem_get_info()
    if free < 8e9:
        pytest.skip("needs 8 GB of free device memory")
    wl = WORKLOADS["apsp_16384"]
    G = wl.operand("A", torch.device("cuda", 0))
    A, B, C, D, kernel = _run_full(wl, operands=(G, G), c_fill=G)
    assert "tma" in kernel, kernel
    _check_lines(wl, A, B, C, D)
    # the squaring can only shorten paths, and the diagonal stays 0
    assert bool((D <= G).all())
    assert bool((D.view(wl.n, wl.n).diagonal() == 0).all())
