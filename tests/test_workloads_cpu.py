"""The seeded generators behind the benchmark workloads: deterministic, and any sub-range of an operand equals the
same range of the whole (ranks and host-side spot checks regenerate only the part they need)."""
import numpy as np
import pytest
import torch

from cuasr_b200 import DType
from cuasr_b200.workloads import TORCH_DTYPE, WORKLOADS, Workload, COL


def _small(wl, n):
    return Workload(**{**wl.__dict__, "name": wl.name + "_small", "m": n, "n": n, "k": n})


@pytest.mark.parametrize("name", ["minplus_f32_8192", "minplus_f64_8192", "maxplus_f64_8192", "apsp_16384",
                                  "maxmin_f32_4096", "plustimes_f64_4096", "xorand_u32_4096", "minplus_s32_4096"])
def test_sub_ranges_equal_the_whole(name):
    wl = _small(WORKLOADS[name], 96)
    for which in ("A", "B"):
        whole = wl.operand(which)
        assert whole.dtype == TORCH_DTYPE[wl.dtype] and whole.numel() == 96 * 96
        assert torch.equal(whole, wl.operand(which))                                  # deterministic
        for start, count in ((0, 96), (96 * 7, 96 * 5), (96 * 95, 96)):
            assert torch.equal(whole[start:start + count], wl.operand(which, start=start, count=count))
    if wl.fill != "apsp":
        assert not torch.equal(wl.operand("A"), wl.operand("B"))                      # different seeds


def test_value_ranges():
    a = _small(WORKLOADS["minplus_f32_8192"], 128).operand("A")
    assert float(a.min()) >= 0.0 and float(a.max()) < 100.0 and a.unique().numel() > 1000
    i = _small(WORKLOADS["minplus_s32_4096"], 128).operand("A")
    assert i.dtype == torch.int32 and int(i.min()) >= 0 and int(i.max()) < 1000
    g = _small(WORKLOADS["apsp_16384"], 256).operand("A").view(256, 256)
    assert torch.all(torch.diagonal(g) == 0)
    present = torch.isfinite(g) & ~torch.eye(256, dtype=torch.bool)
    assert 0.002 < present.float().mean() < 0.03                                     # p = 0.01
    w = g[present]
    assert torch.all(w == w.round()) and float(w.min()) >= 1 and float(w.max()) <= 100
    d = _small(WORKLOADS["minplus_f64_8192"], 256).operand("A").view(256, 256)
    assert 0.05 < (torch.isfinite(d) & ~torch.eye(256, dtype=torch.bool)).float().mean() < 0.15   # 10 % present


def test_operation_count_is_two_m_n_k():
    assert WORKLOADS["minplus_f32_8192"].ops == 2.0 * 8192 ** 3
    assert WORKLOADS["splitk_minplus_f32_s16"].ops == 2.0 * 256 * 256 * 1048576
