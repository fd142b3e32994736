"""The drop-in C++ headers (include/cuasr/...): they compile without CUTLASS, and the reference's three example
wrappers re-hosted on them give the right answers on the GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BINARY = os.path.join(ROOT, "tests", "cpp", "facade_examples")

SNIPPET = r"""
#include "cuasr/functional.h"
#include "cuasr/gemm/device/srgemm.h"
#include "cuasr/gemm/device/srgemm_splitk_parallel.h"
using Col = cutlass::layout::ColumnMajor;
using G = cuasr::gemm::device::Srgemm<cuasr::minimum<float>, cuasr::plus<float>, float, Col, float, Col, float, Col>;
using S = cuasr::gemm::device::SrgemmSplitKParallel<cuasr::maximum<double>, cuasr::plus<double>, double, Col, double, Col, double, Col>;
static_assert(G::kSplitKSerial == false && G::ThreadblockShape::kM == 128, "presets");
static_assert(cuasr::plus<float>::Identity == 0.0f && cuasr::multiplies<int>::Annihilator == 0, "constants");
static_assert(cuasr::minimum<float>::Identity > 3e38f && cuasr::maximum<float>::Identity > 0.0f, "reference 'infinities'");
int main() {
  G::Arguments a({4, 4, 2}, {nullptr, 4}, {nullptr, 2}, {nullptr, 4}, {nullptr, 4});
  G::EpilogueOutputOp op(a.epilogue);
  return (op.is_source_needed() ? 1 : 0) + (sizeof(S) > 0 ? 0 : 1);   // default beta does not need C
}
"""


def test_headers_compile_without_cutlass(tmp_path):
    src = tmp_path / "t.cpp"
    src.write_text(SNIPPET)
    subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-I", os.path.join(ROOT, "include"),
                    "-I", "/usr/local/cuda/include", str(src)], check=True)


@pytest.mark.gpu
def test_rehosted_reference_examples(cuda_device):
    assert os.path.exists(BINARY), "build it with __graft_entry__.build()"
    res = subprocess.run([BINARY], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "ALL OK" in res.stdout
