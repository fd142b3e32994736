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


PROBE = r"""
#include <cstdio>
#include "cuasr/functional.h"
// functors the headers know nothing about, in the shape of examples/01_userdefined_semiring/userdefined_semiring.cu:56-99
template <typename T> struct my_xor  { static constexpr T Identity = 0; T operator()(T l, T const& r) const { return l ^ r; } };
template <typename T> struct my_band { static constexpr T Identity = ~T(0); T operator()(T l, T const& r) const { return l & r; } };
template <typename T> struct my_bor  { static constexpr T Identity = 0; T operator()(T l, T const& r) const { return l | r; } };
template <typename T> struct my_min  { T operator()(T l, T const& r) const { return r < l ? r : l; } };
template <typename T> struct my_max  { T operator()(T l, T const& r) const { return l < r ? r : l; } };
template <typename T> struct my_add  { T operator()(T l, T const& r) const { return l + r; } };
template <typename T> struct my_mul  { T operator()(T l, T const& r) const { return l * r; } };
template <typename T> struct my_land { T operator()(T l, T const& r) const { return T(l && r); } };
template <typename T> struct my_lor  { T operator()(T l, T const& r) const { return T(l || r); } };
template <typename T> struct my_sub  { T operator()(T l, T const& r) const { return l - r; } };
// agree with plus / multiplies on small values only: must NOT be taken for them
template <typename T> struct my_satadd { T operator()(T l, T const& r) const { T s = l + r; return s < T(100) ? s : T(100); } };
template <typename T> struct my_modmul { T operator()(T l, T const& r) const { return T((long long)(l * r) % 1000003); } };
struct tagged { static constexpr int kOpCode = CUASR_OP_MAXIMUM; float operator()(float l, float const& r) const { return l - r; } };
int main() {
  int bad = 0;
#define EXPECT(F, T, CODE) if (cuasr::OpCodeOf<F<T>, T>::get() != (CODE)) { std::printf("%s<%s>\n", #F, #T); ++bad; }
  EXPECT(my_xor, int, CUASR_OP_BIT_XOR)   EXPECT(my_band, unsigned, CUASR_OP_BIT_AND)  EXPECT(my_bor, int, CUASR_OP_BIT_OR)
  EXPECT(my_min, float, CUASR_OP_MINIMUM) EXPECT(my_max, double, CUASR_OP_MAXIMUM)     EXPECT(my_add, float, CUASR_OP_PLUS)
  EXPECT(my_mul, double, CUASR_OP_MULTIPLIES) EXPECT(my_land, int, CUASR_OP_BINARY_AND) EXPECT(my_lor, float, CUASR_OP_BINARY_OR)
  EXPECT(my_min, int, CUASR_OP_MINIMUM)   EXPECT(my_sub, float, -1)                    EXPECT(my_sub, int, -1)
  EXPECT(my_satadd, float, -1)            EXPECT(my_satadd, int, -1)                   EXPECT(my_modmul, int, -1)
  EXPECT(cuasr::minimum, float, CUASR_OP_MINIMUM)                                      // declared functors are not probed
  if (cuasr::OpCodeOf<tagged, float>::get() != CUASR_OP_MAXIMUM) ++bad;               // kOpCode wins over behaviour
  return bad;
}
"""


def test_undeclared_functors_are_recognised_by_what_they_compute(tmp_path):
    src, exe = tmp_path / "probe.cpp", tmp_path / "probe"
    src.write_text(PROBE)
    subprocess.run(["g++", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-I", "/usr/local/cuda/include",
                    str(src), "-o", str(exe)], check=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout


@pytest.mark.gpu
def test_user_defined_functors_run_as_compiled_kernels(cuda_device):
    """Functors without an operator code (a saturating sum, a non-commutative product) through the drop-in templates:
    the headers compile them into a kernel in the caller's translation unit, as the reference does with every functor;
    the program checks the reference's ragged grid in all eight layouts against host loops over the same functors."""
    binary = os.path.join(ROOT, "tests", "cpp", "user_functors")
    assert os.path.exists(binary), "build it with __graft_entry__.build()"
    res = subprocess.run([binary], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "ALL OK" in res.stdout


@pytest.mark.gpu
def test_rehosted_reference_examples(cuda_device):
    assert os.path.exists(BINARY), "build it with __graft_entry__.build()"
    res = subprocess.run([BINARY], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "ALL OK" in res.stdout


@pytest.mark.gpu
def test_multi_gpu_solve_from_a_plain_cpp_host(cuda_device):
    """cuasr_b200_apsp_multi called from a C++ program with cudaMalloc'ed buffers (no Python, no NCCL): repeated
    squaring and blocked Floyd-Warshall on 1, 2 and 4 GPUs as far as the box has them, against a host
    Floyd-Warshall."""
    binary = os.path.join(ROOT, "tests", "cpp", "apsp_multi_host")
    assert os.path.exists(binary), "build it with __graft_entry__.build()"
    res = subprocess.run([binary], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "ALL OK" in res.stdout
