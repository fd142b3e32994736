"""The reference's three example programs (examples/00, 01, 02), compiled UNMODIFIED against this library's
drop-in headers into oracle/_ref/ where the reference checkout is available, run to their own verdicts:
  00  min-plus 4096^3 through cuasr_minplus_srsgemm_nt_n (C aliases D); prints its rate
  01  GF(2) xor-and with the example's own hand-written binary_xor functor (recognised by probing what it computes),
      checked by the example against the reference's host SRGEMM
  02  parallel split-K against the single-pass SRGEMM (the example hands both a leading dimension shorter than the
      row of its row-major operand; read-only overlapping views are accepted)
Skipped where the binaries were not built."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")
CASES = [("example_minplus_srgemm", "Min-Plus SRGEMM FLOP/s"),
         ("example_userdefined_semiring", "PASSED!"),
         ("example_splitk_srgemm", "Split-K matches regular SRGEMM")]


@pytest.mark.gpu
@pytest.mark.parametrize("binary,verdict", CASES)
def test_reference_example_runs_unmodified(cuda_device, binary, verdict):
    path = os.path.join(REF, binary)
    if not os.path.exists(path):
        pytest.skip(f"oracle/_ref/{binary} was not built")
    res = subprocess.run([path], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-1500:]
    assert verdict in res.stdout and "Error code" not in res.stdout
