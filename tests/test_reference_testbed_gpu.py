"""The reference's own device test bed (test/device/testbed.h: TestAllGemm), compiled unmodified against this
library's drop-in headers, for every pre-tuned ring x {float, double} x the eight layout combinations.  The binary is
built into oracle/_ref where the reference checkout is available; skipped where it was not built."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BINARY = os.path.join(ROOT, "oracle", "_ref", "ref_testbed")


@pytest.mark.gpu
@pytest.mark.skipif(not os.path.exists(BINARY), reason="oracle/_ref/ref_testbed was not built")
def test_reference_test_bed_passes_on_the_drop_in_headers(cuda_device):
    res = subprocess.run([BINARY], capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "128 operator instantiations, 0 failed, 0 EXPECT_TRUE failures" in res.stdout
