"""One of the reference's generated benchmark files (bench/device/simt_minimum_plus_ssrgemm_nn_n_sm50.cu), compiled
UNMODIFIED against this library's drop-in headers (google-benchmark replaced by oracle/shim/benchmark/benchmark.h),
run at its small sizes: the harness, its argument set-up and the launch all go through the drop-in operator.
Skipped where oracle/_ref/bench_* was not built."""
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BINARY = os.path.join(ROOT, "oracle", "_ref", "bench_minimum_plus_ssrgemm_nn_n")


@pytest.mark.gpu
@pytest.mark.skipif(not os.path.exists(BINARY), reason="oracle/_ref/bench_minimum_plus_ssrgemm_nn_n was not built")
def test_reference_benchmark_file_runs_on_the_drop_in_headers(cuda_device):
    res = subprocess.run([BINARY, "2", "1024"], capture_output=True, text=True, timeout=600)   # 2 iterations, N <= 1024
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-1500:]
    rates = [float(x) for x in re.findall(r"([0-9.e+]+) Flop/s", res.stdout)]
    assert len(rates) == 6 and all(r > 0 for r in rates), res.stdout       # 2 tile presets x N in {256, 512, 1024}
