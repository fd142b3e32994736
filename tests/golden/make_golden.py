"""Generates the golden fixtures of tests/golden/ from the REFERENCE checkout.  Run in a container that has
a checkout of the reference (path as first argument, or $CUASR_REFERENCE) and oracle/_ref built (`make -C oracle ref`):

    python tests/golden/make_golden.py [/path/to/reference]

Writes
  regress_known_answer.json   the hand-written 4x4x2 min-plus case of test/regress/Srgemm_test.cu:15-62,
                              parsed from the reference's test source
  host_srgemm_outputs.npz     outputs of the reference's own host_srgemm.h (oracle/_ref) for every ring,
                              element type and layout combination on seeded small-integer inputs, with the
                              inputs, so that the fixtures do not depend on any random generator
  fwgemm_outputs.npz          outputs (distances and parents) of the reference's legacy path-tracking routine
                              test/regress/include/fwgpu/cpu_srgemm.hpp (oracle/_ref, `make -C oracle refpath`) on
                              square column-major inputs with many ties, with the inputs
"""
import json
import os
import re
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
import util  # noqa: E402
from cuasr_b200 import DType, Layout  # noqa: E402


def known_answer(reference):
    src = open(os.path.join(reference, "test", "regress", "Srgemm_test.cu")).read()
    body = src[src.index("CpuNaiveCorrect"):src.index("cpu_srgemm_naive(")]
    mats = re.findall(r"Matrix<float>\(\s*(\d+),\s*(\d+),\s*\{(.*?)\}\)", body, flags=re.S)
    names = ["a", "b", "c", "correct"]
    out = {"source": "test/regress/Srgemm_test.cu:15-62", "layout": "column-major", "semiring": "min-plus",
           "epilogue": "C = min(C, A (x) B)"}
    for name, (rows, cols, vals) in zip(names, mats):
        nums = [float(v) for v in re.findall(r"[-+]?\d*\.\d+|\d+", re.sub(r"//.*", "", vals))]
        assert len(nums) == int(rows) * int(cols), (name, len(nums))
        out[name] = {"rows": int(rows), "cols": int(cols), "data": nums}
    return out


def host_outputs():
    rng = np.random.default_rng(2080)
    store = {}
    shapes = [(13, 11, 9)]
    for ring, dt in util.ring_dtype_cases():
        for li, layouts in enumerate(util.ALL_LAYOUTS):
            for (m, n, k) in shapes + ([(65, 33, 47)] if li == 0 else []):
                A, lda = util.make_matrix(rng, dt, layouts[0], m, k)
                B, ldb = util.make_matrix(rng, dt, layouts[1], k, n)
                C, ldc = util.make_matrix(rng, dt, layouts[2], m, n)
                alpha, beta = util.default_scalars(ring, dt)
                key = f"{ring}|{int(dt)}|{''.join(str(int(x)) for x in layouts)}|{m}x{n}x{k}"
                # inputs are integers in [-8, 8]: stored as int8, cast back to the element type on load
                store[key + "|A"], store[key + "|B"], store[key + "|C"] = (x.astype(np.int8) for x in (A, B, C))
                # beta = mult annihilator (TestAllGemm) and beta = mult identity (the source matrix takes part)
                for tag, be in (("ann", beta), ("id", alpha)):
                    D = util.run_oracle(ring, dt, layouts, (m, n, k), alpha, A, lda, B, ldb, be, C, ldc, use_ref=True)
                    store[key + "|D" + tag] = D
    return store


def fwgemm_outputs():
    rng = np.random.default_rng(1905)
    store = {}
    for np_t, tag in ((np.float32, "f32"), (np.float64, "f64")):
        for n in (5, 17, 64):
            # small integers: many equal candidates, so "which k wins a tie" is exercised, and every sum is exact
            A = rng.integers(0, 6, size=n * n).astype(np_t)
            B = rng.integers(0, 6, size=n * n).astype(np_t)
            dist = rng.integers(0, 9, size=n * n).astype(np_t)      # zeros and ones often stay unimproved
            parent = rng.integers(-5, 0, size=n * n).astype(np.int32)
            key = f"{tag}|{n}"
            store[key + "|A"], store[key + "|B"] = A.astype(np.int8), B.astype(np.int8)
            store[key + "|dist_in"], store[key + "|parent_in"] = dist.astype(np.int8), parent.astype(np.int8)
            d, p = oracle.ref_fwgemm(A, B, dist.copy(), parent.copy(), n)
            store[key + "|dist_out"], store[key + "|parent_out"] = d, p
    return store


def main():
    reference = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("CUASR_REFERENCE")
    assert reference, "usage: make_golden.py <reference checkout>   (or set CUASR_REFERENCE)"
    assert oracle.have_ref(), "build oracle/_ref first: make -C oracle ref"
    with open(os.path.join(HERE, "regress_known_answer.json"), "w") as f:
        json.dump(known_answer(reference), f, indent=1)
    store = host_outputs()
    np.savez_compressed(os.path.join(HERE, "host_srgemm_outputs.npz"), **store)
    print(len(store) // 5, "input sets written")
    assert oracle.have_ref_path(), "build the path checker first: make -C oracle refpath"
    np.savez_compressed(os.path.join(HERE, "fwgemm_outputs.npz"), **fwgemm_outputs())


if __name__ == "__main__":
    main()
