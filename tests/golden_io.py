"""Reads the committed golden fixtures (written by tests/golden/make_golden.py)."""
import json
import os

import numpy as np

from cuasr_b200 import DType, Layout
from cuasr_b200.semiring import NUMPY_DTYPE

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def known_answer():
    with open(os.path.join(GOLDEN, "regress_known_answer.json")) as f:
        return json.load(f)


def host_cases():
    """Yields dicts: ring, dtype, layouts, mnk, A, B, C (element type restored), D_ann, D_id."""
    z = np.load(os.path.join(GOLDEN, "host_srgemm_outputs.npz"))
    keys = sorted(k[:-2] for k in z.files if k.endswith("|A"))
    for key in keys:
        ring, dt, lay, shape = key.split("|")
        dt = DType(int(dt))
        np_t = NUMPY_DTYPE[dt]
        yield {
            "key": key, "ring": ring, "dtype": dt, "layouts": tuple(Layout(int(c)) for c in lay),
            "mnk": tuple(int(x) for x in shape.split("x")),
            "A": z[key + "|A"].astype(np_t), "B": z[key + "|B"].astype(np_t), "C": z[key + "|C"].astype(np_t),
            "D_ann": z[key + "|Dann"], "D_id": z[key + "|Did"],
        }


def fwgemm_cases():
    """Yields dicts: dtype (numpy), n, A, B, dist_in, parent_in, dist_out, parent_out of the reference's legacy
    path-tracking routine (square, column-major)."""
    z = np.load(os.path.join(GOLDEN, "fwgemm_outputs.npz"))
    for key in sorted(k[:-2] for k in z.files if k.endswith("|A")):
        tag, n = key.split("|")
        np_t = np.float32 if tag == "f32" else np.float64
        yield {"key": key, "dtype": np_t, "n": int(n), "A": z[key + "|A"].astype(np_t), "B": z[key + "|B"].astype(np_t),
               "dist_in": z[key + "|dist_in"].astype(np_t), "parent_in": z[key + "|parent_in"].astype(np.int32),
               "dist_out": z[key + "|dist_out"], "parent_out": z[key + "|parent_out"]}
