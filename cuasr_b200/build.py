"""Builds cuasr_b200/csrc/libcuasr_b200.so for sm_100a with nvcc, one translation unit per process.

Run as `python -m cuasr_b200.build` (or through `__graft_entry__.build()`).  The library is kept in-tree,
next to its sources; objects go to cuasr_b200/csrc/build/.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")
OUT = os.path.join(CSRC, "libcuasr_b200.so")
NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_mtime():
    inc = os.path.join(os.path.dirname(CSRC), "..", "include")
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    paths += [os.path.join(inc, f) for f in os.listdir(inc) if f.endswith(".h")]
    return max(os.path.getmtime(p) for p in paths)


def _compile(src: str, verbose: bool) -> str:
    obj_dir = os.path.join(CSRC, "build")
    os.makedirs(obj_dir, exist_ok=True)
    obj = os.path.join(obj_dir, src[:-3] + ".o")
    src_path = os.path.join(CSRC, src)
    if os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(src_path), _headers_mtime()):
        return obj
    cmd = ["nvcc", *NVCC_FLAGS, "-c", src_path, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def build(verbose: bool = False, jobs: int | None = None) -> str:
    srcs = _sources()
    jobs = jobs or min(len(srcs), os.cpu_count() or 4)
    with concurrent.futures.ThreadPoolExecutor(max_workers=jobs) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), srcs))
    if not os.path.exists(OUT) or any(os.path.getmtime(o) > os.path.getmtime(OUT) for o in objs):
        # cudart is linked statically and the driver API is reached through the runtime, so the library
        # loads on a machine without a GPU driver
        cmd = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
               "-cudart", "static", "-o", OUT, *objs, "-ldl", "-lpthread"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return OUT


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
