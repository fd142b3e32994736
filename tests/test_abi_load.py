"""The C-ABI library loads without a GPU and exports every function include/cuasr_b200.h declares."""
import ctypes
import os
import re

from cuasr_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = []
    for header in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if not header.endswith(".h"):
            continue
        text = open(os.path.join(ROOT, "include", header)).read()
        names += re.findall(r"CUASR_B200_API\s+[\w\s\*]+?\b(cuasr_b200_\w+)\s*\(", text)
    return names


def test_header_declares_the_entry_points():
    names = declared_functions()
    for must in ("cuasr_b200_srgemm", "cuasr_b200_srgemm_can_implement", "cuasr_b200_srgemm_workspace_size",
                 "cuasr_b200_srgemm_splitk", "cuasr_b200_srgemm_splitk_workspace_size"):
        assert must in names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"


def test_python_binding_covers_every_declared_symbol():
    assert set(declared_functions()) == set(_lib.PROTOTYPES)


def test_no_compute_calls_needed_for_metadata():
    lib = _lib.load()
    assert b"sm_100a" in lib.cuasr_b200_version()
    assert lib.cuasr_b200_status_string(0) == b"success"
    assert lib.cuasr_b200_status_string(6) == b"workspace null"
    assert lib.cuasr_b200_launch_count() == 0


def test_struct_layout_matches_the_header():
    # int32 x 8 ; int32 x 4 + 4 x (ptr, int64) + 4 x 8-byte scalars + ptr + size_t + ptr
    assert ctypes.sizeof(_lib.Desc) == 32
    assert ctypes.sizeof(_lib.Args) == 16 + 4 * 16 + 4 * 8 + 24


def test_headers_are_plain_c(tmp_path):
    """The boundary is a C ABI: both public headers must compile as C11 on their own."""
    import subprocess
    for header in ("cuasr_b200.h", "cuasr_b200_apsp.h", "cuasr_b200_types.h"):
        src = tmp_path / (header + ".c")
        src.write_text(f'#include "{header}"\nint main(void) {{ return 0; }}\n')
        subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), str(src)],
                       check=True)
