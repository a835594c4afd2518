"""The C-ABI library loads and exports every function include/rof_b200.h declares (no compute)."""
import ctypes
import os
import re

from artifact_b200 import _native, build
from conftest import ROOT


def declared_functions():
    text = open(os.path.join(ROOT, "include", "rof_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rof_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    names = declared_functions()
    assert "rof_aggregate" in names and len(names) >= 12
    lib = ctypes.CDLL(build.cuda_lib_path())
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/rof_b200.h but not exported"
    bound = {n for n, _, _ in _native.CUDA_ABI}
    assert bound == set(names), (sorted(bound ^ set(names)))


def test_version_and_error_string():
    lib = _native.cuda()
    assert lib.rof_compiled_arch() == 100
    assert isinstance(lib.rof_last_error(), bytes)
    assert lib.rof_plan_workspace_bytes(None, 8) == -1


def test_host_library_loads():
    lib = _native.host()
    assert hasattr(lib, "rofh_chung_lu_rows") and hasattr(lib, "rofh_symmetrize")


def test_header_is_plain_c(tmp_path):
    """the boundary is a C ABI: the header must compile as C99 on its own, and a C program that
    names every function must link against the library"""
    import subprocess
    hdr = os.path.join(ROOT, "include", "rof_b200.h")
    subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", "-x", "c", hdr])
    src = tmp_path / "use_all.c"
    names = declared_functions()
    src.write_text('#include "rof_b200.h"\n#include <stdio.h>\nint main(void) {\n  const void* f[] = {' +
                   ", ".join(f"(const void*){n}" for n in names) +
                   '};\n  printf("%d %d\\n", (int)(sizeof f / sizeof f[0]), rof_compiled_arch());\n  return rof_version() > 0 ? 0 : 1;\n}\n')
    exe = tmp_path / "use_all"
    libdir = os.path.dirname(build.cuda_lib_path())
    subprocess.check_call(["gcc", "-std=c99", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                           "-L", libdir, "-lrof_b200", f"-Wl,-rpath,{libdir}", "-Wl,-rpath,/usr/local/cuda/lib64"])
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.split() == [str(len(names)), "100"]


def test_argument_checks_of_the_auxiliary_entry_points():
    """bad arguments come back as status codes before anything touches a device"""
    import ctypes
    lib = _native.cuda()
    buf = (ctypes.c_float * 64)()
    p = ctypes.cast(buf, ctypes.c_void_p)
    assert lib.rof_scale_rows(None, 8, 8, None, 0, p, 8, 4, None) == 1            # null x
    assert lib.rof_scale_rows(p, 4, 8, None, 0, p, 8, 4, None) == 1               # ldx < dim
    assert lib.rof_scale_rows(p, 8, 8, None, 1, p, 8, 4, None) == 1               # rsqrt without degrees
    assert lib.rof_scale_rows(p, 8, 8, None, 7, p, 8, 4, None) == 1               # unknown op
    assert lib.rof_scale_rows(p, 8, 8, None, 0, p, 8, 0, None) == 0               # nothing to do
    assert b"rof_scale_rows" in lib.rof_last_error()
    assert lib.rof_probe_read(None, 1024, 1, p, None) == 1
    assert lib.rof_probe_read(ctypes.c_void_p(p.value + 4), 1024, 1, p, None) == 1   # not 16-byte aligned
    assert lib.rof_copy_async(None, p, 16, None) == 1 and lib.rof_copy_async(p, None, 16, None) == 1
    assert lib.rof_copy_async(p, p, -1, None) == 1 and lib.rof_copy_async(None, None, 0, None) == 0
    out_ptr = ctypes.c_void_p()
    assert lib.rof_shared_alloc(0, ctypes.byref(out_ptr), p) == 1 and lib.rof_shared_alloc(64, None, p) == 1
    assert lib.rof_shared_alloc(64, ctypes.byref(out_ptr), None) == 1
    assert lib.rof_shared_open(None, ctypes.byref(out_ptr)) == 1 and lib.rof_shared_open(p, None) == 1
    assert lib.rof_shared_close(None) == 0 and lib.rof_shared_free(None) == 0
    assert lib.rof_plan_take_status(None) == 0
    assert lib.rof_plan_export_tiles(None, None, None, None, None) == 1
    handles = (ctypes.c_void_p * 2)()
    assert lib.rof_plan_create_stages_ranges(None, None, None, 0, 0, handles, None) == 1
