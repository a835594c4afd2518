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
