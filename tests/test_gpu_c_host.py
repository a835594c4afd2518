"""The C ABI from a plain C program (no torch, no Python in the data path): compile
tests/abi/rof_c_example.c against include/rof_b200.h and the built library, run it on the GPU."""
import os
import subprocess

import pytest

from artifact_b200 import build
from conftest import ROOT

pytestmark = pytest.mark.gpu


def test_c_program_runs_an_aggregation(tmp_path):
    exe = str(tmp_path / "rof_c_example")
    libdir = os.path.dirname(build.cuda_lib_path())
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    subprocess.check_call(["gcc", "-std=c99", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
                           "-I", os.path.join(cuda, "include"), os.path.join(ROOT, "tests", "abi", "rof_c_example.c"),
                           "-o", exe, "-L", libdir, "-lrof_b200", "-L", os.path.join(cuda, "lib64"), "-lcudart", "-lm",
                           f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{os.path.join(cuda, 'lib64')}"])
    out = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and out.stdout.startswith("OK"), out.stdout + out.stderr
