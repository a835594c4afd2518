"""In-tree build of the two native libraries.

* ``_lib/librof_b200.so`` — CUDA kernels + plan builder + the C ABI declared in
  ``include/rof_b200.h``; compiled by nvcc for sm_100a only.
* ``_lib/librof_host.so`` — host-only helpers (synthetic graph generators, the
  reuse-group search); compiled by g++ with OpenMP.

Both are plain shared objects loaded with ctypes; nothing here links against torch.
Run ``python -m artifact_b200.build`` (or ``__graft_entry__.build()``).
"""
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "_lib")
INCLUDE = os.path.join(ROOT, "include")

CUDA_SOURCES = ["plan.cu", "kernels.cu", "api.cu", "stages.cu", "static_scratch.cu"]
HOST_SOURCES = [os.path.join("host", "graphgen.cpp"), os.path.join("host", "reuse_search.cpp")]

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC,-fopenmp,-O3",
    "--expt-relaxed-constexpr",
    # no implicit contraction: the kernels round where the source says so.  The GCN terms use an
    # explicit fused multiply-add (one rounding where upstream's __fmul_rn + add has two,
    # reuse_conv_kernel.cu:270); scales, epilogue and the pre-scaling pass are separate roundings
    "-fmad=false",
]


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def cuda_lib_path():
    return os.path.join(LIB, "librof_b200.so")


def host_lib_path():
    return os.path.join(LIB, "librof_host.so")


def build_cuda(force=False, verbose=True, ptxas_info=False):
    os.makedirs(LIB, exist_ok=True)
    srcs = [os.path.join(CSRC, s) for s in CUDA_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    hdrs += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE) if f.endswith(".h")]
    target = cuda_lib_path()
    if not force and not _stale(target, srcs + hdrs + [os.path.abspath(__file__)]):
        return target
    cmd = [_nvcc()] + NVCC_FLAGS + ["-I", INCLUDE, "-I", CSRC, "-shared", "-o", target] + srcs
    if ptxas_info:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-lcudart", "-lgomp"]
    _run(cmd, verbose)
    return target


def build_host(force=False, verbose=True):
    os.makedirs(LIB, exist_ok=True)
    srcs = [os.path.join(CSRC, s) for s in HOST_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    target = host_lib_path()
    if not force and not _stale(target, srcs + [os.path.abspath(__file__)]):
        return target
    cmd = ["g++", "-O3", "-std=c++17", "-fPIC", "-shared", "-fopenmp", "-march=x86-64-v2",
           "-o", target] + srcs
    _run(cmd, verbose)
    return target


def build_all(force=False, verbose=True):
    return build_cuda(force, verbose), build_host(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
