"""Test infrastructure only: compile the upstream `reuse_conv` CUDA extension for sm_100a.

The two upstream translation units are compiled from where they lie (nothing is copied
into this repository) with `ref_compat_shim.h` force-included, and linked into
`oracle/_ref/ROF_ref<EXT_SUFFIX>` — a pybind11 module exposing upstream's seven entry
points (reuse_conv.cpp:353-365).  It is used by the GPU tests as an on-device cross-check
of the CPU oracle and by bench.py as an extra timed column; it is never on the product path.
"""
import argparse
import os
import subprocess
import sys
import sysconfig


def main():
    ap = argparse.ArgumentParser()
    here0 = os.path.dirname(os.path.abspath(__file__))
    ap.add_argument("--ref", default=os.path.join(os.path.dirname(os.path.dirname(here0)), "reference"),
                    help="upstream tree (default: the directory `reference` next to this repository)")
    args = ap.parse_args()
    here = os.path.dirname(os.path.abspath(__file__))
    src = os.path.join(args.ref, "ROF", "reuse_conv")
    if not os.path.isdir(src):
        print("upstream tree not mounted; nothing to build")
        return 0
    from torch.utils import cpp_extension as ce
    import torch

    out_dir = os.path.join(here, "_ref")
    obj_dir = os.path.join(out_dir, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    target = os.path.join(out_dir, "ROF_ref" + suffix)
    incs = []
    for p in ce.include_paths("cuda") + [sysconfig.get_paths()["include"]]:
        incs += ["-isystem", p]
    common = ["-DTORCH_EXTENSION_NAME=ROF_ref", "-DTORCH_API_INCLUDE_EXTENSION_H",
              "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
              "-include", os.path.join(here, "ref_compat_shim.h")] + incs
    cpp_o = os.path.join(obj_dir, "reuse_conv.o")
    cu_o = os.path.join(obj_dir, "reuse_conv_kernel.o")
    cmds = [
        ["g++", "-O2", "-std=c++17", "-fPIC", "-w", "-c", os.path.join(src, "reuse_conv.cpp"), "-o", cpp_o] + common,
        ["nvcc", "-O2", "-std=c++17", "-w", "-Xcompiler", "-fPIC",
         "-gencode", "arch=compute_100a,code=sm_100a", "--expt-relaxed-constexpr",
         "-c", os.path.join(src, "reuse_conv_kernel.cu"), "-o", cu_o] + common,
    ]
    for c in cmds:
        print(" ".join(c), flush=True)
        subprocess.check_call(c)
    libdirs = ce.library_paths("cuda")
    link = ["g++", "-shared", cpp_o, cu_o, "-o", target]
    for d in libdirs:
        link += ["-L" + d, "-Wl,-rpath," + d]
    link += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    print(" ".join(link), flush=True)
    subprocess.check_call(link)
    print("built", target)
    return 0


if __name__ == "__main__":
    sys.exit(main())
