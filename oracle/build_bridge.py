"""Test infrastructure only: link upstream's pybind layer against the new kernels.

Upstream's `reuse_conv.cpp` (the pybind11 module with the seven checked wrappers,
reuse_conv.cpp:121-365) is compiled unmodified from where it lies and linked with
`oracle/bridge/rof_b200_bridge.cpp`, which defines the seven `*_cuda` functions upstream keeps
in reuse_conv_kernel.cu on top of the C ABI of include/rof_b200.h.  The result,
`oracle/_ref/ROF_bridge<EXT_SUFFIX>`, is upstream's own extension module running the new kernels;
tests/test_gpu_bridge.py drives it on the GPU.  Nothing is copied into this repository.
"""
import argparse
import os
import subprocess
import sys
import sysconfig


def main():
    here = os.path.dirname(os.path.abspath(__file__))
    root = os.path.dirname(here)
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.path.join(os.path.dirname(root), "reference"),
                    help="upstream tree (default: the directory `reference` next to this repository)")
    args = ap.parse_args()
    src = os.path.join(args.ref, "ROF", "reuse_conv", "reuse_conv.cpp")
    if not os.path.isfile(src):
        print("upstream tree not mounted; nothing to build")
        return 0
    import torch
    from torch.utils import cpp_extension as ce

    sys.path.insert(0, root)
    from artifact_b200 import build as b
    lib = b.build_cuda(verbose=False)
    out_dir = os.path.join(here, "_ref")
    obj_dir = os.path.join(out_dir, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    target = os.path.join(out_dir, "ROF_bridge" + suffix)
    incs = []
    for p in ce.include_paths("cuda") + [sysconfig.get_paths()["include"]]:
        incs += ["-isystem", p]
    common = ["-O2", "-std=c++17", "-fPIC", "-w", "-DTORCH_EXTENSION_NAME=ROF_bridge", "-DTORCH_API_INCLUDE_EXTENSION_H",
              "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)] + incs
    up_o = os.path.join(obj_dir, "bridge_reuse_conv.o")
    br_o = os.path.join(obj_dir, "bridge_rof_b200.o")
    cmds = [
        ["g++"] + common + ["-c", src, "-o", up_o],
        ["g++"] + common + ["-I", os.path.join(root, "include"), "-c",
                            os.path.join(here, "bridge", "rof_b200_bridge.cpp"), "-o", br_o],
    ]
    for c in cmds:
        print(" ".join(c), flush=True)
        subprocess.check_call(c)
    lib_dir = os.path.dirname(lib)
    link = ["g++", "-shared", up_o, br_o, "-o", target, "-L" + lib_dir, "-lrof_b200",
            "-Wl,-rpath,$ORIGIN/../../artifact_b200/_lib"]
    for d in ce.library_paths("cuda"):
        link += ["-L" + d, "-Wl,-rpath," + d]
    link += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    print(" ".join(link), flush=True)
    subprocess.check_call(link)
    print("built", target)
    return 0


if __name__ == "__main__":
    sys.exit(main())
