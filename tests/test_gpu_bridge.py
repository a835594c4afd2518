"""Upstream's own pybind module over the new kernels.

oracle/build_bridge.py compiles upstream's `reuse_conv.cpp` (its checked wrappers and
PYBIND11_MODULE, reuse_conv.cpp:121-365) unmodified and links it with
oracle/bridge/rof_b200_bridge.cpp, which implements the seven `*_cuda` functions on the C ABI of
include/rof_b200.h.  Here that module — `oracle/_ref/ROF_bridge*.so` — is driven directly and
through the layer class in the role upstream's `import ROF` plays (reuse_conv.py:2, 53-68,
82-88), and checked against the CPU oracle.  Skipped when the module was not built."""
import glob
import importlib.util
import os

import numpy as np
import pytest
import torch

import rof_oracle
from conftest import ROOT, assert_close, layout_args, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def load_bridge():
    so = glob.glob(os.path.join(ROOT, "oracle", "_ref", "ROF_bridge*.so"))
    if not so:
        return None
    spec = importlib.util.spec_from_file_location("ROF_bridge", so[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("name", ["c5_n1024_ps2", "c1_full_ps3", "c2_n640_ps2"])
def test_upstream_pybind_module_over_new_kernels(name):
    br = load_bridge()
    if br is None:
        pytest.skip("bridge module not built (oracle/_ref/ROF_bridge*.so)")
    assert {"SAG", "GNNA_forward", "GNNA_backward", "reuse_forward_v1", "reuse_backward_v1", "reuse_forward_v2",
            "reuse_backward_v2"} <= set(dir(br))
    g = load_golden(name)
    L, n = g["layouts"], g["N"]
    deg_np = np.maximum(g["degrees"], 1.0)
    rng = np.random.default_rng(31)
    X = rng.standard_normal((n, 20)).astype(np.float32)
    W = (rng.standard_normal((20, 16)) / 4).astype(np.float32)
    GO = rng.standard_normal((n, 16)).astype(np.float32)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    i32 = lambda a: t(np.asarray(a, dtype=np.int32))
    tX, tW, tGO, tdeg = t(X), t(W), t(GO), t(deg_np)
    ps, dw, wpb = int(L["part_size"]), 16, 4
    ci, pp, p2n = (i32(a) for a in layout_args(L, "parts"))
    v1 = [i32(a) for a in layout_args(L, "v1")]
    v2 = [i32(a) for a in layout_args(L, "v2")]
    G = len(L["part_pointers_cache"]) - 1
    cache = torch.zeros((G, 17), device=DEV)

    want = rof_oracle.GNNA_forward(X, W, L["original_column_index"], deg_np, L["part_pointers"], L["part2Node"],
                                   exact64=True)[0]
    dX, dW = rof_oracle.GNNA_backward(GO, X, W, L["original_column_index"], deg_np, L["part_pointers"],
                                      L["part2Node"], exact64=True)
    outs = {
        "GNNA": br.GNNA_forward(tX, tW, ci, tdeg, pp, p2n, ps, dw, wpb)[0],
        "ROF_v1": br.reuse_forward_v1(tX, tW, v1[0], tdeg, v1[1], v1[2], ps, dw, wpb, cache, v1[3], v1[4], v1[5])[0],
        "ROF_v2": br.reuse_forward_v2(tX, tW, v2[0], tdeg, v2[1], v2[2], v2[3], ps, dw, wpb)[0],
    }
    for k, o in outs.items():
        assert_close(o.cpu().numpy(), want, rel=2e-5, what=f"bridge {k} forward")
    if G:
        assert (cache[:, 16] == 1.0).all()             # the caching kernel's ready flags (reuse_conv_kernel.cu:485)
    grads = {
        "GNNA": br.GNNA_backward(tGO, tX, tW, ci, tdeg, pp, p2n, ps, dw, wpb),
        "ROF_v1": br.reuse_backward_v1(tGO, tX, tW, v1[0], tdeg, v1[1], v1[2], ps, dw, wpb, cache, v1[3], v1[4], v1[5]),
        "ROF_v2": br.reuse_backward_v2(tGO, tX, tW, v2[0], tdeg, v2[1], v2[2], v2[3], ps, dw, wpb),
    }
    for k, (di, dw_) in grads.items():
        assert_close(di.cpu().numpy(), dX, rel=5e-5, abs_=1e-5, what=f"bridge {k} d_input")
        assert_close(dw_.cpu().numpy(), dW, rel=5e-5, abs_=5e-3, what=f"bridge {k} d_weight")
    sag = br.SAG(tX, i32(g["indptr_dst"]), ci, tdeg, pp, p2n, ps, 20, wpb)
    assert_close(sag.cpu().numpy(), rof_oracle.SAG(X, None, L["original_column_index"], deg_np, L["part_pointers"],
                                                   L["part2Node"], exact64=True), what="bridge SAG")
    # upstream's argument checks still guard the module (reuse_conv.cpp:121-123)
    with pytest.raises(RuntimeError):
        br.GNNA_forward(tX.cpu(), tW, ci, tdeg, pp, p2n, ps, dw, wpb)
    with pytest.raises(RuntimeError):
        br.GNNA_forward(tX.t(), tW, ci, tdeg, pp, p2n, ps, dw, wpb)


def test_layer_runs_over_the_bridge_module(monkeypatch):
    """the autograd function and layer with the bridge module in the place of `import ROF`"""
    br = load_bridge()
    if br is None:
        pytest.skip("bridge module not built (oracle/_ref/ROF_bridge*.so)")
    from artifact_b200 import reuse_conv
    from artifact_b200.models import ROF_inputInfo
    monkeypatch.setattr(reuse_conv, "ROF", br)
    g = load_golden("c1_full_ps2")
    info = ROF_inputInfo.from_layouts(g["indptr_dst"].astype(np.int64), g["layouts"], device=DEV)
    L, n, deg = g["layouts"], g["N"], g["degrees"]
    for kt in ("GNNA", "ROF_v1", "ROF_v2"):
        torch.manual_seed(3)
        layer = reuse_conv.ROF_GCNConv(12, 8, add_self_loops=False, kernel_type=kt, reuse_size=info.reuse_size).to(DEV)
        x = torch.randn((n, 12), device=DEV, requires_grad=True)
        y = layer(x, info)
        y.sum().backward()
        want = rof_oracle.GNNA_forward(x.detach().cpu().numpy(), layer.weight.detach().cpu().numpy(),
                                       L["original_column_index"], deg, L["part_pointers"], L["part2Node"],
                                       exact64=True)[0] + layer.bias.detach().cpu().numpy()
        assert_close(y.detach().cpu().numpy(), want, rel=2e-5, what=f"layer over bridge, {kt}")
        assert torch.isfinite(x.grad).all() and torch.isfinite(layer.weight.grad).all()
