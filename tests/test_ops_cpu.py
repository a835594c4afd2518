"""Argument checks of the drop-in entry points that need no GPU: upstream's CHECK_INPUT messages
(reuse_conv.cpp:121-123) and the layer's constructor behaviour (reuse_conv.py:97-142)."""
import os
import sys

import pytest
import torch

from artifact_b200 import ops
from artifact_b200.models import ROF_GCN, ROF_inputInfo
from artifact_b200.reuse_conv import ROF_GCNConv
from conftest import ROOT


def test_cpu_tensors_are_rejected_like_upstream():
    x = torch.ones((4, 3))
    i = torch.zeros(4, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="input must be a CUDA tensor"):
        ops.GNNA_forward(x, torch.ones((3, 2)), i, torch.ones(4), i, i, 2, 2, 4)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        ops.SAG(x, i, i, torch.ones(4), i, i, 2, 2, 4)
    with pytest.raises(TypeError):
        ops.reuse_forward_v2(None, x, i, x, i, i, i, 2, 2, 4)


def test_layer_construction_matches_upstream_defaults():
    layer = ROF_GCNConv(10, 64)
    assert layer.add_self_loops is True and layer.kernel_type == "ROF_v1" and layer.dimWorker == 32
    assert layer.part_result_cache.shape == (0, 65) and layer.bias.abs().sum() == 0
    small = ROF_GCNConv(10, 7, bias=False, reuse_size=5, dimWorker=0, weight_initializer="uniform")
    assert small.dimWorker == 7 and small.bias is None and small.part_result_cache.shape == (5, 8)
    assert small.weight.abs().max() <= 1.0 / 10 ** 0.5 + 1e-6
    he = ROF_GCNConv(6, 4, weight_initializer="he")
    assert he.weight.abs().max() <= 1.0 / 6 ** 0.5 + 1e-6          # sqrt(6 / ((1 + 5) * fan_in))
    model = ROF_GCN(8, 16, 3, n_layers=2, reuse_size=4, kernel_type="ROF_v2")
    assert [tuple(l.weight.shape) for l in model.layers] == [(8, 16), (16, 16), (16, 3)]


def test_input_info_is_an_attribute_bag_with_to():
    z = torch.zeros(3, dtype=torch.int32)
    info = ROF_inputInfo(z, z, torch.ones(3), z, z, 3, 4, z, torch.zeros(1, dtype=torch.int32), z, z, z, z, z)
    assert info.partSize == 3 and info.warpPerBlock == 4 and info.reuse_size == 0
    assert info.to("cpu") is info and "partSize=3" in repr(info)
    info.with_transposed(ROF_inputInfo(z, z, torch.zeros(3), z, z, 3, 4, z, torch.zeros(1, dtype=torch.int32), z))
    assert info.transposed.degrees is info.degrees


def test_dropin_modules_resolve_like_upstreams_sys_path_convention():
    sys.path.insert(0, os.path.join(ROOT, "artifact_b200", "dropin"))
    try:
        import ROF
        import reuse_conv
        assert {"SAG", "GNNA_forward", "GNNA_backward", "reuse_forward_v1", "reuse_backward_v1", "reuse_forward_v2",
                "reuse_backward_v2"} <= set(dir(ROF))
        assert reuse_conv.ROF_GCNConv is ROF_GCNConv
    finally:
        sys.path.pop(0)
