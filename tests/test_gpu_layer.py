"""The autograd function and layer (upstream reuse_conv.py:30-150) and the model stand-ins on the GPU."""
import numpy as np
import pytest
import torch

import rof_oracle
from artifact_b200 import graphs, search
from artifact_b200.models import ROF_GCN, ROF_GIN, ROF_inputInfo
from artifact_b200.plan import AggregationPlan
from artifact_b200.reuse_conv import ROF_GCNConv, ROF_GCNConvFunc
from conftest import assert_close, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_info(name):
    g = load_golden(name)
    info = ROF_inputInfo.from_layouts(g["indptr_dst"].astype(np.int64), g["layouts"], device=DEV)
    return g, info


@pytest.mark.parametrize("kernel_type", ["GNNA", "ROF_v1", "ROF_v2"])
def test_layer_forward_backward_matches_oracle(kernel_type):
    g, info = make_info("c1_full_ps2")          # symmetric graph with self-loops: backward is the true gradient
    N, L, deg = g["N"], g["layouts"], g["degrees"]
    torch.manual_seed(0)
    layer = ROF_GCNConv(10, 6, add_self_loops=False, kernel_type=kernel_type, reuse_size=info.reuse_size).to(DEV)
    assert layer.part_result_cache.shape == (info.reuse_size, 7) and layer.dimWorker == 6
    x = torch.randn((N, 10), device=DEV, requires_grad=True)
    y = layer(x, info)
    w = torch.randn_like(y)
    (y * w).sum().backward()
    X, W = x.detach().cpu().numpy(), layer.weight.detach().cpu().numpy()
    want = rof_oracle.GNNA_forward(X, W, L["original_column_index"], deg, L["part_pointers"], L["part2Node"],
                                   exact64=True)[0] + layer.bias.detach().cpu().numpy()
    assert_close(y.detach().cpu().numpy(), want, rel=2e-5, what="layer forward")
    dX, dW = rof_oracle.GNNA_backward(w.cpu().numpy(), X, W, L["original_column_index"], deg, L["part_pointers"],
                                      L["part2Node"], exact64=True)
    assert_close(x.grad.cpu().numpy(), dX, rel=5e-5, abs_=1e-5, what="dX")
    assert_close(layer.weight.grad.cpu().numpy(), dW, rel=5e-5, abs_=2e-4, what="dW")
    assert_close(layer.bias.grad.cpu().numpy(), w.sum(0).cpu().numpy(), rel=1e-5, abs_=1e-4, what="db")


def test_symmetric_backward_is_the_true_gradient():
    """on a symmetric graph A_hat^T = A_hat, so autograd through a dense A_hat must agree"""
    g, info = make_info("c1_full_ps3")
    N, deg = g["N"], g["degrees"]
    A = torch.zeros((N, N), dtype=torch.float64)
    dst = np.repeat(np.arange(N), np.diff(g["indptr_dst"]))
    A[dst, g["indices_src"]] = 1.0
    s = torch.from_numpy(1.0 / np.sqrt(deg.astype(np.float64)))
    A_hat = (s[:, None] * A * s[None, :]).to(DEV)
    torch.manual_seed(1)
    x = torch.randn((N, 8), device=DEV, requires_grad=True)
    w = torch.randn((8, 5), device=DEV, requires_grad=True)
    y = ROF_GCNConvFunc.apply(x, w, _with_cache(info, 5), False, "ROF_v2")
    y.pow(2).sum().backward()
    xd, wd = x.detach().double().requires_grad_(), w.detach().double().requires_grad_()
    (A_hat @ (xd @ wd)).pow(2).sum().backward()
    assert_close(x.grad.cpu().numpy(), xd.grad.cpu().numpy(), rel=1e-4, abs_=1e-4, what="dX vs dense autograd")
    assert_close(w.grad.cpu().numpy(), wd.grad.cpu().numpy(), rel=1e-4, abs_=1e-3, what="dW vs dense autograd")


def _with_cache(info, dim):
    info.part_result_cache = torch.zeros((info.reuse_size, dim + 1), device=DEV)
    info.dimWorker = min(dim, 32)
    return info


def test_argument_behaviour_like_upstream():
    g, info = make_info("shared_prefix_12_ps3")
    layer = ROF_GCNConv(4, 4, reuse_size=info.reuse_size).to(DEV)          # add_self_loops defaults to True ...
    with pytest.raises(NotImplementedError):                                 # ... which raises, reuse_conv.py:72-73
        layer(torch.ones((12, 4), device=DEV), info)
    layer = ROF_GCNConv(4, 4, add_self_loops=False, kernel_type="nope", reuse_size=info.reuse_size).to(DEV)
    with pytest.raises(NotImplementedError):
        layer(torch.ones((12, 4), device=DEV), info)
    with pytest.raises(NotImplementedError):
        ROF_GCNConv(4, 4, weight_initializer="other")
    assert ROF_GCNConv(4, 64, bias=False).dimWorker == 32 and ROF_GCNConv(4, 64, bias=False).bias is None


def test_gcn_stack_trains_a_step_and_gin_runs():
    g = graphs.config1()
    L = search.search_graph(g, 3)
    info = ROF_inputInfo.from_layouts(g.indptr_dst, L, device=DEV)
    torch.manual_seed(0)
    feats = (torch.rand((g.num_nodes, 1433), device=DEV) < 0.0127).float()
    feats = feats / feats.sum(1, keepdim=True).clamp(min=1.0)
    labels = torch.randint(0, 7, (g.num_nodes,), device=DEV)
    for kt in ("GNNA", "ROF_v1", "ROF_v2"):
        model = ROF_GCN(1433, 16, 7, 1, dropout=0.0, add_self_loops=False, reuse_size=info.reuse_size,
                        kernel_type=kt).to(DEV)
        opt = torch.optim.Adam(model.parameters(), lr=1e-2, weight_decay=5e-4)
        losses = []
        for _ in range(5):
            opt.zero_grad()
            loss = torch.nn.functional.cross_entropy(model(feats, info), labels)
            loss.backward()
            opt.step()
            losses.append(loss.item())
        assert np.isfinite(losses).all() and losses[-1] < losses[0]
    g3 = graphs.config3(0.02)
    plan = AggregationPlan.from_parts(g3.num_nodes, torch.from_numpy(g3.indices_src).to(DEV),
                                      torch.from_numpy(g3.indptr_dst.astype(np.int32)).to(DEV),
                                      torch.arange(g3.num_nodes, dtype=torch.int32, device=DEV))
    gin = ROF_GIN(128, 256, 40, 3).to(DEV)
    with torch.no_grad():
        out = gin(torch.randn((g3.num_nodes, 128), device=DEV), plan)
    assert out.shape == (g3.num_nodes, 40) and torch.isfinite(out).all()


@pytest.mark.parametrize("kernel_type", ["GNNA", "ROF_v1", "ROF_v2"])
def test_transposed_layouts_give_the_exact_gradient_on_a_directed_graph(kernel_type):
    g = graphs.config2(500 / 232965)                     # directed: A_hat != A_hat^T
    n = g.num_nodes
    fwd = ROF_inputInfo.from_layouts(g.indptr_dst, search.search_graph(g, 2), device=DEV)
    Lt = search.reuse_search(g.indptr_src, g.indices_dst, g.indptr_dst, g.indices_src, 2)   # the two CSRs swapped
    bwd = ROF_inputInfo.from_layouts(g.indptr_src, Lt, device=DEV)
    fwd.degrees = torch.clamp(fwd.degrees, min=1.0)
    fwd.with_transposed(bwd)
    A = torch.zeros((n, n), dtype=torch.float64)
    A[np.repeat(np.arange(n), np.diff(g.indptr_dst)), g.indices_src] = 1.0
    s = fwd.degrees.double().rsqrt().cpu()
    A_hat = (s[:, None] * A * s[None, :]).to(DEV)
    torch.manual_seed(3)
    x = torch.randn((n, 12), device=DEV, requires_grad=True)
    w = torch.randn((12, 8), device=DEV, requires_grad=True)
    y = ROF_GCNConvFunc.apply(x, w, _with_cache(fwd, 8), False, kernel_type)
    y.pow(2).sum().backward()
    xd, wd = x.detach().double().requires_grad_(), w.detach().double().requires_grad_()
    yd = A_hat @ (xd @ wd)
    yd.pow(2).sum().backward()
    assert_close(y.detach().cpu().numpy(), yd.detach().cpu().numpy(), rel=2e-5, what="forward")
    assert_close(x.grad.cpu().numpy(), xd.grad.cpu().numpy(), rel=1e-4, abs_=1e-3, what="dX (exact, transposed)")
    assert_close(w.grad.cpu().numpy(), wd.grad.cpu().numpy(), rel=1e-4, abs_=1e-2, what="dW (exact, transposed)")
    # without the transposed layouts the backward is upstream's convention: the forward operator again
    fwd.transposed = None
    x2 = x.detach().clone().requires_grad_()
    ROF_GCNConvFunc.apply(x2, w.detach(), _with_cache(fwd, 8), False, kernel_type).pow(2).sum().backward()
    up = (A_hat @ (2 * yd.detach())) @ wd.detach().t()
    assert_close(x2.grad.cpu().numpy(), up.cpu().numpy(), rel=1e-4, abs_=1e-3, what="dX (upstream convention)")


def test_gin_inference_matches_a_dense_fp64_model():
    """3-layer GIN (sum aggregation, eps = 0, 2-layer MLPs) on a symmetrised power-law graph"""
    g = graphs.config3(1500 / 169343)
    n = g.num_nodes
    L = search.search_graph(g, 3)
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)
    plan = AggregationPlan.from_v2(n, i32(L["uniqpart_column_index"]), i32(L["uniqpart_pointers"]),
                                   i32(L["part2Node_ptr"]), i32(L["part2Node_col"]))
    torch.manual_seed(4)
    gin = ROF_GIN(128, 256, 40, 3, eps=0.0).to(DEV)
    x = torch.randn((n, 128), device=DEV)
    with torch.no_grad():
        got = gin(x, plan).cpu().numpy()
    A = np.zeros((n, n))
    A[np.repeat(np.arange(n), np.diff(g.indptr_dst)), g.indices_src] = 1.0
    h = x.cpu().numpy().astype(np.float64)
    for i, mlp in enumerate(gin.mlps):
        z = h + A @ h
        w1, b1 = mlp[0].weight.detach().cpu().numpy().astype(np.float64), mlp[0].bias.detach().cpu().numpy()
        w2, b2 = mlp[2].weight.detach().cpu().numpy().astype(np.float64), mlp[2].bias.detach().cpu().numpy()
        h = np.maximum(z @ w1.T + b1, 0.0) @ w2.T + b2
        if i + 1 < len(gin.mlps):
            h = np.maximum(h, 0.0)
    assert_close(got, h, rel=1e-4, abs_=1e-4, what="GIN logits")


@pytest.mark.parametrize("kernel_type", ["GNNA", "ROF_v1", "ROF_v2"])
def test_eval_mode_fused_bias_relu_equals_training_path(kernel_type):
    g, info = make_info("c1_full_ps2")
    torch.manual_seed(6)
    model = ROF_GCN(24, 16, 7, 1, dropout=0.0, add_self_loops=False, reuse_size=info.reuse_size,
                    kernel_type=kernel_type).to(DEV)
    with torch.no_grad():
        for layer in model.layers:
            layer.bias.normal_()
    x = torch.randn((g["N"], 24), device=DEV)
    unfused = model(x, info).detach()                       # autograd path: bias and ReLU as separate passes
    with torch.no_grad():
        fused = model(x, info)                              # inference path: fused into the gather's store
    assert_close(fused.cpu().numpy(), unfused.cpu().numpy(), what="fused bias/ReLU vs separate passes")


@pytest.mark.parametrize("mode", ["sum", "mean"])
def test_sum_aggregate_gradient_matches_dense_autograd(mode):
    """h -> s*h + A h (sum) and s*h + D^-1 A h (mean) on a directed graph with the transposed plan:
    the gradient must be s*g + A^T g and s*g + A^T D^-1 g (degrees differ per node, so a mean
    gradient that divides by the degrees on the wrong side shows up)"""
    from artifact_b200.models import SumAggregate
    g = graphs.config2(400 / 232965)
    n = g.num_nodes
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)
    ids = torch.arange(n, dtype=torch.int32, device=DEV)
    plan = AggregationPlan.from_parts(n, i32(g.indices_src), i32(g.indptr_dst), ids)
    plan_t = AggregationPlan.from_parts(n, i32(g.indices_dst), i32(g.indptr_src), ids)
    deg = torch.from_numpy(g.degrees_f32()).to(DEV)
    A = torch.zeros((n, n), dtype=torch.float64)
    A[np.repeat(np.arange(n), np.diff(g.indptr_dst)), g.indices_src] = 1.0
    if mode == "mean":
        inv = torch.where(deg > 0, 1.0 / deg.double(), torch.zeros_like(deg, dtype=torch.float64)).cpu()
        A = inv[:, None] * A
    A = A.to(DEV)
    torch.manual_seed(8)
    h = torch.randn((n, 9), device=DEV, requires_grad=True)
    w = torch.randn((n, 9), device=DEV)
    y = SumAggregate.apply(h, plan, plan_t, deg, mode, 0.5)
    (y * w).sum().backward()
    hd = h.detach().double().requires_grad_()
    yd = 0.5 * hd + A @ hd
    (yd * w.double()).sum().backward()
    assert_close(y.detach().cpu().numpy(), yd.detach().cpu().numpy(), what=f"{mode} forward")
    assert_close(h.grad.cpu().numpy(), hd.grad.cpu().numpy(), what=f"{mode} gradient")


@pytest.mark.parametrize("kernel_type", ["GNNA", "ROF_v1", "ROF_v2"])
def test_aggregate_first_order_gives_the_same_layer(kernel_type):
    """transform_order='auto' with a narrow input: A_hat (x W) computed as (A_hat x) W; outputs and all
    three gradients must agree with the reference order (symmetric graph: the backward is exact)"""
    g, info = make_info("c1_full_ps2")
    n = g["N"]
    torch.manual_seed(11)
    ref = ROF_GCNConv(6, 20, add_self_loops=False, kernel_type=kernel_type, reuse_size=info.reuse_size).to(DEV)
    alt = ROF_GCNConv(6, 20, add_self_loops=False, kernel_type=kernel_type, reuse_size=info.reuse_size,
                      transform_order="auto").to(DEV)
    alt.load_state_dict(ref.state_dict())
    x1 = torch.randn((n, 6), device=DEV, requires_grad=True)
    x2 = x1.detach().clone().requires_grad_()
    w = torch.randn((n, 20), device=DEV)
    y1 = ref(x1, info); (y1 * w).sum().backward()
    y2 = alt(x2, info); (y2 * w).sum().backward()
    assert_close(y2.detach().cpu().numpy(), y1.detach().cpu().numpy(), rel=2e-5, what="forward")
    assert_close(x2.grad.cpu().numpy(), x1.grad.cpu().numpy(), rel=5e-5, abs_=1e-5, what="dX")
    assert_close(alt.weight.grad.cpu().numpy(), ref.weight.grad.cpu().numpy(), rel=5e-5, abs_=2e-4, what="dW")
    # a wide input keeps the reference order
    wide = ROF_GCNConv(20, 6, add_self_loops=False, kernel_type=kernel_type, reuse_size=info.reuse_size,
                       transform_order="auto").to(DEV)
    assert wide(torch.randn((n, 20), device=DEV), info).shape == (n, 6)
