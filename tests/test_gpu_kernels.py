"""Both gather kernels (lane groups / shared-memory ring), padded leading dimensions, the
pre-scaled GCN mode and the benchmark shapes that have odd widths, against the CPU oracle.
Run with -m gpu on a B200.  Tolerance as in test_gpu_parity.py (rel 1e-5 / abs 1e-6 on the
row scale for reordered fp32 sums; 2e-5 where an fp32 GEMM is part of the call)."""
import numpy as np
import pytest
import torch

import rof_oracle
from artifact_b200 import graphs, ops, search
from artifact_b200.plan import AggregationPlan, empty_padded, padded_width, scale_rows
from conftest import assert_close, layout_args, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev_i32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)


def v2_plan(n, L, **kw):
    return AggregationPlan.from_v2(n, *[dev_i32(a) for a in layout_args(L, "v2")], **kw)


def oracle_v2(L, deg, x, mode):
    return rof_oracle.aggregate_v2(x, L["uniqpart_column_index"], deg, L["uniqpart_pointers"], L["part2Node_ptr"],
                                   L["part2Node_col"], mode, True)


def padded(x_np):
    t = empty_padded(x_np.shape[0], x_np.shape[1], DEV)
    t.copy_(torch.from_numpy(x_np))
    return t


@pytest.fixture(params=["lanes", "ring"])
def kernel(request, monkeypatch):
    monkeypatch.setenv("ROF_KERNEL", request.param)
    return request.param


@pytest.mark.parametrize("dim", [1, 3, 4, 7, 16, 17, 33, 47, 64, 100, 127, 128, 130, 256, 300, 602, 640, 1000,
                                 1025, 1433, 2052])
def test_padded_rows_any_width(kernel, dim):
    """rows padded to a multiple of 4 floats: 128-bit loads with a ragged last vector; the output is
    once contiguous [N, dim] (masked / scalar stores) and once a padded view whose padding must stay"""
    g = load_golden("c5_n1024_ps2")
    n, L = g["N"], g["layouts"]
    rng = np.random.default_rng(1000 + dim)
    x = rng.standard_normal((n, dim)).astype(np.float32)
    plan = v2_plan(n, L)
    deg = torch.from_numpy(g["degrees"]).to(DEV)
    xp = padded(x)
    for mode in ("sum", "mean"):
        want = oracle_v2(L, g["degrees"], x, mode)
        got = plan.aggregate(xp, deg, mode)
        assert got.is_contiguous()
        assert_close(got.cpu().numpy(), want, what=f"{kernel} dim {dim} {mode} contiguous out")
        big = torch.full((n, padded_width(dim) + 4), 7.0, device=DEV)
        plan.aggregate(xp, deg, mode, out=big[:, :dim])
        assert_close(big[:, :dim].cpu().numpy(), want, what=f"{kernel} dim {dim} {mode} padded out")
        assert (big[:, dim:] == 7.0).all(), "columns beyond dim were written"
    assert plan.take_status() == 0


@pytest.mark.parametrize("dim", [7, 47, 64, 256])
def test_prescaled_gcn_equals_gcn(kernel, dim):
    g = load_golden("c2_n640_ps2")
    n, L = g["N"], g["layouts"]
    rng = np.random.default_rng(dim)
    x = rng.standard_normal((n, dim)).astype(np.float32)
    deg_np = np.maximum(g["degrees"], 1.0)
    deg = torch.from_numpy(deg_np).to(DEV)
    plan = v2_plan(n, L)
    xs = scale_rows(torch.from_numpy(x).to(DEV), deg, "rsqrt")
    assert xs.stride(0) == padded_width(dim)
    want_scaled = x * (1.0 / np.sqrt(deg_np.astype(np.float64)))[:, None]
    assert_close(xs.cpu().numpy(), want_scaled, what="scale_rows")
    got = plan.aggregate(xs, deg, "gcn_prescaled")
    assert_close(got.cpu().numpy(), oracle_v2(L, deg_np, x, "gcn"), what=f"{kernel} prescaled gcn dim {dim}")


def test_split_rows_accumulate_and_epilogue(kernel):
    """a hub row cut into segments (finished by its last-arriving segment), a staged pass
    (accumulate) and the fused epilogue, on both kernels"""
    rng = np.random.default_rng(11)
    n, dim = 3000, 72
    deg_list = np.full(n, 3)
    deg_list[5] = 2900
    deg_list[17] = 1200
    indptr = np.zeros(n + 1, np.int64)
    np.cumsum(deg_list, out=indptr[1:])
    cols = np.concatenate([np.sort(rng.choice(n, d, replace=False)) for d in deg_list]).astype(np.int32)
    plan = AggregationPlan.from_parts(n, dev_i32(cols), dev_i32(indptr), dev_i32(np.arange(n)))
    assert plan.info["split_rows"] >= 2
    x = rng.standard_normal((n, dim)).astype(np.float32)
    deg = np.diff(indptr).astype(np.float32)
    A = np.zeros((n, n))
    A[np.repeat(np.arange(n), deg_list), cols] = 1.0
    want = A @ x.astype(np.float64)
    xd, dd = torch.from_numpy(x).to(DEV), torch.from_numpy(deg).to(DEV)
    for rep in range(2):                       # twice: the arrival counters must be back at zero
        got = plan.aggregate(xd, dd, "sum")
        assert_close(got.cpu().numpy(), want, what=f"{kernel} split rows, pass {rep}")
    got = plan.aggregate(xd, dd, "mean", tiles=3)
    assert_close(got.cpu().numpy(), want / deg[:, None], what=f"{kernel} tiled mean")
    bias = torch.from_numpy(rng.standard_normal(dim).astype(np.float32)).to(DEV)
    got = plan.aggregate(xd, dd, "sum", tiles=2, bias=bias, self_x=xd, self_scale=1.5, relu=True)
    ref = np.maximum(want + 1.5 * x + bias.cpu().numpy(), 0.0)
    assert_close(got.cpu().numpy(), ref, what=f"{kernel} tiled epilogue")
    # phases issued one by one: the separate segment-reduce launch
    out = torch.empty((n, dim), device=DEV)
    for ph in (1, 2, 4):
        plan.aggregate(xd, dd, "sum", out=out, phases=ph)
    assert_close(out.cpu().numpy(), want, what=f"{kernel} phases one by one")
    assert plan.take_status() == 0


@pytest.mark.parametrize("dim", [256, 47])
def test_c4_shape_gcn_parity(kernel, dim):
    """the large undirected power-law configuration at 1 % scale (N = 24,490, ~1.24M directed edges),
    GCN normalisation, hidden width 256 and class width 47, through the drop-in entry points"""
    g = graphs.config4(0.01)
    n = g.num_nodes
    L = search.search_graph(g, 2)
    deg_np = g.degrees_f32()
    assert deg_np.min() >= 1.0
    rng = np.random.default_rng(dim)
    x = rng.standard_normal((n, 24)).astype(np.float32)
    w = (rng.standard_normal((24, dim)) / 5.0).astype(np.float32)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    idx = [dev_i32(L[k]) for k in ("uniqpart_column_index", "uniqpart_pointers", "part2Node_ptr", "part2Node_col")]
    deg = t(deg_np)
    got = ops.reuse_forward_v2(t(x), t(w), idx[0], deg, idx[1], idx[2], idx[3], 2, 32, 4)[0]
    want = rof_oracle.reuse_forward_v2(x, w, L["uniqpart_column_index"], deg_np, L["uniqpart_pointers"],
                                       L["part2Node_ptr"], L["part2Node_col"], exact64=True)[0]
    assert got.shape == (n, dim)
    assert_close(got.cpu().numpy(), want, rel=2e-5, what=f"{kernel} c4-shape forward D={dim}")
    go = rng.standard_normal((n, dim)).astype(np.float32)
    d_in, d_w = ops.reuse_backward_v2(t(go), t(x), t(w), idx[0], deg, idx[1], idx[2], idx[3], 2, 32, 4)
    dX, dW = rof_oracle.reuse_backward_v2(go, x, w, L["uniqpart_column_index"], deg_np, L["uniqpart_pointers"],
                                          L["part2Node_ptr"], L["part2Node_col"], exact64=True)
    assert_close(d_in.cpu().numpy(), dX, rel=5e-5, abs_=1e-5, what="dX")
    assert_close(d_w.cpu().numpy(), dW, rel=5e-5, abs_=5e-3, what="dW")


@pytest.mark.parametrize("which", ["GNNA", "ROF_v1", "ROF_v2"])
def test_c1_class_width_7(kernel, which):
    """the small GCN's output layer: 16 -> 7 on the 2,708-node graph with self-loops"""
    g = load_golden("c1_full_ps3")
    n, L, deg_np = g["N"], g["layouts"], g["degrees"]
    rng = np.random.default_rng(7)
    x = rng.standard_normal((n, 16)).astype(np.float32)
    w = rng.standard_normal((16, 7)).astype(np.float32)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    deg = t(deg_np)
    if which == "GNNA":
        a = [dev_i32(v) for v in layout_args(L, "parts")]
        got = ops.GNNA_forward(t(x), t(w), a[0], deg, a[1], a[2], 3, 7, 4)[0]
    elif which == "ROF_v1":
        a = [dev_i32(v) for v in layout_args(L, "v1")]
        cache = torch.zeros((len(L["part_pointers_cache"]) - 1, 8), device=DEV)
        got = ops.reuse_forward_v1(t(x), t(w), a[0], deg, a[1], a[2], 3, 7, 4, cache, a[3], a[4], a[5])[0]
        assert (cache[:, 7] == 1.0).all()
    else:
        a = [dev_i32(v) for v in layout_args(L, "v2")]
        got = ops.reuse_forward_v2(t(x), t(w), a[0], deg, a[1], a[2], a[3], 3, 7, 4)[0]
    want = rof_oracle.GNNA_forward(x, w, L["original_column_index"], deg_np, L["part_pointers"], L["part2Node"],
                                   exact64=True)[0]
    assert got.shape == (n, 7) and got.is_contiguous()
    assert_close(got.cpu().numpy(), want, rel=2e-5, what=f"{kernel} {which} D=7")


@pytest.mark.parametrize("name", ["c5_n1024_ps2", "c5_n1024_ps4", "c3_n1500_ps3", "c1_full_ps2", "c2_n640_ps2"])
@pytest.mark.parametrize("dim", [8, 47, 64, 100, 256])
@pytest.mark.parametrize("wide_groups", [False, True])
def test_shared_memory_tiles(name, dim, wide_groups, monkeypatch):
    """the tile kernel (forced on): short rows read their shared entries from shared memory; all
    three modes plus the pre-scaled one, padded rows, a staged pass and the fused epilogue; with the
    default lane groups (two vectors per lane up to 32 vectors) and with the one-vector shapes"""
    monkeypatch.setenv("ROF_TILES", "1")
    if wide_groups:
        monkeypatch.setenv("ROF_SHORT_ROWS", "0")
    monkeypatch.delenv("ROF_KERNEL", raising=False)
    g = load_golden(name)
    n, L = g["N"], g["layouts"]
    plan = v2_plan(n, L)
    assert plan.info["num_tiles"] > 0 and plan.info["tile_shared_entries"] > 0
    rng = np.random.default_rng(dim)
    x = rng.standard_normal((n, dim)).astype(np.float32)
    deg_np = np.maximum(g["degrees"], 1.0)
    deg = torch.from_numpy(deg_np).to(DEV)
    xp = padded(x)
    for mode in ("gcn", "sum", "mean"):
        got = plan.aggregate(xp, deg, mode)
        assert_close(got.cpu().numpy(), oracle_v2(L, deg_np, x, mode), what=f"tiles {name} dim {dim} {mode}")
    got = plan.aggregate(scale_rows(xp, deg, "rsqrt"), deg, "gcn_prescaled")
    assert_close(got.cpu().numpy(), oracle_v2(L, deg_np, x, "gcn"), what=f"tiles {name} dim {dim} prescaled")
    bias = torch.from_numpy(rng.standard_normal(dim).astype(np.float32)).to(DEV)
    got = plan.aggregate(xp, deg, "sum", tiles=2, bias=bias, self_x=xp, self_scale=0.5, relu=True)
    ref = np.maximum(oracle_v2(L, deg_np, x, "sum") + 0.5 * x + bias.cpu().numpy(), 0.0)
    assert_close(got.cpu().numpy(), ref, what=f"tiles {name} dim {dim} staged pass with epilogue")
    if dim == 64:   # rows that are not 16-byte aligned leave the tiles to the lane-group kernel
        xu = torch.from_numpy(np.pad(x, ((0, 0), (1, 0)))).to(DEV)[:, 1:]
        got = plan.aggregate(xu, deg, "sum")
        assert_close(got.cpu().numpy(), oracle_v2(L, deg_np, x, "sum"), what="unaligned rows")


@pytest.mark.parametrize("name", ["c5_n1024_ps2", "c2_n640_ps2"])
def test_v1_cache_mirror_with_source_tiles(name):
    """ROF_v1 with the pass cut into source tiles: every tile fills the rows of the caller's
    part_result_cache whose groups it builds (under their original ids), flag column included, and the
    output equals the untiled pass"""
    g = load_golden(name)
    n, L = g["N"], g["layouts"]
    plan = AggregationPlan.from_v1(n, *[dev_i32(a) for a in layout_args(L, "v1")])
    G = plan.info["num_groups"]
    assert G > 0
    dim = 24
    rng = np.random.default_rng(5)
    x = rng.standard_normal((n, dim)).astype(np.float32)
    deg_np = np.maximum(g["degrees"], 1.0)
    xd, deg = torch.from_numpy(x).to(DEV), torch.from_numpy(deg_np).to(DEV)
    c1 = torch.zeros((G, dim + 1), device=DEV)
    c3 = torch.full((G, dim + 1), -7.0, device=DEV)
    o1 = plan.aggregate(xd, deg, "gcn", cache_result=c1)
    o3 = plan.aggregate(xd, deg, "gcn", cache_result=c3, tiles=3)
    cache = np.zeros((G, dim + 1), np.float32)
    want = rof_oracle.aggregate_v1(x, L["column_index"], deg_np, L["part_pointers"], L["part2Node"], cache,
                                   L["part_cache_flagindex"], L["part_pointers_cache"], L["column_index_cache"],
                                   "gcn", True)
    assert_close(o1.cpu().numpy(), want, what="untiled")
    assert_close(o3.cpu().numpy(), want, what="three source tiles")
    assert (c3[:, dim] == 1.0).all() and (c1[:, dim] == 1.0).all()
    assert_close(c3.cpu().numpy(), c1.cpu().numpy(), what="part_result_cache rows, tiled vs untiled")
    with pytest.raises(RuntimeError):
        plan.aggregate(xd, deg, "gcn", cache_result=torch.zeros((G + 1, dim + 1), device=DEV), tiles=3)


@pytest.mark.parametrize("short", ["0", "1"])
@pytest.mark.parametrize("name", ["c3_n1500_ps3", "c2_n640_ps2", "c5_n1024_ps2"])
def test_short_item_lane_groups(monkeypatch, short, name):
    """widths of 9..32 vectors run on half as many lanes per item (two vectors per lane) when the items
    are short; forced on and off here over short and long rows, reuse groups (phase A items of
    part_size entries) included, in every mode, with contiguous and padded outputs"""
    monkeypatch.setenv("ROF_SHORT_ROWS", short)
    monkeypatch.setenv("ROF_TILES", "0")
    g = load_golden(name)
    n, L = g["N"], g["layouts"]
    deg_np = np.maximum(g["degrees"], 1.0)
    deg = torch.from_numpy(deg_np).to(DEV)
    plan = v2_plan(n, L)
    for dim in (33, 36, 47, 64, 65, 100, 128):
        x = np.random.default_rng(dim).standard_normal((n, dim)).astype(np.float32)
        xp = padded(x)
        for mode in ("sum", "gcn", "mean"):
            want = oracle_v2(L, deg_np, x, mode)
            got = plan.aggregate(xp, deg, mode)
            assert_close(got.cpu().numpy(), want, what=f"short={short} {name} dim {dim} {mode}")
        acc = torch.from_numpy(want.astype(np.float32)).to(DEV).contiguous()
        plan.aggregate(xp, deg, "mean", out=acc, accumulate=True)
        assert_close(acc.cpu().numpy(), 2 * want, what=f"short={short} {name} dim {dim} accumulate")
