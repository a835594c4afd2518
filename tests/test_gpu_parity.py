"""Parity of the CUDA path (through the C ABI) with the CPU oracle.  Run with -m gpu on a B200.

Tolerance: the benchmark's rel 1e-5 / abs 1e-6 for fp32 sums reordered by reuse (conftest.assert_close);
index structures are compared bit-exactly in test_plan_cpu.py."""
import numpy as np
import pytest
import torch

import rof_oracle
from artifact_b200 import graphs, ops
from artifact_b200.plan import AggregationPlan
from conftest import assert_close, layout_args, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BUILDERS = {"parts": AggregationPlan.from_parts, "v1": AggregationPlan.from_v1, "v2": AggregationPlan.from_v2}


def dev_i32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)


def oracle(golden, which, x, mode, exact64=True):
    L, deg = golden["layouts"], golden["degrees"]
    if which == "parts":
        return rof_oracle.aggregate_parts(x, L["original_column_index"], deg, L["part_pointers"], L["part2Node"], mode, exact64)
    if which == "v1":
        cache = np.zeros((len(L["part_pointers_cache"]) - 1, x.shape[1] + 1), np.float32)
        return rof_oracle.aggregate_v1(x, L["column_index"], deg, L["part_pointers"], L["part2Node"], cache,
                                       L["part_cache_flagindex"], L["part_pointers_cache"], L["column_index_cache"],
                                       mode, exact64)
    return rof_oracle.aggregate_v2(x, L["uniqpart_column_index"], deg, L["uniqpart_pointers"], L["part2Node_ptr"],
                                   L["part2Node_col"], mode, exact64)


@pytest.mark.parametrize("mode", ["gcn", "sum", "mean"])
@pytest.mark.parametrize("which", ["parts", "v1", "v2"])
def test_fixture_parity(golden, which, mode):
    N = golden["N"]
    deg = golden["degrees"]
    rng = np.random.default_rng(5)
    x = rng.standard_normal((N, 16)).astype(np.float32)
    plan = BUILDERS[which](N, *[dev_i32(a) for a in layout_args(golden["layouts"], which)])
    got = plan.aggregate(torch.from_numpy(x).to(DEV), torch.from_numpy(deg).to(DEV), mode).cpu().numpy()
    want = oracle(golden, which, x, mode)
    assert_close(got, want, what=f"{golden['name']} {which} {mode}")
    if "dense_" + mode in golden and mode != "gcn":
        got8 = plan.aggregate(torch.from_numpy(golden["x"]).to(DEV), torch.from_numpy(deg).to(DEV), mode).cpu().numpy()
        assert_close(got8, golden["dense_" + mode], what="vs dense fp64 fixture")


# every lane-group / vector-width path: scalar (odd), float2 (even, not /4), float4; C = 1..16; tiled (> 2048)
@pytest.mark.parametrize("dim", [1, 2, 3, 4, 7, 8, 16, 20, 32, 47, 64, 100, 128, 130, 256, 384, 602, 640, 1000, 1433,
                                 2048, 2052])
def test_feature_widths(dim):
    g = load_golden("c5_n1024_ps2")
    N = g["N"]
    rng = np.random.default_rng(dim)
    x = rng.standard_normal((N, dim)).astype(np.float32)
    plan = AggregationPlan.from_v2(N, *[dev_i32(a) for a in layout_args(g["layouts"], "v2")])
    deg = torch.from_numpy(g["degrees"]).to(DEV)
    for mode in ("gcn", "sum"):
        got = plan.aggregate(torch.from_numpy(x).to(DEV), deg, mode).cpu().numpy()
        assert_close(got, oracle(g, "v2", x, mode), what=f"dim {dim} {mode}")


def test_strided_inputs_and_outputs():
    g = load_golden("c3_n1500_ps3")
    N = g["N"]
    rng = np.random.default_rng(1)
    big = torch.from_numpy(rng.standard_normal((N, 40)).astype(np.float32)).to(DEV)
    x = big[:, 3:27]                     # ld 40, offset 3 floats: forces the scalar path
    out_big = torch.full((N, 50), 7.0, device=DEV)
    out = out_big[:, 2:26]
    plan = AggregationPlan.from_v1(N, *[dev_i32(a) for a in layout_args(g["layouts"], "v1")])
    plan.aggregate(x, torch.from_numpy(g["degrees"]).to(DEV), "sum", out=out)
    want = oracle(g, "v1", x.cpu().numpy(), "sum")
    assert_close(out.cpu().numpy(), want, what="strided")
    assert (out_big[:, :2] == 7.0).all() and (out_big[:, 26:] == 7.0).all()


def test_v1_cache_mirror_matches_upstream_semantics():
    g = load_golden("c5_n1024_ps4")
    N, L = g["N"], g["layouts"]
    dim = 12
    rng = np.random.default_rng(2)
    x = rng.standard_normal((N, dim)).astype(np.float32)
    G = len(L["part_pointers_cache"]) - 1
    cache = torch.zeros((G, dim + 1), device=DEV)
    plan = AggregationPlan.from_v1(N, *[dev_i32(a) for a in layout_args(L, "v1")])
    plan.aggregate(torch.from_numpy(x).to(DEV), torch.from_numpy(g["degrees"]).to(DEV), "gcn", cache_result=cache)
    want_cache = np.zeros((G, dim + 1), np.float32)
    rof_oracle.aggregate_v1(x, L["column_index"], g["degrees"], L["part_pointers"], L["part2Node"], want_cache,
                            L["part_cache_flagindex"], L["part_pointers_cache"], L["column_index_cache"], "gcn", False)
    c = cache.cpu().numpy()
    assert (c[:, dim] == 1.0).all()
    assert_close(c[:, :dim], want_cache[:, :dim], what="part_result_cache rows")


def _csr_as_parts(g, part_size):
    """split_part of upstream (reuse_search_ext.h:82-148) in numpy: fixed-size chunks per row"""
    ip = g.indptr_dst
    deg = np.diff(ip)
    nparts = (deg + part_size - 1) // part_size
    p2n = np.repeat(np.arange(g.num_nodes, dtype=np.int32), nparts)
    first = np.concatenate([[0], np.cumsum(nparts)])[:-1]
    within = np.arange(nparts.sum()) - np.repeat(first, nparts)
    start = np.repeat(ip[:-1], nparts) + within * part_size
    end = np.minimum(start + part_size, np.repeat(ip[1:], nparts))
    pp = np.concatenate([start, end[-1:]]).astype(np.int32) if len(start) else np.zeros(1, np.int32)
    return g.indices_src, pp, p2n


@pytest.mark.parametrize("mode", ["sum", "mean", "gcn"])
def test_long_rows_are_split_and_reduced(mode):
    """rows far beyond the segment limit (256 entries for a plan this small; degree cap 20,000 in the benchmark graph)"""
    g = graphs.config2(3000 / 232965)            # ~1.47M edges, max in-degree ~750 ... boost below
    n = g.num_nodes
    # add two very long rows: node 0 <- every node, node 1 <- every second node
    rows = [np.arange(n, dtype=np.int32), np.arange(0, n, 2, dtype=np.int32)]
    ip = [0, n, n + len(rows[1])]
    idx = [rows[0], rows[1]]
    for v in range(2, n):
        r = g.indices_src[g.indptr_dst[v]:g.indptr_dst[v + 1]]
        idx.append(r)
        ip.append(ip[-1] + len(r))
    gg = graphs.Graph("long", n, np.array(ip, np.int64), np.concatenate(idx), None, None, False, 0)
    col, pp, p2n = _csr_as_parts(gg, 3)
    deg = gg.degrees_f32()
    x = np.random.default_rng(0).standard_normal((n, 32)).astype(np.float32)
    if mode == "gcn":
        deg = np.maximum(deg, 1.0)
    plan = AggregationPlan.from_parts(n, dev_i32(col), dev_i32(pp), dev_i32(p2n))
    assert plan.info["split_rows"] >= 2 and plan.info["num_slots"] >= 3 + 2
    got = plan.aggregate(torch.from_numpy(x).to(DEV), torch.from_numpy(deg).to(DEV), mode).cpu().numpy()
    want = rof_oracle.aggregate_parts(x, col, deg, pp, p2n, mode, exact64=True)
    assert_close(got, want, what="split rows " + mode)
    # and bit-for-bit repeatable (fixed reduction order, no atomics)
    again = plan.aggregate(torch.from_numpy(x).to(DEV), torch.from_numpy(deg).to(DEV), mode).cpu().numpy()
    assert np.array_equal(got, again)


def test_empty_rows_zero_degree_and_tiny_graphs():
    # N = 1 with a self-loop; N = 3 with no edges at all; zero-width features
    p = AggregationPlan.from_parts(1, dev_i32([0]), dev_i32([0, 1]), dev_i32([0]))
    out = p.aggregate(torch.tensor([[2.0, 3.0]], device=DEV), torch.tensor([1.0], device=DEV), "gcn")
    assert out.cpu().tolist() == [[2.0, 3.0]]
    z = np.zeros(0, np.int32)
    p = AggregationPlan.from_parts(3, dev_i32(z), dev_i32(z), dev_i32(z))
    out = p.aggregate(torch.ones((3, 5), device=DEV), torch.zeros(3, device=DEV), "mean")
    assert out.shape == (3, 5) and (out == 0).all()         # empty rows are written as zeros, never left stale
    out = p.aggregate(torch.ones((3, 0), device=DEV), torch.zeros(3, device=DEV), "sum")
    assert out.shape == (3, 0)


def test_zero_in_degree_source_matches_upstream_arithmetic():
    """rsqrt(0) = inf on a source without in-edges (reuse_conv_kernel.cu:254): inf/nan must appear
    exactly where the oracle puts them"""
    # 0 -> 1, 0 -> 2, 1 -> 2 ; node 0 has in-degree 0
    col, pp, p2n = [0, 0, 1], [0, 1, 3], [1, 2]
    deg = np.array([0, 1, 2], np.float32)
    x = np.array([[1.0, 0.0], [2.0, -1.0], [3.0, 5.0]], np.float32)
    p = AggregationPlan.from_parts(3, dev_i32(col), dev_i32(pp), dev_i32(p2n))
    got = p.aggregate(torch.from_numpy(x).to(DEV), torch.from_numpy(deg).to(DEV), "gcn").cpu().numpy()
    want = rof_oracle.aggregate_parts(x, col, deg, pp, p2n, "gcn", exact64=False)
    assert np.array_equal(np.isnan(got), np.isnan(want)) and np.array_equal(np.isinf(got), np.isinf(want))
    assert_close(got, want, what="zero-degree source")


def test_upstream_entry_points_forward_backward(golden):
    """the seven `ROF.*` functions against their oracle twins, called the way reuse_conv.py:53-68,82-88 does"""
    L, N = golden["layouts"], golden["N"]
    deg = np.maximum(golden["degrees"], 1.0)        # gcn norm: keep every rsqrt finite
    rng = np.random.default_rng(9)
    X = rng.standard_normal((N, 24)).astype(np.float32)
    W = (rng.standard_normal((24, 16)) / 5).astype(np.float32)
    dO = rng.standard_normal((N, 16)).astype(np.float32)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    tX, tW, tdO, tdeg = t(X), t(W), t(dO), t(deg)
    ps, dw, wpb = L["part_size"], 16, 4
    G = len(L["part_pointers_cache"]) - 1
    cache = torch.zeros((G, 17), device=DEV)
    np_cache = np.zeros((G, 17), np.float32)
    ci, pp, p2n = (dev_i32(a) for a in layout_args(L, "parts"))
    v1 = [dev_i32(a) for a in layout_args(L, "v1")]
    v2 = [dev_i32(a) for a in layout_args(L, "v2")]

    f = ops.GNNA_forward(tX, tW, ci, tdeg, pp, p2n, ps, dw, wpb)
    assert isinstance(f, list) and len(f) == 1
    want = rof_oracle.GNNA_forward(X, W, L["original_column_index"], deg, L["part_pointers"], L["part2Node"], exact64=True)[0]
    assert_close(f[0].cpu().numpy(), want, rel=2e-5, what="GNNA_forward")       # includes the fp32 GEMM (TF32 off)

    f1 = ops.reuse_forward_v1(tX, tW, v1[0], tdeg, v1[1], v1[2], ps, dw, wpb, cache, v1[3], v1[4], v1[5])[0]
    f2 = ops.reuse_forward_v2(tX, tW, v2[0], tdeg, v2[1], v2[2], v2[3], ps, dw, wpb)[0]
    assert_close(f1.cpu().numpy(), want, rel=2e-5, what="reuse_forward_v1")
    assert_close(f2.cpu().numpy(), want, rel=2e-5, what="reuse_forward_v2")
    if G:
        assert (cache[:, 16] == 1).all()

    wb = rof_oracle.GNNA_backward(dO, X, W, L["original_column_index"], deg, L["part_pointers"], L["part2Node"], exact64=True)
    for name, res in (("GNNA_backward", ops.GNNA_backward(tdO, tX, tW, ci, tdeg, pp, p2n, ps, dw, wpb)),
                      ("reuse_backward_v1", ops.reuse_backward_v1(tdO, tX, tW, v1[0], tdeg, v1[1], v1[2], ps, dw, wpb,
                                                                  cache, v1[3], v1[4], v1[5])),
                      ("reuse_backward_v2", ops.reuse_backward_v2(tdO, tX, tW, v2[0], tdeg, v2[1], v2[2], v2[3], ps,
                                                                  dw, wpb))):
        assert len(res) == 2
        assert_close(res[0].cpu().numpy(), wb[0], rel=5e-5, abs_=1e-5, what=name + " d_input")
        assert_close(res[1].cpu().numpy(), wb[1], rel=5e-5, abs_=2e-4, what=name + " d_weight")

    s = ops.SAG(tX, t(golden["indptr_dst"]), ci, tdeg, pp, p2n, ps, dw, wpb)
    assert_close(s.cpu().numpy(), rof_oracle.SAG(X, None, L["original_column_index"], deg, L["part_pointers"],
                                                 L["part2Node"], exact64=True), what="SAG")


def test_check_input_errors_like_upstream():
    g = load_golden("shared_prefix_12_ps3")
    L = g["layouts"]
    ci, pp, p2n = (dev_i32(a) for a in layout_args(L, "parts"))
    x = torch.ones((12, 4), device=DEV)
    w = torch.ones((4, 4), device=DEV)
    deg = torch.ones(12, device=DEV)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        ops.GNNA_forward(x.cpu(), w, ci, deg, pp, p2n, 3, 4, 4)
    with pytest.raises(RuntimeError, match="must be contiguous"):
        ops.GNNA_forward(torch.ones((4, 12), device=DEV).t(), w, ci, deg, pp, p2n, 3, 4, 4)
    plan = AggregationPlan.from_parts(12, ci, pp, p2n)
    with pytest.raises(RuntimeError):
        plan.aggregate(torch.ones((11, 4), device=DEV), deg, "gcn")
    with pytest.raises(RuntimeError, match="degrees"):
        plan.aggregate(x, None, "gcn")


def test_current_stream_is_honoured():
    """work goes to torch's current stream (upstream: legacy default stream, reuse_conv_kernel.cu:313)"""
    g = load_golden("c5_n1024_ps2")
    N = g["N"]
    plan = AggregationPlan.from_v2(N, *[dev_i32(a) for a in layout_args(g["layouts"], "v2")])
    x = torch.randn((N, 64), device=DEV)
    ref = plan.aggregate(x, None, "sum")
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        y = x * 2.0                      # produced on s; consumed by the aggregation on s without a sync
        out = plan.aggregate(y, None, "sum")
    s.synchronize()
    assert torch.allclose(out, ref * 2.0, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("tiles", [2, 3, 8])
@pytest.mark.parametrize("mode", ["sum", "gcn", "mean"])
def test_source_tiles_give_the_same_sums(tiles, mode):
    """walking the feature matrix in source tiles (per-tile plans accumulated into out) only
    reorders the adds"""
    g = load_golden("c2_n640_ps2")
    N = g["N"]
    x = np.random.default_rng(12).standard_normal((N, 40)).astype(np.float32)
    deg = torch.from_numpy(np.maximum(g["degrees"], 1.0)).to(DEV)
    plan = AggregationPlan.from_v2(N, *[dev_i32(a) for a in layout_args(g["layouts"], "v2")])
    events = []
    got = plan.aggregate(torch.from_numpy(x).to(DEV), deg, mode, tiles=tiles, gather_events=events).cpu().numpy()
    assert len(events) == tiles and plan.last_launch_count() >= tiles
    gg = dict(g)
    gg["degrees"] = np.maximum(g["degrees"], 1.0)
    assert_close(got, oracle(gg, "v2", x, mode), what=f"{tiles} tiles {mode}")
    assert plan.auto_tiles(40) == 1 and plan.auto_tiles(1 << 20) >= 1


@pytest.mark.parametrize("dim", [7, 48, 2052])
@pytest.mark.parametrize("tiles", [1, 3])
@pytest.mark.parametrize("mode", ["sum", "gcn"])
def test_fused_epilogue_equals_separate_elementwise_passes(dim, tiles, mode):
    """out = relu(aggregate + self_scale * x_self + bias) fused into the store (rof_aggregate_fused)
    against the plain pass followed by torch element-wise ops; rows split into segments take the
    epilogue in the segment-reduce kernel, tiled passes only in their last tile"""
    n = 1200
    rows = [np.arange(n, dtype=np.int32), np.arange(1, n, 3, dtype=np.int32)] + \
           [np.unique(np.array([(5 * v) % n, (7 * v + 1) % n, (v * v) % n], dtype=np.int32)) for v in range(2, n)]
    rows[17] = np.zeros(0, np.int32)                       # an empty row still gets bias and self term
    ptr = np.concatenate([[0], np.cumsum([len(r) for r in rows])]).astype(np.int32)
    plan = AggregationPlan.from_parts(n, dev_i32(np.concatenate(rows)), dev_i32(ptr), dev_i32(np.arange(n)))
    assert plan.info["split_rows"] == 2
    gen = torch.Generator(device=DEV); gen.manual_seed(dim * 10 + tiles)
    x = torch.randn((n, dim), device=DEV, generator=gen)
    xs = torch.randn((n, dim), device=DEV, generator=gen)
    b = torch.randn((dim,), device=DEV, generator=gen)
    deg = torch.from_numpy(np.maximum(np.diff(ptr), 1).astype(np.float32)).to(DEV)
    base = plan.aggregate(x, deg, mode, tiles=tiles)
    for kw, want in (
        (dict(bias=b), base + b),
        (dict(self_x=xs, self_scale=1.5), base + 1.5 * xs),
        (dict(bias=b, self_x=xs, self_scale=-0.25, relu=True), torch.relu(base - 0.25 * xs + b)),
        (dict(relu=True), torch.relu(base)),
    ):
        got = plan.aggregate(x, deg, mode, tiles=tiles, **kw)
        assert_close(got.cpu().numpy(), want.cpu().numpy(), what=f"{sorted(kw)} dim {dim} tiles {tiles} {mode}")


def test_fused_epilogue_with_reuse_groups():
    g = load_golden("c5_n1024_ps2")
    N = g["N"]
    plan = AggregationPlan.from_v2(N, *[dev_i32(a) for a in layout_args(g["layouts"], "v2")])
    x = torch.randn((N, 64), device=DEV)
    b = torch.randn((64,), device=DEV)
    deg = torch.from_numpy(np.maximum(g["degrees"], 1.0)).to(DEV)
    want = torch.relu(plan.aggregate(x, deg, "gcn") + 2.0 * x + b)
    got = plan.aggregate(x, deg, "gcn", bias=b, self_x=x, self_scale=2.0, relu=True)
    assert_close(got.cpu().numpy(), want.cpu().numpy(), what="fused epilogue, ROF_v2 plan")


def test_fuzz_kernels_on_random_graphs():
    """random small graphs (empty rows, dense rows, every part size, groups or none) through the
    product's search, all three layouts, all three modes, random widths, against the fp64 oracle"""
    from artifact_b200 import search as rsearch
    rng = np.random.default_rng(4242)
    for trial in range(30):
        n = int(rng.integers(3, 90))
        p = float(rng.choice([0.05, 0.2, 0.5, 0.85]))
        ps = int(rng.integers(2, 6))
        a = rng.random((n, n)) < p
        rows = [np.flatnonzero(a[v]).astype(np.int32) for v in range(n)]
        ip = np.concatenate([[0], np.cumsum([len(r) for r in rows])]).astype(np.int64)
        ix = np.concatenate(rows).astype(np.int32) if ip[-1] else np.zeros(0, np.int32)
        t_ip, t_ix = graphs.transpose_csr(n, ip, ix)
        L = rsearch.reuse_search(ip, ix, t_ip, t_ix, ps)
        dim = int(rng.choice([1, 3, 4, 6, 16, 33, 64, 100]))
        x = rng.standard_normal((n, dim)).astype(np.float32)
        degs = np.maximum(np.diff(ip), 1).astype(np.float32)
        fake = {"layouts": L, "degrees": degs}
        tx, tdeg = torch.from_numpy(x).to(DEV), torch.from_numpy(degs).to(DEV)
        for which in ("parts", "v1", "v2"):
            plan = BUILDERS[which](n, *[dev_i32(arr) for arr in layout_args(L, which)])
            for mode in ("gcn", "sum", "mean"):
                got = plan.aggregate(tx, tdeg, mode, tiles=int(rng.integers(1, 4))).cpu().numpy()
                assert_close(got, oracle(fake, which, x, mode), what=f"trial {trial} n={n} ps={ps} {which} {mode} D={dim}")
