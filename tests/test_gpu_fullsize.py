"""The benchmark's full-size configuration (232,965 nodes, ~114.6M edges) through size-independent
properties — the CPU oracle would need minutes per pass there:

* reuse plan (ROF_v2 layout from the search) and plain plan (original CSR) are two different index
  structures over the same graph and must agree;
* checksum: for sum aggregation 1^T (A x) = sum_n outdeg(n) x[n], computed in fp64 on the host;
* linearity: agg(a x + b y) = a agg(x) + b agg(y);
* mean of an all-ones matrix is 1 on every non-empty row; GCN of rsqrt-scaled ones is deg * rsqrt(deg) ...
* a sample of destination rows (the longest, the shortest, random ones) summed directly in fp64.
"""
import numpy as np
import pytest
import torch

from artifact_b200 import graphs, search
from artifact_b200.plan import AggregationPlan
from conftest import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def full():
    g = graphs.config2(1.0)
    L = search.search_graph(g, 2)
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32))
    n = g.num_nodes
    reuse = AggregationPlan.from_v2(n, i32(L["uniqpart_column_index"]), i32(L["uniqpart_pointers"]),
                                    i32(L["part2Node_ptr"]), i32(L["part2Node_col"]), device=torch.device(DEV))
    plain = AggregationPlan.from_parts(n, i32(g.indices_src), i32(g.indptr_dst), i32(np.arange(n)),
                                       device=torch.device(DEV))
    return g, L, reuse, plain


def test_full_size_plan_accounting(full):
    g, L, reuse, plain = full
    fan = L["picked_fanout"].astype(np.int64)
    assert plain.info["gather_entries"] == g.num_edges == reuse.info["original_edges"]
    assert reuse.info["num_groups"] == len(fan) > 50000
    assert reuse.info["gather_entries"] == g.num_edges - 2 * fan.sum() + fan.sum()
    assert reuse.info["num_items"] >= g.num_nodes


@pytest.mark.parametrize("dim,tiles", [(64, 1), (256, "auto"), (602, "auto")])
def test_full_size_reuse_equals_plain_and_checksum(full, dim, tiles):
    g, L, reuse, plain = full
    n = g.num_nodes
    gen = torch.Generator(device=DEV); gen.manual_seed(dim)
    x = torch.randn((n, dim), device=DEV, generator=gen)
    a = reuse.aggregate(x, None, "sum", tiles=tiles)
    b = plain.aggregate(x, None, "sum", tiles=1)
    # two layouts, one operator: row sums differ only by fp32 add order (rows up to 17,420 terms)
    scale = b.abs().amax(dim=1, keepdim=True).clamp(min=1.0)
    assert ((a - b).abs() / scale).max().item() < 2e-5
    outdeg = torch.from_numpy(np.diff(g.indptr_src).astype(np.float64)).to(DEV)
    want = (outdeg[:, None] * x.double()).sum(0)
    got = a.double().sum(0)
    # the column totals cancel heavily (N(0,1) features), so the error is measured against the
    # magnitude of what was added up: sum_v |out_v|, each term carrying ~1e-6 relative fp32 error
    assert ((got - want).abs() / a.double().abs().sum(0)).max().item() < 1e-6


def test_full_size_linearity_and_constants(full):
    g, L, reuse, plain = full
    n = g.num_nodes
    deg = torch.from_numpy(g.degrees_f32()).to(DEV)
    gen = torch.Generator(device=DEV); gen.manual_seed(5)
    x = torch.randn((n, 32), device=DEV, generator=gen)
    y = torch.randn((n, 32), device=DEV, generator=gen)
    lhs = reuse.aggregate(2.0 * x - 0.5 * y, deg, "mean")
    rhs = 2.0 * reuse.aggregate(x, deg, "mean") - 0.5 * reuse.aggregate(y, deg, "mean")
    assert (lhs - rhs).abs().max().item() < 1e-4
    ones = torch.ones((n, 8), device=DEV)
    m = reuse.aggregate(ones, deg, "mean")
    nonempty = deg > 0
    assert torch.allclose(m[nonempty], torch.ones_like(m[nonempty]), rtol=0, atol=2e-6)
    assert (m[~nonempty] == 0).all()
    s = plain.aggregate(ones, None, "sum")
    assert torch.equal(s[:, 0], deg)                      # exact: integer sums below 2^24


def test_full_size_sampled_rows_against_fp64(full):
    g, L, reuse, plain = full
    n = g.num_nodes
    degn = g.in_degree
    dsafe = np.maximum(g.degrees_f32(), 1.0)
    deg = torch.from_numpy(dsafe).to(DEV)
    gen = torch.Generator(device=DEV); gen.manual_seed(9)
    x = torch.randn((n, 128), device=DEV, generator=gen)
    out = reuse.aggregate(x, deg, "gcn", tiles="auto").cpu().numpy()
    xh = x.cpu().numpy().astype(np.float64)
    rows = list(np.argsort(degn)[-3:]) + list(np.argsort(degn)[:3]) + list(np.random.default_rng(0).integers(0, n, 40))
    w = 1.0 / np.sqrt(dsafe.astype(np.float64))
    want = np.stack([w[v] * (w[g.indices_src[g.indptr_dst[v]:g.indptr_dst[v + 1]], None]
                             * xh[g.indices_src[g.indptr_dst[v]:g.indptr_dst[v + 1]]]).sum(0) for v in rows])
    assert_close(out[rows], want, what="sampled rows, gcn, full size")
