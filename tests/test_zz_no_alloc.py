"""rof_aggregate_static_scratch — the entry point for hosts that cannot allocate device memory
when they call (all of HBM already belongs to their own pool, or an allocation's device-wide
synchronisation is not acceptable where they call from).  It must give what rof_aggregate() gives
with a caller workspace, call after call, although every call reuses the same built-in scratch
and finds the previous call's data in it.  Collected last on purpose (file name), and written to
pass both on its own in a fresh process and after the rest of the suite."""
import ctypes

import numpy as np
import pytest
import torch

from artifact_b200 import _native
from artifact_b200.plan import AggregationPlan
from conftest import assert_close, layout_args, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
STATIC_SCRATCH_BYTES = 32 << 20          # ROF_STATIC_SCRATCH_BYTES in include/rof_b200.h


def dev_i32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)


def reuse_plan():
    g = load_golden("c5_n1024_ps2")                       # 261 reuse groups: phase A rows live in the scratch
    return g, AggregationPlan.from_v2(g["N"], *[dev_i32(a) for a in layout_args(g["layouts"], "v2")])


def long_row_plan(n=5000):
    """two rows far beyond the segment limit (256 entries for a plan this small): their segment sums live in the scratch"""
    rows = [np.arange(n, dtype=np.int32), np.arange(0, n, 2, dtype=np.int32)] + \
           [np.array([(7 * v) % n, (11 * v + 3) % n], dtype=np.int32) for v in range(2, n)]
    ptr = np.concatenate([[0], np.cumsum([len(r) for r in rows])]).astype(np.int32)
    plan = AggregationPlan.from_parts(n, dev_i32(np.concatenate(rows)), dev_i32(ptr), dev_i32(np.arange(n)))
    assert plan.info["split_rows"] == 2
    return n, plan


def test_static_scratch_matches_workspace_entry_point_call_after_call():
    g, rp = reuse_plan()
    n_long, lp = long_row_plan()
    deg_r = torch.from_numpy(np.maximum(g["degrees"], 1.0)).to(DEV)
    deg_l = torch.full((n_long,), 3.0, device=DEV)
    gen = torch.Generator(device=DEV); gen.manual_seed(77)
    # calls in a row with different plans, widths and modes: each finds the other's leftovers in the scratch
    for it, (plan, n, deg, dim, mode) in enumerate([(rp, g["N"], deg_r, 64, "gcn"), (rp, g["N"], deg_r, 64, "gcn"),
                                                    (lp, n_long, deg_l, 48, "sum"), (rp, g["N"], deg_r, 20, "mean"),
                                                    (lp, n_long, deg_l, 130, "gcn"), (lp, n_long, deg_l, 130, "gcn")]):
        x = torch.randn((n, dim), device=DEV, generator=gen)
        want = plan.aggregate(x, deg, mode)                               # existing entry point, caller workspace
        got = torch.full_like(want, float("nan"))
        plan.aggregate_static_scratch(x, deg, mode, out=got)              # new entry point, through the C ABI
        torch.cuda.synchronize()
        assert 0 < plan.workspace_bytes(dim) <= STATIC_SCRATCH_BYTES
        assert_close(got.cpu().numpy(), want.cpu().numpy(), what=f"call {it}: {mode} dim {dim}")
        assert torch.equal(got, want)                                     # same kernels, same order: bit-identical


def test_static_scratch_against_the_cpu_oracle():
    """the same entry point judged by the CPU oracle instead of by the library's other entry point"""
    import rof_oracle
    g, rp = reuse_plan()
    L = g["layouts"]
    rng = np.random.default_rng(12)
    deg_np = np.maximum(g["degrees"], 1.0)
    deg = torch.from_numpy(deg_np).to(DEV)
    for dim, mode in ((36, "gcn"), (64, "sum")):
        x = rng.standard_normal((g["N"], dim)).astype(np.float32)
        want = rof_oracle.aggregate_v2(x, L["uniqpart_column_index"], deg_np, L["uniqpart_pointers"],
                                       L["part2Node_ptr"], L["part2Node_col"], mode, True)
        for call in range(2):
            got = rp.aggregate_static_scratch(torch.from_numpy(x).to(DEV), deg, mode)
            assert_close(got.cpu().numpy(), want, what=f"static scratch vs oracle, {mode} dim {dim}, call {call}")


def test_static_scratch_checks_its_tensors_like_aggregate():
    g, rp = reuse_plan()
    n = g["N"]
    x = torch.zeros((n, 16), device=DEV)
    deg = torch.ones(n, device=DEV)
    with pytest.raises(RuntimeError):
        rp.aggregate_static_scratch(x, deg, "sum", out=torch.zeros((16, n), device=DEV).t())   # column stride != 1
    with pytest.raises(RuntimeError):
        rp.aggregate_static_scratch(x, torch.ones(2 * n, device=DEV)[::2], "gcn")               # strided degrees
    with pytest.raises(RuntimeError):
        rp.aggregate_static_scratch(x, torch.ones(n), "gcn")                                    # degrees on the host
    with pytest.raises(RuntimeError):
        rp.aggregate_static_scratch(x, deg, "sum", out=torch.zeros((n, 16)))                    # out on the host


def test_static_scratch_refuses_what_does_not_fit():
    g, rp = reuse_plan()
    dim = 40000                                            # 261 partial rows x 160 KB > 32 MiB
    assert rp.workspace_bytes(dim) > STATIC_SCRATCH_BYTES
    x = torch.zeros((g["N"], dim), device=DEV)
    out = torch.full((g["N"], dim), 5.0, device=DEV)
    with pytest.raises(_native.RofError) as e:
        rp.aggregate_static_scratch(x, None, "sum", out=out)
    assert e.value.status == 4 and "built-in scratch" in str(e.value)
    torch.cuda.synchronize()
    assert (out == 5.0).all()                              # nothing was launched
    # bad arguments are refused the same way as by rof_aggregate
    lib = _native.cuda()
    assert lib.rof_aggregate_static_scratch(None, 0, None, 0, 8, None, None, 0, None) == 1
