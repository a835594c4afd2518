"""The CPU oracle against upstream's real preprocessor output (fixtures) and a dense fp64
formula; and the three layouts against each other.  No GPU."""
import numpy as np
import pytest

import rof_oracle
from conftest import assert_close, layout_args


def _run(golden, which, x, mode, exact64=False):
    L, deg = golden["layouts"], golden["degrees"]
    if which == "parts":
        return rof_oracle.aggregate_parts(x, L["original_column_index"], deg, L["part_pointers"], L["part2Node"], mode, exact64)
    if which == "v1":
        cache = np.zeros((len(L["part_pointers_cache"]) - 1, x.shape[1] + 1), np.float32)
        out = rof_oracle.aggregate_v1(x, L["column_index"], deg, L["part_pointers"], L["part2Node"], cache,
                                      L["part_cache_flagindex"], L["part_pointers_cache"], L["column_index_cache"],
                                      mode, exact64)
        if cache.shape[0]:
            assert (cache[:, -1] == 1.0).all()          # ready flags, reuse_conv_kernel.cu:485
        return out
    return rof_oracle.aggregate_v2(x, L["uniqpart_column_index"], deg, L["uniqpart_pointers"], L["part2Node_ptr"],
                                   L["part2Node_col"], mode, exact64)


@pytest.mark.parametrize("mode", ["gcn", "sum", "mean"])
@pytest.mark.parametrize("which", ["parts", "v1", "v2"])
def test_oracle_matches_dense(golden, which, mode):
    if "x" not in golden:
        pytest.skip("fixture without dense expectation")
    want = golden["dense_" + mode]
    finite_rows = np.isfinite(want).all(axis=1)
    got64 = _run(golden, which, golden["x"], mode, exact64=True)
    got32 = _run(golden, which, golden["x"], mode, exact64=False)
    assert_close(got64[finite_rows], want[finite_rows], rel=1e-6, abs_=1e-7, what="fp64 oracle vs dense")
    assert_close(got32[finite_rows], want[finite_rows], what="fp32 oracle vs dense")


@pytest.mark.parametrize("mode", ["gcn", "sum"])
def test_three_layouts_agree(golden, mode):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((golden["N"], 5)).astype(np.float32)
    deg = golden["degrees"]
    if mode == "gcn" and (deg[np.unique(golden["indices_src"])] == 0).any():
        x[deg == 0] = 0.0  # sources with in-degree 0 give inf*0 = nan in every layout alike
    base = _run(golden, "parts", x, mode, exact64=True)
    for which in ("v1", "v2"):
        other = _run(golden, which, x, mode, exact64=True)
        assert_close(other, base, rel=1e-6, abs_=1e-7, what=f"{which} vs parts")


def test_rsqrt_is_correctly_rounded():
    # __frsqrt_rn (reuse_conv_kernel.cu:254) on every degree value the configs can produce
    from fractions import Fraction
    import math
    for d in list(range(1, 3000)) + [4096, 17420, 20000, 65535, 1 << 20, (1 << 24) - 1]:
        r = np.float32(rof_oracle.rsqrt_rn(float(d)))
        lo, hi = np.nextafter(r, np.float32(0)), np.nextafter(r, np.float32(2))
        # r is nearest to 1/sqrt(d)  <=>  the midpoints to both neighbours bracket 1/sqrt(d)
        m_lo = (Fraction(float(lo)) + Fraction(float(r))) / 2
        m_hi = (Fraction(float(hi)) + Fraction(float(r))) / 2
        assert m_lo * m_lo * d <= 1 <= m_hi * m_hi * d, d
    assert math.isinf(rof_oracle.rsqrt_rn(0.0))


def test_entry_point_mirror_shapes(golden):
    """the seven numpy entry points return what upstream's do: list of one / two arrays"""
    L, deg, N = golden["layouts"], golden["degrees"], golden["N"]
    if (deg == 0).any():
        pytest.skip("gcn norm with empty rows")
    rng = np.random.default_rng(3)
    X = rng.standard_normal((N, 6)).astype(np.float32)
    W = rng.standard_normal((6, 4)).astype(np.float32)
    G = rng.standard_normal((N, 4)).astype(np.float32)
    f0 = rof_oracle.GNNA_forward(X, W, *layout_args(L, "parts")[:1], deg, *layout_args(L, "parts")[1:])
    f2 = rof_oracle.reuse_forward_v2(X, W, L["uniqpart_column_index"], deg, L["uniqpart_pointers"], L["part2Node_ptr"],
                                     L["part2Node_col"])
    assert len(f0) == 1 and len(f2) == 1 and f0[0].shape == (N, 4)
    assert_close(f2[0], f0[0], what="v2 forward vs GNNA forward")
    b0 = rof_oracle.GNNA_backward(G, X, W, L["original_column_index"], deg, L["part_pointers"], L["part2Node"])
    assert [a.shape for a in b0] == [(N, 6), (6, 4)]
    s = rof_oracle.SAG(X, golden["indptr_dst"], L["original_column_index"], deg, L["part_pointers"], L["part2Node"])
    assert s.shape == X.shape
