import glob
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


# The suite exercises the reuse machinery on every fixture: ROF_v2 plans keep every group the search
# picked, also where the library's cost rule would inline them (test_plan_cpu.py tests the rule itself).
os.environ.setdefault("ROF_REUSE_MIN", "0")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    # the CPU suite needs the native libraries too (host helpers, plan builder, oracle)
    from artifact_b200 import build
    build.build_all(verbose=False)
    import rof_oracle
    rof_oracle.build()


def golden_names():
    return sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(GOLDEN, "*.npz")))


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    d = {k: z[k] for k in z.files}
    d["name"] = name
    d["N"] = int(d["num_nodes"])
    d["layouts"] = {k[4:]: v for k, v in d.items() if k.startswith("ref_")}
    d["layouts"]["part_size"] = int(d["layouts"]["part_size"])
    d["degrees"] = np.diff(d["indptr_dst"]).astype(np.float32)
    return d


@pytest.fixture(params=golden_names())
def golden(request):
    return load_golden(request.param)


def layout_args(L, which):
    """positional index arguments of the three plan constructors / oracle calls"""
    if which == "parts":
        return (L["original_column_index"], L["part_pointers"], L["part2Node"])
    if which == "v1":
        return (L["column_index"], L["part_pointers"], L["part2Node"], L["part_cache_flagindex"],
                L["part_pointers_cache"], L["column_index_cache"])
    return (L["uniqpart_column_index"], L["uniqpart_pointers"], L["part2Node_ptr"], L["part2Node_col"])


def assert_close(got, want, rel=1e-5, abs_=1e-6, what=""):
    """the benchmark's tolerance for reordered fp32 sums: |got-want| <= abs + rel*|want| with the
    magnitude taken per row (sums of mixed-sign terms are compared against the row's scale)"""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    both_nan = np.isnan(got) & np.isnan(want)
    same_inf = np.isinf(got) & np.isinf(want) & (np.sign(got) == np.sign(want))
    ok_special = both_nan | same_inf
    g = np.where(ok_special, 0.0, got)
    w = np.where(ok_special, 0.0, want)
    scale = np.maximum(np.abs(w), np.abs(w).max(axis=-1, keepdims=True) if w.ndim > 1 and w.shape[-1] else np.abs(w))
    err = np.abs(g - w)
    bad = err > abs_ + rel * scale
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.size} off; max err {err.max():.3e} (scale {scale.max():.3e})"
