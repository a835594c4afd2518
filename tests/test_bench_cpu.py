"""bench.py's reference arm (CPU plain aggregation) runs without a GPU and prints the contract's keys."""
import json
import os
import subprocess
import sys

from conftest import ROOT


def test_reference_arm_prints_one_json_line():
    env = dict(os.environ, OMP_NUM_THREADS="4")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--scale", "0.01",
                          "--steps", "2", "--warmup", "1", "--dim", "32"], capture_output=True, text=True, env=env,
                         timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "edges/s" and d["value"] > 0 and d["higher_is_better"] is True
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and "sample" in d["cpu_baseline"]
    assert d["e2e"] == {"value": d["value"], "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"] and "model" not in d["config"]


def test_non_zero_rank_of_reference_arm_is_silent():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                          "--scale", "0.01"], capture_output=True, text=True, env=env, timeout=120)
    assert out.returncode == 0 and out.stdout.strip() == ""


def _prep_worker(rank, world, port, cache_dir, q):
    import argparse
    import numpy as np
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), ROF_CACHE_DIR=cache_dir, OMP_NUM_THREADS="2")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    args = argparse.Namespace(workload="c5", scale=2048 / 1048576, part_size=2)
    g, L, _, _ = bench.prepare_workload(args, rank, world)
    q.put((rank, int(g.num_edges), int(np.asarray(L["uniqpart_column_index"]).sum()), len(L["picked_fanout"])))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_share_one_search_through_the_cache(tmp_path):
    """rank 0 computes the workload and leaves it in the cache directory, rank 1 loads it: same arrays, no
    deadlock whether the cache is cold or warm"""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    for attempt in range(2):                                   # cold cache, then warm cache
        q = ctx.Queue()
        port = 29500 + (os.getpid() + 31 * attempt) % 2000
        procs = [ctx.Process(target=_prep_worker, args=(r, 2, port, str(tmp_path), q)) for r in range(2)]
        for p in procs:
            p.start()
        got = sorted(q.get(timeout=180) for _ in range(2))
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
        assert got[0][1:] == got[1][1:] and got[0][3] > 0
    assert len(list(tmp_path.glob("*.npz"))) == 1


def test_default_pipeline_and_its_description():
    """N > 1 defaults: the stage pipeline at every GPU count; an explicit kind passes through; the
    configuration text names the path that runs"""
    import argparse
    sys.path.insert(0, ROOT)
    import bench

    class G:
        num_nodes, num_edges = 1000, 50000

    auto = argparse.Namespace(pipeline_kind="auto", pieces=0, dim=64, gpus=8, workload="c2", mode="sum", part_size=2,
                              scale=1.0, tiles="auto", pipeline=True)
    for world in (2, 4, 8):
        assert bench.pipeline_kind(auto, world, G) == "stages"
    for kind in ("pieces", "columns", "stages", "grid"):
        ns = argparse.Namespace(**dict(vars(auto), pipeline_kind=kind))
        assert bench.pipeline_kind(ns, 8, G) == kind
        assert "row-block x8" in bench.workload_config(ns, G, None)["parallelism"]
    assert "copy engines" in bench.workload_config(auto, G, None)["parallelism"]
    one = argparse.Namespace(**dict(vars(auto), gpus=1))
    assert bench.workload_config(one, G, None)["parallelism"] == "single GPU"
