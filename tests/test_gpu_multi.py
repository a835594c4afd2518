"""Row-block sharded aggregation on 2+ GPUs over NCCL: the plain all-gather path and the staged
pipeline must both reproduce the oracle.  Skipped on a single-GPU box (the host logic is covered by
test_sharding_cpu.py / test_stages_cpu.py with gloo)."""
import os
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT, layout_args, load_golden

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, name, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from artifact_b200.plan import AggregationPlan
    from artifact_b200.sharding import PipelinedAggregator, ShardedAggregator, ShardedFeatures
    g = load_golden(name)
    n, dim = g["N"], 24
    x = np.random.default_rng(4).standard_normal((n, dim)).astype(np.float32)
    deg = torch.from_numpy(np.maximum(g["degrees"], 1.0)).to(dev)
    feats = ShardedFeatures(n, dim, rank, world, dev)
    r0, r1 = feats.blocks[rank]
    local = torch.zeros((feats.block, dim), device=dev)
    local[:r1 - r0] = torch.from_numpy(x[r0:r1]).to(dev)
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)
    plan = AggregationPlan.from_v2(n, *[i32(a) for a in layout_args(g["layouts"], "v2")], rows=(r0, r1))
    res = {}
    for mode in ("sum", "gcn"):
        a = ShardedAggregator(plan, feats).aggregate(local, deg, mode).cpu().numpy()
        feats.full.zero_()
        out = torch.empty((r1 - r0, dim), device=dev)
        pipe = PipelinedAggregator(plan, feats)
        for _ in range(3):                                 # repeated passes reuse buffers and events
            pipe.aggregate(local, deg, mode, out)
        torch.cuda.synchronize()
        # a schedule whose first stage already needs peers' blocks
        half = max(world // 2, 1)
        out2 = torch.empty((r1 - r0, dim), device=dev)
        pipe2 = PipelinedAggregator(plan, feats, schedule=[list(range(half)), list(range(half, world))])
        feats.full.zero_()
        for _ in range(2):
            pipe2.aggregate(local, deg, mode, out2)
        torch.cuda.synchronize()
        # blocks of equal work instead of equal row counts, transfer stages cut into small compute stages
        from artifact_b200.sharding import row_blocks
        _, bal = row_blocks(n, world, indptr=g["indptr_dst"])
        b0, b1 = bal[rank]
        feats_b = ShardedFeatures(n, dim, rank, world, dev, bounds=bal)
        feats_b.local_view().copy_(torch.from_numpy(x[b0:b1]).to(dev))
        plan_b = AggregationPlan.from_v2(n, *[i32(a_) for a_ in layout_args(g["layouts"], "v2")], rows=(b0, b1))
        out3 = torch.empty((b1 - b0, dim), device=dev)
        pipe3 = PipelinedAggregator(plan_b, feats_b, tile_bytes=n * dim * 4 / 6, pieces=3)
        for _ in range(2):
            pipe3.aggregate(None, deg, mode, out3)
        torch.cuda.synchronize()
        # features exchanged as column chunks, one all-gather each
        from artifact_b200.sharding import ColumnChunkedFeatures, ColumnPipelinedAggregator
        cf = ColumnChunkedFeatures(n, dim, rank, world, dev, chunks=3)
        out4 = torch.empty((r1 - r0, dim), device=dev)
        cp = ColumnPipelinedAggregator(plan, cf)
        for _ in range(2):
            cp.aggregate(local[:r1 - r0], deg, mode, out4)
        torch.cuda.synchronize()
        # piece-major features: one all-gather per piece, the plan reads permuted source ids
        from artifact_b200.sharding import PieceMajorFeatures, PieceMajorPipeline
        pf = PieceMajorFeatures(n, dim, rank, world, dev, 3)
        pplan = PieceMajorPipeline.plan_from_v2(pf, *layout_args(g["layouts"], "v2"))
        pp = PieceMajorPipeline(pplan, pf)
        out5 = torch.empty((r1 - r0, dim), device=dev)
        dpad = pp.pad_degrees(deg)
        for _ in range(3):
            pp.aggregate(local[:r1 - r0], dpad, mode, out5)
        torch.cuda.synchronize()
        # the staged pipeline with the peers' blocks pulled by the copy engines out of shared buffers
        feats_c = ShardedFeatures(n, dim, rank, world, dev, bounds=bal, shared=True)
        feats_c.local_view().copy_(torch.from_numpy(x[b0:b1]).to(dev))
        out7 = torch.empty((b1 - b0, dim), device=dev)
        pipe7 = PipelinedAggregator(plan_b, feats_c, transport="copy", pieces=2)
        for it in range(3):
            if it == 2:        # new rows in the own block between passes: peers must see them, not a mix
                feats_c.local_view().copy_(torch.from_numpy(x[b0:b1]).to(dev))
            else:
                feats_c.local_view().copy_(torch.from_numpy(x[b0:b1] * (it + 2.0)).to(dev))
            pipe7.aggregate(None, deg, mode, out7)
        torch.cuda.synchronize()
        pipe7.windows.close()
        dist.barrier()
        feats_c.shared.close()
        # destinations x sources grid: all-gather inside the column group, reduce-scatter of partial
        # rows inside the destination group (2 GPUs: a 1 x 2 grid, reduce-scatter only; 4: 2 x 2)
        from artifact_b200.grid import GridLayout, GridPipeline
        gl = GridLayout(n, world, rank, GridPipeline.default_cols(world), chunks=3)
        if mode == "sum":
            grid_groups = GridPipeline.make_groups(gl)
            grid_plans = gl.chunk_plans(g["indptr_dst"], g["indices_src"], device=dev)
        gp = GridPipeline(gl, grid_plans, dim, dev, groups=grid_groups)
        out6 = torch.empty((r1 - r0, dim), device=dev)
        for _ in range(3):
            gp.aggregate(local[:r1 - r0], deg[r0:r1], mode, out6)
        torch.cuda.synchronize()
        # the same grid with every transfer a copy-engine pull out of the peers' shared buffers
        gc = GridPipeline(gl, grid_plans, dim, dev, groups=grid_groups, transport="copy")
        out8 = torch.empty((r1 - r0, dim), device=dev)
        for it in range(3):
            gc.aggregate(local[:r1 - r0] * (1.0 if it == 2 else it + 2.0), deg[r0:r1], mode, out8)
        torch.cuda.synchronize()
        gc.close_windows()
        dist.barrier()
        gc.src_store.close(); gc.part_store.close()
        res[mode] = (a, out.cpu().numpy(), out2.cpu().numpy(), (b0, out3.cpu().numpy()), out4.cpu().numpy(),
                     out5.cpu().numpy(), out6.cpu().numpy(), (b0, out7.cpu().numpy()), out8.cpu().numpy())
    gathered = [None] * world
    dist.all_gather_object(gathered, (r0, res))
    if rank == 0:
        q.put(gathered)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("name", ["c5_n1024_ps2", "c2_n640_ps2"])
def test_sharded_and_pipelined_match_oracle(name):
    import rof_oracle
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    g = load_golden(name)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + len(name)) % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, name, q)) for r in range(world)]
    for p in procs:
        p.start()
    gathered = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    x = np.random.default_rng(4).standard_normal((g["N"], 24)).astype(np.float32)
    L = g["layouts"]
    deg = np.maximum(g["degrees"], 1.0)
    from conftest import assert_close
    for mode in ("sum", "gcn"):
        want = rof_oracle.aggregate_v2(x, L["uniqpart_column_index"], deg, L["uniqpart_pointers"], L["part2Node_ptr"],
                                       L["part2Node_col"], mode, exact64=True)
        plain = np.concatenate([r[mode][0] for _, r in sorted(gathered, key=lambda t: t[0])])
        piped = np.concatenate([r[mode][1] for _, r in sorted(gathered, key=lambda t: t[0])])
        assert_close(plain, want, what=f"all-gather then aggregate, {mode}")
        assert_close(piped, want, what=f"pipelined, {mode}")
        piped2 = np.concatenate([r[mode][2] for _, r in sorted(gathered, key=lambda t: t[0])])
        assert_close(piped2, want, what=f"pipelined, two half stages, {mode}")
        piped5 = np.concatenate([r[mode][5] for _, r in sorted(gathered, key=lambda t: t[0])])
        assert_close(piped5, want, what=f"piece-major pipeline, {mode}")
        pulled = np.concatenate([o for _, o in sorted((r[mode][7] for _, r in gathered), key=lambda t: t[0])])
        assert_close(pulled, want, what=f"pipelined, copy-engine transport, {mode}")
        grid_c = np.concatenate([r[mode][8] for _, r in sorted(gathered, key=lambda t: t[0])])
        assert_close(grid_c, want, what=f"destination x source grid, copy-engine transport, {mode}")
        grid = np.concatenate([r[mode][6] for _, r in sorted(gathered, key=lambda t: t[0])])
        assert_close(grid, want, what=f"destination x source grid, {mode}")
        piped4 = np.concatenate([r[mode][4] for _, r in sorted(gathered, key=lambda t: t[0])])
        assert_close(piped4, want, what=f"column chunks, {mode}")
        piped3 = np.concatenate([o for _, o in sorted((r[mode][3] for _, r in gathered), key=lambda t: t[0])])
        assert_close(piped3, want, what=f"pipelined, blocks of equal work, transfers in 3 pieces, tiled stages, {mode}")


def test_static_scratch_entry_point_on_a_second_device():
    """the built-in scratch array exists once per GPU and its address is looked up per device: the
    no-allocation entry point must work on cuda:1 of the same process, before and after cuda:0"""
    import rof_oracle
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    from artifact_b200.plan import AggregationPlan
    from conftest import assert_close
    g = load_golden("c5_n1024_ps2")
    n, L = g["N"], g["layouts"]
    x = np.random.default_rng(9).standard_normal((n, 40)).astype(np.float32)
    want = rof_oracle.aggregate_v2(x, L["uniqpart_column_index"], g["degrees"], L["uniqpart_pointers"],
                                   L["part2Node_ptr"], L["part2Node_col"], "sum", exact64=True)
    for d in (1, 0, 1):
        dev = torch.device("cuda", d)
        i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)
        plan = AggregationPlan.from_v2(n, *[i32(a) for a in layout_args(L, "v2")], device=dev)
        got = plan.aggregate_static_scratch(torch.from_numpy(x).to(dev), None, "sum")
        assert got.device == dev
        assert_close(got.cpu().numpy(), want, what=f"static scratch on cuda:{d}")
