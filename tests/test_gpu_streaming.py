"""Host-streamed passes and the pipeline's prepared calls on one GPU (the multi-GPU versions are in
test_gpu_multi.py).  Run with -m gpu on a B200."""
import numpy as np
import pytest
import torch

import rof_oracle
from artifact_b200.plan import AggregationPlan
from artifact_b200.sharding import PipelinedAggregator, ShardedFeatures
from artifact_b200.streaming import HostStreamedAggregator
from conftest import assert_close, layout_args, load_golden

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def dev_i32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)


def oracle_sum(g, x):
    L = g["layouts"]
    return rof_oracle.aggregate_v2(x, L["uniqpart_column_index"], g["degrees"], L["uniqpart_pointers"],
                                   L["part2Node_ptr"], L["part2Node_col"], "sum", True)


def test_host_streamed_passes_match_the_oracle():
    """six passes with different pinned host inputs through two device slots: every result must be the
    aggregate of its own input (no slot is overwritten before it was read or downloaded)"""
    g = load_golden("c5_n1024_ps2")
    n, dim = g["N"], 40
    plan = AggregationPlan.from_v2(n, *[dev_i32(a) for a in layout_args(g["layouts"], "v2")])
    slots = []
    for _ in range(2):
        x_dev = torch.zeros((n, dim), device=DEV)
        out_dev = torch.zeros((n, dim), device=DEV)
        slots.append((x_dev, out_dev, (lambda x=x_dev, o=out_dev: plan.aggregate(x, None, "sum", out=o))))
    hs = HostStreamedAggregator(slots, DEV)
    rng = np.random.default_rng(2)
    xs = [rng.standard_normal((n, dim)).astype(np.float32) for _ in range(6)]
    h_in = [torch.from_numpy(x).pin_memory() for x in xs]
    h_out = [torch.empty((n, dim)).pin_memory() for _ in xs]
    for a, b in zip(h_in, h_out):
        hs.submit(a, b)
    hs.synchronize()
    for k, (x, o) in enumerate(zip(xs, h_out)):
        assert_close(o.numpy(), oracle_sum(g, x), what=f"streamed pass {k}")
    assert hs.h2d_bytes == 6 * n * dim * 4 == hs.d2h_bytes
    with pytest.raises(RuntimeError):
        hs.submit(torch.zeros((n, dim)), h_out[0])              # not pinned
    # the copy-only schedule runs no pass: the slot's output buffer is downloaded as it is
    slots[0][1].fill_(3.0)
    hs2 = HostStreamedAggregator(slots[:1], DEV)
    hs2.submit(h_in[0], h_out[0], aggregate=False)
    hs2.synchronize()
    assert (h_out[0] == 3.0).all()


@pytest.mark.parametrize("mode", ["sum", "gcn"])
def test_pipeline_prepared_calls_on_one_gpu(mode):
    """world = 1: the pipeline is the plan itself; the first pass is checked call by call, the following
    ones go through the prepared C-ABI calls and must follow the buffer's new contents"""
    g = load_golden("c2_n640_ps2")
    n, dim, L = g["N"], 24, g["layouts"]
    plan = AggregationPlan.from_v2(n, *[dev_i32(a) for a in layout_args(L, "v2")])
    feats = ShardedFeatures(n, dim, 0, 1, DEV)
    pipe = PipelinedAggregator(plan, feats)
    deg_np = np.maximum(g["degrees"], 1.0)
    deg = torch.from_numpy(deg_np).to(DEV)
    out = torch.empty((n, dim), device=DEV)
    rng = np.random.default_rng(6)
    for it in range(3):
        x = rng.standard_normal((n, dim)).astype(np.float32)
        pipe.aggregate(torch.from_numpy(x).to(DEV), deg, mode, out)
        want = rof_oracle.aggregate_v2(x, L["uniqpart_column_index"], deg_np, L["uniqpart_pointers"],
                                       L["part2Node_ptr"], L["part2Node_col"], mode, True)
        assert_close(out.cpu().numpy(), want, what=f"pass {it} ({'checked' if it == 0 else 'prepared'})")
        assert (pipe._prepared is not None) and pipe.launches > 0
    # another output buffer invalidates the prepared calls (and is checked again)
    out2 = torch.empty((n, dim), device=DEV)
    pipe.aggregate(None, deg, mode, out2)
    assert torch.equal(out2, out)


@pytest.mark.parametrize("dim,chunks", [(256, None), (128, None), (100, 3), (47, 2), (64, None)])
def test_column_chunked_pipeline_on_one_gpu(dim, chunks):
    """world = 1: the features live in K column chunk buffers and every chunk is aggregated into its
    columns of the output; the result must equal the oracle on the row-major matrix"""
    from artifact_b200.sharding import ColumnChunkedFeatures, ColumnPipelinedAggregator, column_chunks
    g = load_golden("c3_n1500_ps3")
    n = g["N"]
    plan = AggregationPlan.from_v2(n, *[dev_i32(a) for a in layout_args(g["layouts"], "v2")])
    feats = ColumnChunkedFeatures(n, dim, 0, 1, DEV, chunks=chunks)
    assert feats.cols == column_chunks(dim, chunks) and feats.cols[0][0] == 0 and feats.cols[-1][1] == dim
    pipe = ColumnPipelinedAggregator(plan, feats)
    rng = np.random.default_rng(dim)
    deg_np = np.maximum(g["degrees"], 1.0)
    deg = torch.from_numpy(deg_np).to(DEV)
    out = torch.full((n, dim), 9.0, device=DEV)
    L = g["layouts"]
    for mode in ("sum", "gcn"):
        x = rng.standard_normal((n, dim)).astype(np.float32)
        pipe.aggregate(torch.from_numpy(x).to(DEV), deg, mode, out)
        want = rof_oracle.aggregate_v2(x, L["uniqpart_column_index"], deg_np, L["uniqpart_pointers"],
                                       L["part2Node_ptr"], L["part2Node_col"], mode, True)
        assert_close(out.cpu().numpy(), want, what=f"column chunks, dim {dim}, {mode}")
        idx = torch.tensor([0, n - 1, 7], device=DEV)
        assert torch.equal(feats.rows(idx).cpu(), torch.from_numpy(x)[idx.cpu()])


@pytest.mark.parametrize("dim,pieces", [(64, 2), (47, 3), (256, 4)])
def test_piece_major_pipeline_on_one_gpu(dim, pieces):
    """world = 1: the features are scattered (for GCN: scaled) into the piece-major buffer, the plan reads
    them through permuted source ids, piece by piece; repeated passes use the prepared calls"""
    from artifact_b200.sharding import PieceMajorFeatures, PieceMajorPipeline
    g = load_golden("c2_n640_ps2")
    n, L = g["N"], g["layouts"]
    feats = PieceMajorFeatures(n, dim, 0, 1, DEV, pieces)
    plan = PieceMajorPipeline.plan_from_v2(feats, *layout_args(L, "v2"))
    pipe = PieceMajorPipeline(plan, feats)
    assert len(pipe.stage_plans) == pieces
    deg_np = np.maximum(g["degrees"], 1.0)
    deg_pad = pipe.pad_degrees(torch.from_numpy(deg_np).to(DEV))
    out = torch.empty((n, dim), device=DEV)
    rng = np.random.default_rng(dim + pieces)
    for mode in ("sum", "gcn", "mean", "gcn"):
        x = rng.standard_normal((n, dim)).astype(np.float32)
        xd = torch.from_numpy(x).to(DEV)
        pipe.aggregate(xd, deg_pad, mode, out)
        want = rof_oracle.aggregate_v2(x, L["uniqpart_column_index"], deg_np, L["uniqpart_pointers"],
                                       L["part2Node_ptr"], L["part2Node_col"], mode, True)
        assert_close(out.cpu().numpy(), want, what=f"piece-major, dim {dim}, {pieces} pieces, {mode}")
    idx = torch.tensor([0, 1, n // 2, n - 1], device=DEV)
    got_rows = feats.rows(idx).cpu().numpy()                 # last pass was GCN: the buffer holds scaled rows
    assert_close(got_rows, x[idx.cpu().numpy()] / np.sqrt(deg_np[idx.cpu().numpy()])[:, None], what="scaled rows in the buffer")


@pytest.mark.gpu
@pytest.mark.parametrize("world,rank,pieces", [(3, 1, 2), (4, 0, 1), (2, 1, 3)])
def test_piece_major_own_rows_first(world, rank, pieces):
    """rank `rank` of `world` emulated on one GPU (the whole piece-major buffer is filled here, nothing
    travels): with own_first the plan has one stage more, over the rank's own slots, and the stages
    together still give the block's rows of the operator"""
    from artifact_b200.sharding import PieceMajorFeatures, PieceMajorPipeline
    g = load_golden("c2_n640_ps2")
    n, L, dim = g["N"], g["layouts"], 40
    feats = PieceMajorFeatures(n, dim, rank, world, DEV, pieces)
    plan = PieceMajorPipeline.plan_from_v2(feats, *layout_args(L, "v2"))
    pipe = PieceMajorPipeline(plan, feats, own_first=True)
    twin = PieceMajorPipeline(plan, feats, like=pipe)
    assert pipe.own_first and twin.own_first and len(pipe.stage_plans) == pieces + 1
    bounds, stage = PieceMajorPipeline.own_first_ranges(pieces, world, feats.pb, rank)
    assert bounds[0] == 0 and bounds[-1] == feats.size and sorted(set(stage)) == list(range(pieces + 1))
    own = sum(b - a for a, b, s in zip(bounds, bounds[1:], stage) if s == 0)
    assert own == pieces * feats.pb
    r0, r1 = feats.blocks[rank]
    deg_np = np.maximum(g["degrees"], 1.0)
    deg_pad = pipe.pad_degrees(torch.from_numpy(deg_np).to(DEV))
    out = torch.empty((r1 - r0, dim), device=DEV)
    rng = np.random.default_rng(world * 10 + rank)
    where = feats.perm(torch.arange(n, device=DEV))
    for mode in ("sum", "gcn", "mean"):
        x = rng.standard_normal((n, dim)).astype(np.float32)
        travelled = x / np.sqrt(deg_np)[:, None] if mode == "gcn" else x        # GCN rows travel pre-scaled
        feats.full[where] = torch.from_numpy(travelled.astype(np.float32)).to(DEV)
        for p in (pipe, twin, pipe):                                            # third time: prepared calls
            out.fill_(float("nan"))
            p.aggregate_only(deg_pad, mode, out)
            want = rof_oracle.aggregate_v2(x, L["uniqpart_column_index"], deg_np, L["uniqpart_pointers"],
                                           L["part2Node_ptr"], L["part2Node_col"], mode, True)[r0:r1]
            assert_close(out.cpu().numpy(), want, what=f"own rows first, rank {rank}/{world}, {pieces} pieces, {mode}")


@pytest.mark.gpu
@pytest.mark.parametrize("world,cols,chunks", [(4, 2, 3), (8, 4, 2), (2, 1, 2)])
def test_grid_pipeline_ranks_emulated_on_one_gpu(world, cols, chunks):
    """destination x source grid: every rank's buffers and chunk plans on one GPU, the all-gather
    replaced by filling the source buffer, the reduce-scatter by adding the partial rows of a
    destination group; kernels, scaling passes and the chunk-major row order are the real ones"""
    from artifact_b200.grid import GridLayout, GridPipeline
    from artifact_b200.plan import scale_rows
    g = load_golden("c2_n640_ps2")
    n, dim = g["N"], 20
    deg_np = np.maximum(g["degrees"], 1.0)
    deg = torch.from_numpy(deg_np).to(DEV)
    L0 = g["layouts"]
    rng = np.random.default_rng(world)
    pipes = []
    for rank in range(world):
        gl = GridLayout(n, world, rank, cols, chunks)
        pipes.append(GridPipeline(gl, gl.chunk_plans(g["indptr_dst"], g["indices_src"], device=DEV), dim, DEV))
    for mode in ("sum", "gcn", "mean"):
        x = rng.standard_normal((n, dim)).astype(np.float32)
        xd = torch.from_numpy(x).to(DEV)
        for p in pipes:                                            # own rows into the own slot (scaled for GCN)
            r0, r1 = p.layout.blocks[p.layout.rank]
            p.set_local(xd[r0:r1], deg[r0:r1], mode)
        for p in pipes:                                            # "all-gather" inside the column group
            for ii, rr in enumerate(p.layout.column_group()):
                p._src[ii * p.layout.blk:(ii + 1) * p.layout.blk].copy_(pipes[rr].own_slot())
        for p in pipes:
            for q in range(chunks):
                p.compute_chunk(q)
        want = rof_oracle.aggregate_v2(x, L0["uniqpart_column_index"], deg_np, L0["uniqpart_pointers"],
                                       L0["part2Node_ptr"], L0["part2Node_col"], mode, True)
        for p in pipes:                                            # "reduce-scatter" inside the destination group
            gl = p.layout
            total = sum(pipes[rr]._partial for rr in gl.destination_group())
            r0, r1 = gl.blocks[gl.rank]
            mine = torch.cat([total[q * gl.c * gl.cb + gl.j * gl.cb:q * gl.c * gl.cb + (gl.j + 1) * gl.cb] for q in range(chunks)])
            op = {"sum": "copy", "mean": "reciprocal", "gcn": "rsqrt"}[mode]
            out = torch.empty((r1 - r0, dim), device=DEV)
            scale_rows(mine[:r1 - r0, :dim], deg[r0:r1], op, out=out)
            assert_close(out.cpu().numpy(), want[r0:r1], what=f"grid {world // cols}x{cols}, rank {gl.rank}, {mode}")


@pytest.mark.gpu
def test_shared_store_and_copy_entry_point():
    """the buffer peers map for copy-engine transfers: its own allocation wrapped (not copied) by a
    torch tensor, usable as a feature matrix, and rof_copy_async between two such buffers"""
    import ctypes
    from artifact_b200 import _native
    from artifact_b200.sharding import ShardedFeatures, SharedStore
    a, b = SharedStore(100, 12, DEV), SharedStore(100, 12, DEV)
    assert a.tensor.data_ptr() == a.ptr and a.tensor.shape == (100, 12) and len(a.handle) == 64
    assert float(a.tensor.abs().sum()) == 0.0
    a.tensor.copy_(torch.arange(1200, device=DEV, dtype=torch.float32).view(100, 12))
    st = torch.cuda.current_stream()
    _native.check(_native.cuda().rof_copy_async(ctypes.c_void_p(b.ptr + 10 * 48), ctypes.c_void_p(a.ptr + 20 * 48), 30 * 48,
                                                ctypes.c_void_p(st.cuda_stream)))
    torch.cuda.synchronize()
    assert torch.equal(b.tensor[10:40], a.tensor[20:50]) and float(b.tensor[:10].abs().sum()) == 0.0
    a.close(); b.close()
    # a feature buffer on a shared store behaves like any other
    g = load_golden("c2_n640_ps2")
    n, L, dim = g["N"], g["layouts"], 10
    f = ShardedFeatures(n, dim, 0, 1, DEV, shared=True)
    x = np.random.default_rng(3).standard_normal((n, dim)).astype(np.float32)
    f.full.copy_(torch.from_numpy(x))
    plan = AggregationPlan.from_v2(n, *[torch.from_numpy(np.ascontiguousarray(v, dtype=np.int32)).to(DEV) for v in layout_args(L, "v2")])
    got = plan.aggregate(f.full[:n], None, "sum")
    want = rof_oracle.aggregate_v2(x, L["uniqpart_column_index"], g["degrees"], L["uniqpart_pointers"],
                                   L["part2Node_ptr"], L["part2Node_col"], "sum", True)
    assert_close(got.cpu().numpy(), want, what="features on a shared store")
    del got, plan
    f.shared.close()
