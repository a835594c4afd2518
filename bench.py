#!/usr/bin/env python
"""Benchmark of the reuse aggregation hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c5] [--dim D]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...      # CPU plain aggregation on the host cores

One *step* is one forward plus one backward aggregation pass (the backward applies the same
operator to the incoming gradient, reuse_conv.py:76-92) of fp32 features of width D over the
seeded synthetic graph of the workload, through the reuse plan built from the ROF_v2 layout.
`value` is edges/s with the ORIGINAL edge count (reuse shows up as more edges per second),
inputs resident in HBM; `e2e` is the same step through the public API with pinned-host inputs
and outputs, copies inside the timed region.  With N > 1 the destination rows are cut into N
blocks of equal work; every pass moves the feature blocks between the ranks over NVLink in stages
that overlap the per-stage aggregation (by default the copy engines pull the peers' blocks out of
shared buffers; --transport nccl, --pipeline-kind and --no-pipeline select the other paths) and the
same total work is divided (strong scaling).  On one GPU a feature matrix
larger than L2 is walked in source tiles (--tiles).  After the timed region every rank
recomputes a sample of its output rows in fp64 on the host (`check`); a failed check makes the
run exit non-zero.  Prints ONE JSON line on rank 0.
"""
import argparse
import glob
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (default feature width, part_size, mode)
    "c2": (256, 2, "sum"),
    "c3": (128, 2, "sum"),
    "c4": (256, 2, "gcn"),
    "c5": (64, 2, "sum"),
}
CACHE_VERSION = 2          # bump when the graph generators or the search change what they produce


# dram__bytes_read.sum + dram__bytes_write.sum of one pass of the dominant kernel, from committed
# ncu captures (one per kernel change); None where no capture exists
NCU_DRAM_BYTES_PER_PASS = {
    "c2:D256:sum": 3.35e9,     # 4 source tiles; two captured: 0.71 and 0.96 GB (untiled first version: 25.0 GB)
    "c2:D256:gcn": 3.9e9,      # two of four tiles captured: 0.84 and 1.11 GB
    "c2:D128:sum": 1.5e9,      # one of two tiles captured: 0.76 GB
    "c2:D602:sum": 17.2e9,     # two of eight tiles captured: 1.80 and 2.49 GB
    "c5:D64:sum": 2.04e9,      # tile kernel
}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 50 ms while the timed region (a few hundred ms) runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = [l for (t, l) in self.lines if t0 - 0.2 <= t <= t1 + 0.3] or [l for (_, l) in self.lines]
        for l in inside:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_graph(name, scale):
    from artifact_b200 import graphs
    return graphs.CONFIGS[name](scale)


# --------------------------------------------------------------------------------------------
# reference arm: the reuse-free CSR gather-sum on the host cores (C/OpenMP restatement; upstream
# has no CPU implementation of this path, reuse_conv.cpp:238,278,310,341)
# --------------------------------------------------------------------------------------------
def cpu_plain(g, dim, mode, seconds_budget, steps=1, warmup=0, threads=0):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import rof_oracle
    n = g.num_nodes
    rng = np.random.default_rng(1)
    x = rng.standard_normal((n, dim), dtype=np.float32)
    deg = np.maximum(g.degrees_f32(), 1.0)
    out = np.zeros((n, dim), np.float32)
    from artifact_b200 import _native
    cores = threads or _native.host_cores()          # all cores of the affinity mask, whatever OMP_NUM_THREADS says
    ip = g.indptr_dst
    # probe ~1% of the edges to size a sample that fits the budget
    r_probe = int(np.searchsorted(ip, max(1, g.num_edges // 100)))
    t = time.perf_counter()
    rof_oracle.plain_csr(x, ip, g.indices_src, deg, mode, rows=(0, max(1, r_probe)), num_threads=cores, out=out)
    rate = max(ip[max(1, r_probe)], 1) / max(time.perf_counter() - t, 1e-6)            # edges/s, cold
    per_step = seconds_budget / max(steps + warmup, 1)
    want_edges = int(min(g.num_edges, max(rate * per_step, g.num_edges * 0.01)))
    r1 = int(np.searchsorted(ip, want_edges))
    r1 = min(max(r1, 1), n)
    edges = int(ip[r1])
    times = []
    for i in range(warmup + steps):
        t = time.perf_counter()
        for _ in range(2):                                 # forward + backward pass, like the GPU step
            rof_oracle.plain_csr(x, ip, g.indices_src, deg, mode, rows=(0, r1), num_threads=cores, out=out)
        dt = time.perf_counter() - t
        if i >= warmup:
            times.append(dt)
    ms = 1e3 * float(np.mean(times))
    return {"value": 2 * edges / (ms / 1e3), "unit": "edges/s", "cores": int(cores), "kind": "port",
            "sample": f"rows [0,{r1}) of the workload = {edges} of {g.num_edges} edges, fwd+bwd, D={dim}, "
                      f"{steps} step(s)", "ms_per_step": ms}


def cpu_torch_sparse(g, dim, seconds_budget=6.0):
    """The same reuse-free sum as torch's own CSR x dense product on the host cores: the stand-in for
    the PyG / torch_sparse CPU path the benchmark names (not installable here, no network)."""
    import torch
    from artifact_b200 import _native
    cores = _native.host_cores()
    torch.set_num_threads(cores)
    n, ip = g.num_nodes, g.indptr_dst
    r1 = int(min(n, max(1, np.searchsorted(ip, max(1, g.num_edges // 50)))))
    x = torch.randn((n, dim))

    def make(rows):
        e = int(ip[rows])
        return torch.sparse_csr_tensor(torch.from_numpy(ip[:rows + 1].astype(np.int64)),
                                       torch.from_numpy(g.indices_src[:e].astype(np.int64)), torch.ones(e),
                                       size=(rows, n)), e

    a, e = make(r1)
    t = time.perf_counter(); a @ x; dt = max(time.perf_counter() - t, 1e-6)
    want = int(min(g.num_edges, max(e, e * (seconds_budget / 4.0) / dt)))
    r1 = int(min(n, max(1, np.searchsorted(ip, want))))
    a, e = make(r1)
    a @ x
    times = []
    for _ in range(3):
        t = time.perf_counter(); a @ x; times.append(time.perf_counter() - t)
    s = float(np.mean(times))
    return {"value": e / s, "unit": "edges/s", "cores": int(cores), "kind": "torch.sparse CSR x dense (forward pass)",
            "sample": f"rows [0,{r1}) = {e} of {g.num_edges} edges, D={dim}, 3 passes"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl, dim, mode = args.workload, args.dim, args.mode
    g = build_graph(wl, args.scale)
    cb = cpu_plain(g, dim, mode, seconds_budget=120.0, steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": "aggregation edges/s", "value": cb["value"], "unit": "edges/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, g, None),
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


_V2_KEYS = ("uniqpart_column_index", "uniqpart_pointers", "part2Node_ptr", "part2Node_col", "picked_fanout",
            "part2Node")
_V1_KEYS = ("column_index", "part_pointers", "part_cache_flagindex", "part_pointers_cache", "column_index_cache")


class _Lazy(dict):
    """layout arrays read from the cache file on first use (the ROF_v1 arrays are only needed by the
    upstream-kernel comparison)"""

    def __init__(self, z, keys):
        super().__init__()
        self._z, self._keys = z, set(keys)

    def __missing__(self, k):
        if k not in self._keys:
            raise KeyError(k)
        v = self._z[k]
        self[k] = v
        return v

    def __contains__(self, k):
        return dict.__contains__(self, k) or k in self._keys


def prepare_workload(args, rank, world):
    """-> (graph, layouts, seconds for graph, seconds for search).  Everything is seeded, so every
    rank could compute it; to keep the host cores for one search, rank 0 computes and leaves the
    arrays in a cache directory that the other ranks (and the next invocation on the same box) load."""
    from artifact_b200 import graphs
    cache_dir = os.environ.get("ROF_CACHE_DIR", "/tmp/rof_b200_cache")
    path = os.path.join(cache_dir, f"{args.workload}_scale{args.scale}_ps{args.part_size}_v{CACHE_VERSION}.npz")

    def compute():
        from artifact_b200 import _native, search
        _native.use_all_host_cores()          # torchrun exports OMP_NUM_THREADS=1; only rank 0 computes
        t0 = time.time()
        g = build_graph(args.workload, args.scale)
        tg = time.time() - t0
        t0 = time.time()
        L = search.search_graph(g, args.part_size)
        return g, L, tg, time.time() - t0

    def load():
        z = np.load(path)
        g = graphs.Graph(args.workload, int(z["num_nodes"]), z["indptr_dst"], z["indices_src"], None, None,
                         bool(z["symmetric"]), 0)
        L = _Lazy(z, _V2_KEYS + _V1_KEYS)
        L["part_size"] = args.part_size
        L["original_column_index"] = g.indices_src
        return g, L

    result = None
    if rank == 0:
        if os.path.exists(path):
            try:
                t0 = time.time()
                g, L = load()
                result = (g, L, time.time() - t0, 0.0)
            except Exception:
                result = None
        if result is None:
            result = compute()
            g, L = result[0], result[1]
            try:
                os.makedirs(cache_dir, exist_ok=True)
                tmp = path + f".tmp{os.getpid()}.npz"
                np.savez(tmp, num_nodes=np.int64(g.num_nodes), symmetric=np.int64(g.symmetric),
                         indptr_dst=g.indptr_dst, indices_src=g.indices_src,
                         **{k: L[k] for k in _V2_KEYS + _V1_KEYS})
                os.replace(tmp, path)
            except Exception:
                pass
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    if result is None:
        try:
            t0 = time.time()
            g, L = load()
            result = (g, L, time.time() - t0, 0.0)
        except Exception:
            result = compute()
    return result


def pipeline_kind(args, world, g):
    """--pipeline-kind auto: the stage pipeline, whose transfers the copy engines carry (4 B200s: 3.17 ms per
    step against 3.62 ms with piece-major all-gathers on the 114.6M-edge graph, 11.97 against 12.55 and 0.81
    against 1.09 on the other two configurations; 2 B200s: 16.8 against 19.8 ms where the gather is HBM-bound)."""
    kind = getattr(args, "pipeline_kind", "auto")
    return "stages" if kind == "auto" else kind


def workload_config(args, g, ratios):
    c = {"workload": f"{args.workload}: seeded synthetic graph N={g.num_nodes} E={g.num_edges}, fp32 features "
                     f"D={args.dim}, {args.mode} aggregation, forward+backward pass per step",
         "part_size": args.part_size, "layout": "ROF_v2", "scale": args.scale, "source_tiles": args.tiles,
         "l2": "feature matrix and index arrays together exceed L2 (126 MB); no flush between iterations",
         "parallelism": (f"row-block x{args.gpus}, "
                         + ({"pieces": "piece-major features: one all-gather per L2-sized piece of every block, overlapped "
                                       "with the aggregation of the piece before",
                             "columns": "features exchanged in column chunks, one all-gather each, overlapped with the "
                                        "chunks' aggregation",
                             "stages": "blocks of equal work, peers' blocks fetched in stages (copy engines, or NCCL "
                                       "send/receive) overlapped with per-stage aggregation",
                             "grid": "destination x source grid: all-gather inside the column group, partial rows "
                                     "reduce-scattered inside the destination group chunk by chunk"
                             }[pipeline_kind(args, args.gpus, g)]
                            if args.pipeline else "all-gather then aggregate"))
         if args.gpus > 1 else "single GPU"}
    if ratios is not None:
        c["reuse"] = ratios
    return c


# --------------------------------------------------------------------------------------------
# one workload on this rank: plans, buffers, timing, check
# --------------------------------------------------------------------------------------------
class Job:
    def __init__(self, ns, rank, world, dev, want_plain):
        import torch
        from artifact_b200 import search
        from artifact_b200.plan import AggregationPlan
        from artifact_b200.sharding import (ColumnChunkedFeatures, ColumnPipelinedAggregator, PieceMajorFeatures,
                                            PieceMajorPipeline, PipelinedAggregator, ShardedFeatures, row_blocks)
        self.torch, self.ns, self.rank, self.world, self.dev = torch, ns, rank, world, dev
        self.g, self.L, self.t_graph, self.t_search = prepare_workload(ns, rank, world)
        g, L = self.g, self.L
        self.n, self.E, self.D, self.mode = g.num_nodes, g.num_edges, ns.dim, ns.mode
        self.ratios = search.reuse_ratios(L)
        n, D = self.n, self.D
        kind = pipeline_kind(ns, world, g) if (world > 1 and ns.pipeline) else None
        self.kind = kind
        # the staged pipeline's transfers are point to point and take any block size: blocks of equal work;
        # the collectives of the other paths need equal row counts
        self.blk, self.blocks = row_blocks(n, world, indptr=g.indptr_dst if kind == "stages" else None)
        self.r0, self.r1 = self.blocks[rank]
        t0 = time.time()
        i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32))
        self.full_x = self.full_g = None
        if kind == "grid":
            from artifact_b200.grid import GridLayout, GridPipeline
            self.grid = GridLayout(n, world, rank, getattr(ns, "grid_cols", 0) or GridPipeline.default_cols(world),
                                   getattr(ns, "chunks", 0) or 4)
            self.grid_groups = GridPipeline.make_groups(self.grid)
            self.grid_plans = self.grid.chunk_plans(g.indptr_dst, g.indices_src, device=dev)
            self.plan = self.grid_plans[0]
        elif kind == "pieces":
            P = getattr(ns, "pieces", 0) or PieceMajorPipeline.default_pieces(n, D, world, g.num_edges / max(n, 1))
            self.feat_x = PieceMajorFeatures(n, D, rank, world, dev, P)
            self.feat_g = PieceMajorFeatures(n, D, rank, world, dev, P)
            self.plan = PieceMajorPipeline.plan_from_v2(self.feat_x, *[L[k] for k in (
                "uniqpart_column_index", "uniqpart_pointers", "part2Node_ptr", "part2Node_col")], device=dev)
        else:
            v2 = [i32(L[k]) for k in ("uniqpart_column_index", "uniqpart_pointers", "part2Node_ptr", "part2Node_col")]
            self.plan = AggregationPlan.from_v2(n, *v2, rows=(self.r0, self.r1), device=dev)
            del v2
        # the plan uses the groups only where they save enough gathered rows (rof_plan_create_v2)
        self.ratios["groups_used_by_this_rank_s_plan"] = self.plan.info["num_groups"]
        self.ratios["gathered_rows_of_this_rank_s_plan"] = (self.plan.info["gather_entries"] if kind != "grid" else
                                                            sum(p.info["gather_entries"] for p in self.grid_plans))
        self.plain = None
        if want_plain:
            self.plain = AggregationPlan.from_parts(n, i32(g.indices_src), i32(g.indptr_dst), i32(np.arange(n)),
                                                    rows=(self.r0, self.r1), device=dev)
        self.deg = torch.from_numpy(np.maximum(g.degrees_f32(), 1.0)).to(dev)
        gen = torch.Generator(device=dev); gen.manual_seed(1234)
        rows = self.r1 - self.r0
        self.out_f = torch.empty((rows, D), device=dev)
        self.out_b = torch.empty((rows, D), device=dev)
        self.pipes = {}
        self.tiles = 1
        if kind == "pieces":
            # every rank draws the same full row-major matrices: its own rows are what it contributes per
            # pass (scattered, and for GCN scaled, into its slots of the piece-major buffer), the rest is
            # what the output check compares against
            self.full_x = torch.empty((n, D), device=dev).normal_(generator=gen)
            self.full_g = torch.empty((n, D), device=dev).normal_(generator=gen)
            px = PieceMajorPipeline(self.plan, self.feat_x, own_first=bool(getattr(ns, "own_first", 0)))
            self.pipes = {id(self.feat_x): px, id(self.feat_g): PieceMajorPipeline(self.plan, self.feat_g, like=px)}
            self.deg_pad = px.pad_degrees(self.deg)
            self.stage_info = {"kind": "piece-major features, one all-gather per piece, plan split by piece",
                               "pieces": self.feat_x.pieces, "rows_per_rank_and_piece": self.feat_x.pb,
                               "own_rows_first": px.own_first, "compute_stages": len(px.stage_plans)}
        elif kind == "grid":
            self.full_x = torch.empty((n, D), device=dev).normal_(generator=gen)
            self.full_g = torch.empty((n, D), device=dev).normal_(generator=gen)
            tr = "nccl" if getattr(ns, "transport", "auto") == "nccl" else "copy"
            px = GridPipeline(self.grid, self.grid_plans, D, dev, groups=self.grid_groups, transport=tr)
            pg = GridPipeline(self.grid, self.grid_plans, D, dev, like=px, transport=tr)
            self.feat_x, self.feat_g = px, pg
            self.pipes = {id(px): px, id(pg): pg}
            self.deg_local = self.deg[self.r0:self.r1].contiguous()
            self.stage_info = {"kind": "destination x source grid", "transport": px.transport, "grid": [self.grid.r, self.grid.c],
                               "destination_chunks": self.grid.q, "rows_per_rank_and_chunk": self.grid.cb,
                               "received_rows_fraction": round((self.grid.r + self.grid.c - 2) / world, 4)}
        elif kind == "columns":
            # every rank draws the same full matrices, so the all-gathered content is what it already holds
            self.feat_x = ColumnChunkedFeatures(n, D, rank, world, dev, chunks=getattr(ns, "chunks", 0) or None)
            self.feat_g = ColumnChunkedFeatures(n, D, rank, world, dev, chunks=getattr(ns, "chunks", 0) or None)
            self.feat_x.fill_normal_(gen); self.feat_g.fill_normal_(gen)
            px = ColumnPipelinedAggregator(self.plan, self.feat_x)
            self.pipes = {id(self.feat_x): px, id(self.feat_g): ColumnPipelinedAggregator(self.plan, self.feat_g)}
            self.stage_info = {"kind": "column chunks, one all-gather each", "column_chunks": self.feat_x.cols,
                               "source_tiles_per_chunk": px.tiles}
        else:
            bounds = self.blocks if kind == "stages" else None
            want = getattr(ns, "transport", "auto") if kind == "stages" else "nccl"
            sched = [[int(k) for k in st.split(",")] for st in ns.schedule.split("|")] if getattr(ns, "schedule", "") else None

            def build(transport):
                fx = ShardedFeatures(n, D, rank, world, dev, bounds=bounds, shared=transport == "copy")
                fg = ShardedFeatures(n, D, rank, world, dev, bounds=bounds, shared=transport == "copy")
                if kind != "stages":
                    return fx, fg, None, None
                px = PipelinedAggregator(self.plan, fx, schedule=sched, pieces=getattr(ns, "pieces", 0) or None,
                                         transport=transport)
                return fx, fg, px, PipelinedAggregator(self.plan, fg, like=px, transport=transport)

            transport, why = ("copy" if want in ("auto", "copy") else "nccl"), None
            if transport == "copy":
                # mapping the peers' buffers can fail where interprocess handles are not allowed; every rank
                # then falls back to NCCL send/receive together (the constructors' collectives have completed
                # on every rank by the time one of them raises)
                built = None
                try:
                    built = build("copy")
                except Exception as ex:          # noqa: BLE001 - reported in the JSON line
                    why = repr(ex)[:200]
                import torch.distributed as dist
                flag = torch.tensor([1 if built is not None else 0], device=dev)
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                if int(flag.item()) == 0:
                    if want == "copy":
                        raise RuntimeError(f"--transport copy: a rank could not map its peers' buffers ({why})")
                    built, transport = None, "nccl"
            if transport == "nccl":
                built = build("nccl")
            self.feat_x, self.feat_g, px, pg = built
            self.feat_x.full.normal_(generator=gen); self.feat_g.full.normal_(generator=gen)
            if kind == "stages":
                self.pipes = {id(self.feat_x): px, id(self.feat_g): pg}
                self.stage_info = {"kind": "stages of source blocks, " + ("grouped send/receive" if transport == "nccl" else
                                                                         "peers' blocks pulled by the copy engines"),
                                   "transport": transport, "peer_groups": px.schedule,
                                   "pieces_per_group": px.pieces, "transfer_stages": len(px.transfers),
                                   "compute_stages": len(px.stage_plans)}
                if why and transport == "nccl":
                    self.stage_info["copy_transport_unavailable"] = why
            else:
                self.tiles = self.plan.auto_tiles(D) if ns.tiles == "auto" else int(ns.tiles)
        self.t_plan = time.time() - t0
        self.launches = 0
        self.gather_events = []

    def ev(self):
        return self.torch.cuda.Event(enable_timing=True)

    def one_pass(self, p, feat, out, timed_gather=False):
        if self.pipes and p is self.plan:       # transfers overlapped with the aggregation
            pipe = self.pipes[id(feat)]
            if self.kind == "pieces":
                full = self.full_x if feat is self.feat_x else self.full_g
                pipe.aggregate(full[self.r0:self.r1], self.deg_pad, self.mode, out)
            elif self.kind == "grid":
                full = self.full_x if feat is self.feat_x else self.full_g
                pipe.aggregate(full[self.r0:self.r1], self.deg_local, self.mode, out)
            else:
                pipe.aggregate(None, self.deg, self.mode, out)
            self.launches += pipe.launches
            return
        xs = feat.all_gather(None) if self.world > 1 else feat.full[:self.n]           # one collective, then the plan
        p.aggregate(xs, self.deg, self.mode, out=out, tiles=self.tiles,
                    gather_events=self.gather_events if timed_gather else None)
        self.launches += p.last_launch_count()

    def step(self, p, timed_gather=False):
        self.one_pass(p, self.feat_x, self.out_f, timed_gather)
        self.one_pass(p, self.feat_g, self.out_b, timed_gather)

    def _bracket(self, fn, steps, warmup):
        """`fn` x steps timed with events between barriers; max over ranks; -> (ms per call, wall t0, t1)"""
        torch = self.torch
        import torch.distributed as dist
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s, e = self.ev(), self.ev()
        w0 = time.time()
        s.record()
        for _ in range(steps):
            fn()
        e.record()
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        w1 = time.time()
        ms = torch.tensor([s.elapsed_time(e)], device=self.dev)
        if self.world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()) / steps, w0, w1

    def timed(self, p, steps, warmup, timed_gather=False):
        for _ in range(warmup):
            self.step(p)
        self.launches = 0
        self.gather_events = []
        return self._bracket(lambda: self.step(p, timed_gather), steps, 0)

    # ---- correctness: a sample of this rank's output rows recomputed on the host in fp64 ----
    def check(self, rows_wanted=48):
        torch = self.torch
        import torch.distributed as dist
        g, r0, r1 = self.g, self.r0, self.r1
        ip = g.indptr_dst
        lens = np.diff(ip[r0:r1 + 1])
        worst, count = 0.0, 0
        if r1 > r0:
            order = np.argsort(lens, kind="stable")
            nonempty = order[lens[order] > 0]
            rng = np.random.default_rng(77 + self.rank)
            pick = set(order[-3:].tolist()) | set(nonempty[:3].tolist()) | set(order[:1].tolist())
            pick |= set(rng.integers(0, r1 - r0, size=max(0, rows_wanted - len(pick))).tolist())
            deg64 = np.maximum(g.degrees_f32(), 1.0).astype(np.float64)
            for feat, out in ((self.feat_x, self.out_f), (self.feat_g, self.out_b)):
                if self.kind in ("pieces", "grid"):
                    fetch = (lambda ix, full=(self.full_x if feat is self.feat_x else self.full_g): full[ix])
                else:
                    fetch = feat.rows if hasattr(feat, "rows") else (lambda ix, full=feat.full[:self.n]: full[ix])
                for lr in sorted(pick):
                    v = r0 + lr
                    idx = g.indices_src[ip[v]:ip[v + 1]].astype(np.int64)
                    xs = fetch(torch.from_numpy(idx).to(self.dev)).cpu().numpy().astype(np.float64)
                    if self.mode == "gcn":
                        want = (xs / np.sqrt(deg64[idx])[:, None]).sum(0) / np.sqrt(deg64[v])
                    elif self.mode == "mean":
                        want = xs.sum(0) / deg64[v] if len(idx) else xs.sum(0)
                    else:
                        want = xs.sum(0)
                    got = out[lr].cpu().numpy().astype(np.float64)
                    tol = 1e-6 + 1e-5 * max(np.abs(want).max(), 1e-30)
                    err = np.abs(got - want).max() / tol if np.isfinite(got).all() else float("inf")
                    worst = max(worst, float(err))
                    count += 1
        t = torch.tensor([worst, float(count)], device=self.dev, dtype=torch.float64)
        if self.world > 1:
            w = t[:1].clone(); c = t[1:].clone()
            dist.all_reduce(w, op=dist.ReduceOp.MAX)
            dist.all_reduce(c, op=dist.ReduceOp.SUM)
            worst, count = float(w.item()), float(c.item())
        return {"rows": int(count), "max_scaled_err": worst, "ok": bool(worst <= 1.0),
                "what": "sampled output rows of every rank (3 longest, 3 shortest, random) of the forward and the "
                        "backward pass, recomputed from the CSR in fp64 on the host; error in units of the "
                        "tolerance 1e-6 + 1e-5 x row maximum"}

    # ---- the dominant kernel: phase B of this rank's block ------------------------------------
    def roofline(self, hbm_peak, peak_kind):
        torch = self.torch
        ge = self.gather_events
        chunks = 1
        if not ge and self.kind == "columns":      # phase B of every column chunk, bracketed by events
            f = self.feat_x
            chunks = len(f.cols)
            px = self.pipes[id(f)]
            for i in range(8):
                for k, (c0, c1) in enumerate(f.cols):
                    self.plan.aggregate(f.chunk_full(k), self.deg, self.mode, out=self.out_f[:, c0:c1], tiles=px.tiles[k],
                                        gather_events=ge if i >= 3 else None)
            torch.cuda.synchronize()
            per_pass = sum(px.tiles)
        elif not ge and self.kind == "pieces":     # phase B of every piece's plan
            px = self.pipes[id(self.feat_x)]
            for i in range(8):
                for k, sp in enumerate(px.stage_plans):
                    sp.aggregate(self.feat_x.full, self.deg_pad, "gcn_prescaled" if self.mode == "gcn" else self.mode,
                                 out=self.out_f, accumulate=k > 0, gather_events=ge if i >= 3 else None)
            torch.cuda.synchronize()
            per_pass = len(px.stage_plans)
        elif not ge and self.kind == "grid":       # the gather of every destination chunk
            px = self.pipes[id(self.feat_x)]
            for i in range(8):
                for q in range(self.grid.q):
                    e0, e1 = self.ev(), self.ev()
                    e0.record(); px.compute_chunk(q); e1.record()
                    if i >= 3:
                        ge.append((e0, e1))
            torch.cuda.synchronize()
            per_pass = self.grid.q
        elif not ge:           # staged run: time this rank's whole-block gather on its own
            xs = self.feat_x.full[:self.n]
            for i in range(8):
                e0, e1 = self.ev(), self.ev()
                e0.record(); self.plan.aggregate(xs, self.deg, self.mode, out=self.out_f, phases=2); e1.record()
                if i >= 3:
                    ge.append((e0, e1))
            torch.cuda.synchronize()
            per_pass = 1
        else:
            per_pass = max(self.tiles, 1)
        gms = float(np.sum([a.elapsed_time(b) for a, b in ge])) / (len(ge) / per_pass)
        info, rows, D = self.plan.info, self.r1 - self.r0, self.D
        if self.kind == "grid":                    # the rank's tile: partial rows of the whole destination group
            info = dict(info, gather_entries=sum(p.info["gather_entries"] for p in self.grid_plans), partial_entries=0)
            rows = self.grid.dst_rows
        # a pass over K column chunks reads the index entries (and degrees) once per chunk
        gather_bytes = 4.0 * D * (info["gather_entries"] + rows) + chunks * (4.0 * info["gather_entries"] + 4.0 * (rows + 1))
        if self.mode == "gcn":
            gather_bytes += chunks * 4.0 * (info["gather_entries"] - info["partial_entries"])
        achieved = gather_bytes / (gms / 1e3) / 1e9
        kernel = "gather_tiles_kernel + gather_rows_kernel (phase B)" if info["num_tiles"] else "gather_rows_kernel (phase B)"
        r = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
             "traffic": None, "kernel": kernel, "ms_per_launch": gms, "launches_per_pass": per_pass,
             "algorithmic_bytes_per_launch": gather_bytes, "peak_kind": f"{peak_kind} copy bandwidth",
             "note": "algorithmic bytes = (gathered rows + written rows) x 4D + 4 per index; rows gathered more than "
                     "once are re-read from L2, so achieved can exceed the DRAM peak: roofline_l2 is the bound then"}
        ns = self.ns
        if self.world == 1 and ns.scale == 1.0 and ns.part_size == WORKLOADS[ns.workload][1]:
            r["traffic"] = NCU_DRAM_BYTES_PER_PASS.get(f"{ns.workload}:D{D}:{self.mode}")
        return r

    # ---- N > 1: where a pass's time goes ------------------------------------------------------
    def breakdown(self, iters=10):
        if not self.pipes:
            return None
        px, pg = self.pipes[id(self.feat_x)], self.pipes[id(self.feat_g)]
        deg = self.deg_pad if self.kind == "pieces" else (self.deg_local if self.kind == "grid" else self.deg)
        t_all, _, _ = self._bracket(lambda: (self.one_pass(self.plan, self.feat_x, self.out_f),
                                             self.one_pass(self.plan, self.feat_g, self.out_b)), iters, 2)
        t_tr, _, _ = self._bracket(lambda: (px.transfer_only(), pg.transfer_only()), iters, 2)
        t_ag, _, _ = self._bracket(lambda: (px.aggregate_only(deg, self.mode, self.out_f),
                                            pg.aggregate_only(deg, self.mode, self.out_b)), iters, 2)
        recv = sum((b - a) for i, (a, b) in enumerate(self.blocks) if i != self.rank) * self.D * 4
        if self.kind == "columns":               # whole padded blocks travel
            recv = (self.world - 1) * self.feat_x.block * sum(st.shape[1] for st in self.feat_x._stores) * 4
        if self.kind == "pieces":
            recv = (self.world - 1) * self.feat_x.pieces * self.feat_x.pb * self.feat_x._store.shape[1] * 4
        if self.kind == "grid":
            recv = px.received_bytes_per_pass()
        return {"overlapped_ms": round(t_all, 4), "transfer_only_ms": round(t_tr, 4), "aggregate_only_ms": round(t_ag, 4),
                "received_bytes_per_pass": int(recv),
                "receive_GBs_transfer_only": round(2 * recv / (t_tr / 1e3) / 1e9, 1) if t_tr > 0 else None,
                "note": "per step (two passes), max over ranks: the transfers of the pipeline without its kernels, its "
                        "kernels without transfers, and both together"}

    # ---- end to end: pinned host buffers in and out, copies inside the timed region -----------
    def e2e(self, steps):
        torch = self.torch
        from artifact_b200.streaming import HostStreamedAggregator, device_host_node, pinned_near
        rows, D, n = self.r1 - self.r0, self.D, self.n
        columns = self.kind in ("columns", "pieces", "grid")
        # what a pass's upload lands in: this rank's rows of the feature buffer, or (column chunks) a
        # row-major staging block that the pass scatters into the chunk buffers first
        def landing(feat):
            return torch.empty((rows, D), device=self.dev) if columns else feat.local_view()
        land_x, land_g = landing(self.feat_x), landing(self.feat_g)
        up_rows = land_x.shape[0]
        di = self.dev.index if self.dev.index is not None else torch.cuda.current_device()
        h_x = pinned_near(di, (up_rows, D))
        h_g = pinned_near(di, (up_rows, D))
        if self.kind in ("pieces", "grid"):
            h_x.copy_(self.full_x[self.r0:self.r1]); h_g.copy_(self.full_g[self.r0:self.r1])
        elif columns:
            h_x.copy_(torch.cat([self.feat_x.chunk_local(k)[:rows] for k in range(len(self.feat_x.cols))], 1))
            h_g.copy_(torch.cat([self.feat_g.chunk_local(k)[:rows] for k in range(len(self.feat_g.cols))], 1))
        else:
            h_x.copy_(land_x); h_g.copy_(land_g)
        h_of = pinned_near(di, (rows, D))
        h_ob = pinned_near(di, (rows, D))
        # two device slots: slot 0 is the benchmark's x buffers, slot 1 its gradient buffers; the forward
        # pass of a step goes through one, the backward pass through the other, so that the upload of a
        # pass overlaps the kernels of the pass before it and the download those of the pass after it
        def run_pass(feat, land, out):
            if columns:
                deg = self.deg_pad if self.kind == "pieces" else (self.deg_local if self.kind == "grid" else self.deg)
                self.pipes[id(feat)].aggregate(land, deg, self.mode, out)
                self.launches += self.pipes[id(feat)].launches
            else:
                self.one_pass(self.plan, feat, out)
        slots = [(land_x, self.out_f, lambda: run_pass(self.feat_x, land_x, self.out_f)),
                 (land_g, self.out_b, lambda: run_pass(self.feat_g, land_g, self.out_b))]
        hs = HostStreamedAggregator(slots, self.dev)

        def e2e_step(aggregate=True):
            hs.submit(h_x, h_of, aggregate)
            hs.submit(h_g, h_ob, aggregate)

        def run(aggregate):
            def fn():
                e2e_step(aggregate)
            # the last step's downloads must have landed before the end event
            def fn_all():
                for _ in range(steps):
                    fn()
                hs.join()
            ms, _, _ = self._bracket(fn_all, 1, 1)
            return ms / steps

        ms_e2e = run(True)
        ms_copy = run(False)
        # restore the device-resident inputs the other measurements use
        if self.kind in ("pieces", "grid"):
            pass                                   # every pass scatters its rows into the buffer anyway
        elif columns:
            self.feat_x.set_local(h_x.to(self.dev)); self.feat_g.set_local(h_g.to(self.dev))
        else:
            self.feat_x.local_view().copy_(h_x); self.feat_g.local_view().copy_(h_g)
        torch.cuda.synchronize()
        return {"value": 2.0 * self.E / (ms_e2e / 1e3), "unit": "edges/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": 2 * n * D * 4, "d2h_bytes_per_step": 2 * n * D * 4,
                "copy_only_ms": ms_copy, "host_numa_node": device_host_node(di)[0],
                "note": "features and gradients copied from pinned host memory, both results copied back, every step "
                        "(artifact_b200.streaming.HostStreamedAggregator: uploads and downloads on their own streams, "
                        "double-buffered on the device, host buffers on the GPU's own socket where sysfs tells it); copy_only_ms is the same schedule without the kernels; bytes "
                        "are summed over the ranks; the graph plan stays resident like upstream's inputInfo tensors"}

    def release(self):
        # buffers that peers have mapped: every rank unmaps first, then the owners free
        mapped = [p for p in (self.pipes or {}).values() if getattr(p, "transport", "") == "copy"]
        if mapped:
            import torch.distributed as dist
            self.torch.cuda.synchronize()
            for p in mapped:
                p.close_windows() if hasattr(p, "close_windows") else p.windows.close()
            dist.barrier()
        for k in ("plan", "plain", "pipes", "feat_x", "feat_g", "full_x", "full_g", "out_f", "out_b", "deg", "L", "g",
                  "grid_plans"):
            setattr(self, k, None)
        self.torch.cuda.empty_cache()


# --------------------------------------------------------------------------------------------
# upstream's own CUDA kernels on the same GPU and graph (single GPU; skipped when not built)
# --------------------------------------------------------------------------------------------
def upstream_gpu(job, dims=(128, 256), warmup=5, iters=10):
    import importlib.util
    import torch
    so = glob.glob(os.path.join(ROOT, "oracle", "_ref", "ROF_ref*.so"))
    if not so:
        return {"skipped": "upstream CUDA extension not built (oracle/_ref/ROF_ref*.so absent)"}
    from artifact_b200 import ops
    spec = importlib.util.spec_from_file_location("ROF_ref", so[0])
    up = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(up)
    g, L, dev, n = job.g, job.L, job.dev, job.n
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)
    ci, pp, p2n = t(g.indices_src), t(L["part_pointers"]), t(L["part2Node"])
    v1 = [t(L[k]) for k in ("column_index", "part_pointers", "part2Node", "part_cache_flagindex",
                            "part_pointers_cache", "column_index_cache")]
    v2 = [t(L[k]) for k in ("uniqpart_column_index", "uniqpart_pointers", "part2Node_ptr", "part2Node_col")]
    G = len(L["part_pointers_cache"]) - 1
    if G < 1:
        return {"skipped": "no reuse group: upstream's ROF_v1 path exits the process then"}
    ps, wpb, f_in = int(L["part_size"]), 4, 64
    X = torch.randn((n, f_in), device=dev)
    res = {"method": f"{warmup} warm-up + {iters} timed calls, CUDA events around each call with a device "
                     "synchronise, X.W time subtracted (ROF_evaluation/cuda/small-main.py:360-390, 434-478); "
                     "forward aggregation of the whole graph", "f_in": f_in, "rows": []}

    def timed(fn):
        ms = []
        for i in range(warmup + iters):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(); fn(); e.record(); torch.cuda.synchronize()
            if i >= warmup:
                ms.append(s.elapsed_time(e))
        return float(np.mean(ms))

    for D in dims:
        W = torch.randn((f_in, D), device=dev)
        cache = torch.zeros((G, D + 1), device=dev)
        dw = min(D, 32)
        mm = timed(lambda: torch.mm(X, W))
        row = {"D": D, "mm_ms": round(mm, 4)}
        for name, mod in (("upstream", up), ("new", ops)):
            row[name] = {
                "GNNA": round(timed(lambda: mod.GNNA_forward(X, W, ci, job.deg, pp, p2n, ps, dw, wpb)) - mm, 4),
                "ROF_v1": round(timed(lambda: mod.reuse_forward_v1(X, W, v1[0], job.deg, v1[1], v1[2], ps, dw, wpb, cache,
                                                                   v1[3], v1[4], v1[5])) - mm, 4),
                "ROF_v2": round(timed(lambda: mod.reuse_forward_v2(X, W, v2[0], job.deg, v2[1], v2[2], v2[3], ps, dw,
                                                                   wpb)) - mm, 4),
            }
        row["speedup"] = {k: round(row["upstream"][k] / max(row["new"][k], 1e-6), 1) for k in row["new"]}
        res["rows"].append(row)
        del W, cache
    ops.clear_plan_cache()
    return res


def side_config(name, args, rank, world, dev, steps):
    """ms per step and check of another benchmark configuration, with the same machinery"""
    d, ps, mode = WORKLOADS[name]
    ns = argparse.Namespace(**vars(args))
    ns.workload, ns.dim, ns.part_size, ns.mode, ns.tiles, ns.schedule, ns.pieces = name, d, ps, mode, "auto", "", 0
    job = Job(ns, rank, world, dev, want_plain=(world == 1))
    try:
        ms, _, _ = job.timed(job.plan, steps, 3)
        out = {"workload": workload_config(ns, job.g, job.ratios)["workload"], "ms_per_step": round(ms, 4),
               "edges_per_s": 2.0 * job.E / (ms / 1e3), "check": job.check(24), "n_gpus": world,
               "tile_kernel": {"tiles": job.plan.info["num_tiles"],
                               "entries_from_shared_memory": job.plan.info["tile_shared_entries"]}}
        if job.plain is not None:
            mp_, _, _ = job.timed(job.plain, max(3, steps // 2), 3)
            out["plain_ms_per_step"] = round(mp_, 4)
            out["reuse_speedup"] = round(mp_ / ms, 4)
        bd = job.breakdown(5)
        if bd:
            out["breakdown"] = bd
            out["stages"] = job.stage_info
        out["setup_s"] = {"graph": round(job.t_graph, 2), "reuse_search": round(job.t_search, 2),
                          "plans": round(job.t_plan, 2)}
        return out
    finally:
        job.release()


# --------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--dim", type=int, default=0)
    ap.add_argument("--part-size", type=int, default=0)
    ap.add_argument("--mode", default="")
    ap.add_argument("--scale", type=float, default=1.0, help="shrink the graph (tests / profiling only)")
    ap.add_argument("--no-pipeline", dest="pipeline", action="store_false",
                    help="N > 1: one all-gather, then the aggregation (no overlap)")
    ap.add_argument("--transport", default="auto", choices=["auto", "nccl", "copy"],
                    help="N > 1, stage pipeline: copy engines pulling from the peers' buffers (auto: with NCCL send/receive "
                         "as the fall-back where the buffers cannot be mapped), or grouped NCCL send/receive")
    ap.add_argument("--grid-cols", type=int, default=0, help="N > 1, grid pipeline: columns of the grid (0: by world size)")
    ap.add_argument("--pipeline-kind", default="auto", choices=["auto", "pieces", "columns", "stages", "grid"],
                    help="N > 1: exchange the features piece-major (one all-gather per L2-sized piece of every block), "
                         "in column chunks (one all-gather each) or in stages of source blocks (grouped send/receive)")
    ap.add_argument("--own-first", type=int, default=0, choices=[0, 1],
                    help="N > 1, piece-major pipeline: a first stage over the rank's own rows while piece 0 travels")
    ap.add_argument("--chunks", type=int, default=0, help="N > 1: column chunks of the column pipeline (0: by width), destination chunks of the grid (0: 4)")
    ap.add_argument("--schedule", default="", help="N > 1 pipeline stages as ring offsets, e.g. '0|1,2,3|4,5,6,7'")
    ap.add_argument("--pieces", type=int, default=0, help="N > 1: pieces each peer group's transfer is cut into (0: by size)")
    ap.add_argument("--tiles", default="auto", help="source tiles per pass on one GPU: auto or an integer")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the other benchmark configurations (c4, c5, c3)")
    ap.add_argument("--no-upstream", action="store_true", help="skip timing upstream's own CUDA kernels")
    ap.add_argument("--only-kernel", action="store_true", help="only the timed steps (profiling)")
    args = ap.parse_args()
    d_dim, d_ps, d_mode = WORKLOADS[args.workload]
    args.dim = args.dim or d_dim
    args.part_size = args.part_size or d_ps
    args.mode = args.mode or d_mode
    args.warmup = max(args.warmup, 3)
    if args.only_kernel:
        args.no_sweep = args.no_cpu = args.no_configs = args.no_upstream = True

    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from artifact_b200.plan import probe_read_gbs

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the aggregation path has no CPU fallback")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    hbm_peak, peak_kind = load_peaks()

    job = Job(args, rank, world, dev, want_plain=(world == 1 and not args.only_kernel))
    E, D, mode, n = job.E, job.D, job.mode, job.n

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    ms_step, w0, w1 = job.timed(job.plan, args.steps, args.warmup, timed_gather=True)
    clocks = sampler.stop(w0, w1) if sampler else None
    n_launch = job.launches
    value = 2.0 * E / (ms_step / 1e3)
    check = job.check()
    roofline = job.roofline(hbm_peak, peak_kind)

    extra = {}
    if not args.only_kernel:
        # L2 -> SM read bandwidth of a plain streaming kernel over a 64 MB buffer: the roof of the gather when
        # the rows it re-reads are L2-resident (they are: DRAM traffic is a few % of the algorithmic bytes)
        l2_peak = probe_read_gbs(64 << 20, dev)
        extra["roofline_l2"] = {"bound": "l2", "achieved": roofline["achieved"], "peak": l2_peak, "unit": "GB/s",
                                "frac": roofline["achieved"] / l2_peak if l2_peak else None,
                                "peak_kind": "measured in this run: 128-bit L1-bypassing reads of a 64 MB buffer "
                                             "(rof_probe_read); the gather also hits L1, so it can read above 1",
                                "hbm_read_probe_GBs": probe_read_gbs(4 << 30, dev, repeats=2, iters=2)}
    if job.plain is not None:
        ms_plain, _, _ = job.timed(job.plain, max(3, args.steps // 2), 3)
        extra["plain"] = {"ms_per_step": ms_plain, "edges_per_s": 2.0 * E / (ms_plain / 1e3),
                          "algorithmic_GBs": 2 * job.plain.algorithmic_bytes(D, mode) / ms_plain / 1e6}
        extra["reuse"] = {"ms_per_step": ms_step, "edges_per_s": value,
                          "algorithmic_GBs": 2 * job.plan.algorithmic_bytes(D, mode) / ms_step / 1e6}
        extra["reuse_speedup"] = ms_plain / ms_step
    if world > 1 and not args.only_kernel:
        extra["breakdown"] = job.breakdown()
        if job.pipes:
            extra["stages"] = job.stage_info

    e2e = None if args.only_kernel else job.e2e(max(3, min(args.steps, 10)))

    # ---- width / mode sweep (single GPU only; informational) -----------------------------------
    if world == 1 and not args.no_sweep:
        from artifact_b200.plan import empty_padded
        sweep = []
        for d in (7, 32, 47, 64, 100, 128, 256, 602):
            xs = empty_padded(n, d, dev); xs.normal_()
            o = torch.empty((n, d), device=dev)
            for m in ("sum", "mean", "gcn"):
                row = {"D": d, "mode": m}
                for nm, p in (("reuse", job.plan), ("plain", job.plain)):
                    t = p.auto_tiles(d)
                    row[nm + "_tiles"] = t
                    for _ in range(3):
                        p.aggregate(xs, job.deg, m, out=o, tiles=t)
                    s, e = job.ev(), job.ev()
                    s.record()
                    for _ in range(5):
                        p.aggregate(xs, job.deg, m, out=o, tiles=t)
                    e.record(); torch.cuda.synchronize()
                    ms = s.elapsed_time(e) / 5
                    row[nm] = {"ms": round(ms, 4), "gedges_per_s": round(E / ms / 1e6, 3),
                               "algorithmic_GBs": round(p.algorithmic_bytes(d, m) / ms / 1e6, 1)}
                sweep.append(row)
            del xs, o
        extra["sweep_forward_pass"] = sweep
        extra["sweep_note"] = "feature rows padded to a multiple of 4 floats (what the drop-in entry points allocate)"

    # ---- one GCN layer through the drop-in layer API (informational: "GCN layer ms") -----------
    if world == 1 and not args.no_sweep:
        from artifact_b200.models import ROF_inputInfo
        from artifact_b200.reuse_conv import ROF_GCNConv
        i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32))
        f_in = {"c2": 602, "c3": 128, "c4": 100, "c5": 64}[args.workload]
        t = lambda k: i32(job.L[k]).to(dev)
        info = ROF_inputInfo(None, None, job.deg, None, None, args.part_size, 4, None, None, None,
                             t("uniqpart_column_index"), t("uniqpart_pointers"), t("part2Node_ptr"), t("part2Node_col"))
        layer = ROF_GCNConv(f_in, D, add_self_loops=False, kernel_type="ROF_v2").to(dev)
        xin = torch.randn((n, f_in), device=dev, requires_grad=True)
        gout = job.feat_g.full[:n]

        def layer_step():
            y = layer(xin, info)
            y.backward(gout)
            xin.grad = None; layer.zero_grad(set_to_none=True)

        for _ in range(3):
            layer_step()
        s, e = job.ev(), job.ev()
        s.record()
        for _ in range(5):
            layer_step()
        e.record(); torch.cuda.synchronize()
        ms_layer = s.elapsed_time(e) / 5
        with torch.no_grad():
            w_ = layer.weight.detach()
            s.record()
            for _ in range(5):
                torch.mm(xin, w_); torch.mm(gout, w_.t()); torch.mm(xin.t(), gout)
            e.record(); torch.cuda.synchronize()
        ms_mm = s.elapsed_time(e) / 5
        extra["gcn_layer"] = {"shape": [n, f_in, D], "kernel_type": "ROF_v2", "fwd_bwd_ms": round(ms_layer, 3),
                              "of_which_dense_mm_ms": round(ms_mm, 3),
                              "note": "ROF_GCNConv forward+backward; the three fp32 GEMMs (X.W, dX, dW) stay on cuBLAS"}
        del info, layer, xin
        from artifact_b200 import ops
        ops.clear_plan_cache()

    if world == 1 and not args.no_upstream and args.workload == "c2" and args.scale == 1.0:
        try:
            extra["upstream_gpu"] = upstream_gpu(job)
        except Exception as ex:                          # never lose the headline to the comparison
            extra["upstream_gpu"] = {"skipped": f"{type(ex).__name__}: {ex}"[:300]}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cb = cpu_plain(job.g, D, mode, seconds_budget=20.0, steps=3, warmup=1)
        cpu = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
        try:
            extra["cpu_torch_sparse"] = cpu_torch_sparse(job.g, D)
        except Exception as ex:
            extra["cpu_torch_sparse"] = {"skipped": f"{type(ex).__name__}: {ex}"[:300]}

    line = {
        "metric": "aggregation edges/s", "value": value, "unit": "edges/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(args, job.g, job.ratios),
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": n_launch, "clocks": clocks,
        "check": check,
        "setup_s": {"graph": round(job.t_graph, 2), "reuse_search": round(job.t_search, 2), "plans": round(job.t_plan, 2)},
        "shard": {"rows": job.r1 - job.r0, "edges_rank0": int(job.g.indptr_dst[job.r1] - job.g.indptr_dst[job.r0])},
    }
    line.update(extra)
    ok = check["ok"]
    job.release()

    # ---- the other benchmark configurations, same machinery, so that the record carries them ----
    if not args.no_configs:
        configs = {}
        names = [w for w in ("c4", "c5") if w != args.workload] + (["c3"] if world == 1 and args.workload != "c3" else [])
        for name in names:
            try:
                configs[name] = side_config(name, args, rank, world, dev, steps=max(3, min(args.steps, 10)))
                ok = ok and configs[name]["check"]["ok"]
            except Exception as ex:
                if world > 1:
                    raise                                # ranks must not diverge around collectives
                configs[name] = {"skipped": f"{type(ex).__name__}: {ex}"[:300]}
        line["configs"] = configs

    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not ok:
        sys.stderr.write("bench.py: the output check failed (see \"check\" in the JSON line)\n")
        sys.exit(3)


if __name__ == "__main__":
    main()
