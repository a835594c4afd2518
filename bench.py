#!/usr/bin/env python
"""Benchmark of the reuse aggregation hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c4|c5] [--dim D]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...      # CPU plain aggregation on the host cores

One *step* is one forward plus one backward aggregation pass (the backward applies the same
operator to the incoming gradient, reuse_conv.py:76-92) of fp32 features of width D over the
seeded synthetic graph of the workload, through the reuse plan built from the ROF_v2 layout.
`value` is edges/s with the ORIGINAL edge count (reuse shows up as more edges per second),
inputs resident in HBM; `e2e` is the same step through the public API with pinned-host inputs
and outputs, copies inside the timed region.  With N > 1 the destination rows are cut into N
equal blocks; every pass moves the feature blocks between the ranks over NCCL (staged
send/receive groups overlapped with the per-stage aggregation, or one all-gather with
--no-pipeline) and the same total work is divided (strong scaling).  On one GPU a feature matrix
larger than L2 is walked in source tiles (--tiles).  Prints ONE JSON line on rank 0.
"""
import argparse
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
    # name: (config function key, default feature width, part_size, mode)
    "c2": ("c2", 256, 2, "sum"),
    "c4": ("c4", 256, 2, "gcn"),
    "c5": ("c5", 64, 2, "sum"),
}


# dram__bytes_read.sum + dram__bytes_write.sum of one phase-B launch, from the ncu captures
# summarised in profiles/gather_rows_<workload>_d<D>_<mode>.md (captured once per kernel change)
NCU_DRAM_BYTES_PER_LAUNCH = {
    "c2:D256:sum": 5.13e9,     # one pass = 4 source tiles x 1.28 GB (untiled: 25.03 GB)
    "c2:D64:sum": 1.44e9,
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
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "200"],
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
    return graphs.CONFIGS[WORKLOADS[name][0]](scale)


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


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl, dim, ps, mode = args.workload, args.dim, args.part_size, args.mode
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


def prepare_workload(args, rank, world):
    """-> (graph, layouts needed for the ROF_v2 plan, seconds for graph, seconds for search)"""
    from artifact_b200 import graphs, search
    cache_dir = os.environ.get("ROF_CACHE_DIR", "/tmp/rof_b200_cache")
    path = os.path.join(cache_dir, f"{args.workload}_scale{args.scale}_ps{args.part_size}.npz")
    def compute():
        from artifact_b200 import _native
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
        L = {k: z[k] for k in _V2_KEYS}
        L["part_size"] = args.part_size
        L["original_column_index"] = g.indices_src
        return g, L

    # rank 0 makes sure the cache file exists (loading it, or computing and saving); every rank
    # then passes the same barrier, and the other ranks load the file
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
                         indptr_dst=g.indptr_dst, indices_src=g.indices_src, **{k: L[k] for k in _V2_KEYS})
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


def workload_config(args, g, ratios):
    c = {"workload": f"{args.workload}: seeded synthetic graph N={g.num_nodes} E={g.num_edges}, fp32 features "
                     f"D={args.dim}, {args.mode} aggregation, forward+backward pass per step",
         "part_size": args.part_size, "layout": "ROF_v2", "scale": args.scale, "source_tiles": args.tiles,
         "l2": "feature matrix and index arrays together exceed L2 (126 MB); no flush between iterations",
         "parallelism": (f"row-block x{args.gpus}, " + ("all-gather rounds overlapped with staged aggregation"
                                                        if args.pipeline else "all-gather then aggregate"))
         if args.gpus > 1 else "single GPU"}
    if ratios is not None:
        c["reuse"] = ratios
    return c


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
    ap.add_argument("--schedule", default="", help="N > 1 pipeline stages as ring offsets, e.g. '0|1,2,3|4,5,6,7'")
    ap.add_argument("--tiles", default="auto", help="source tiles per pass on one GPU: auto or an integer")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--only-kernel", action="store_true", help="skip sweep, CPU baseline and e2e (profiling)")
    args = ap.parse_args()
    _, d_dim, d_ps, d_mode = WORKLOADS[args.workload]
    args.dim = args.dim or d_dim
    args.part_size = args.part_size or d_ps
    args.mode = args.mode or d_mode
    args.warmup = max(args.warmup, 3)
    if args.only_kernel:
        args.no_sweep = args.no_cpu = True

    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from artifact_b200 import search
    from artifact_b200.plan import AggregationPlan

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

    # ---- workload: graph -> reuse search -> plans ------------------------------------------
    # Everything is seeded, so every rank could compute it; to keep the host cores for one
    # search, rank 0 computes and leaves the arrays in a cache directory the other ranks (and
    # the next invocation on the same box) load.
    g, L, t_graph, t_search = prepare_workload(args, rank, world)
    n, E, D, mode = g.num_nodes, g.num_edges, args.dim, args.mode
    ratios = search.reuse_ratios(L)
    blk = (n + world - 1) // world
    n_pad = blk * world
    r0, r1 = min(rank * blk, n), min((rank + 1) * blk, n)
    t0 = time.time()
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32))
    v2 = [i32(L[k]) for k in ("uniqpart_column_index", "uniqpart_pointers", "part2Node_ptr", "part2Node_col")]
    plan = AggregationPlan.from_v2(n, *v2, rows=(r0, r1), device=dev)
    plain = AggregationPlan.from_parts(n, i32(g.indices_src), i32(g.indptr_dst), i32(np.arange(n)), rows=(r0, r1),
                                       device=dev)
    t_plan = time.time() - t0
    del v2
    my_edges = int(g.indptr_dst[r1] - g.indptr_dst[r0])
    deg = torch.from_numpy(np.maximum(g.degrees_f32(), 1.0)).to(dev)

    from artifact_b200.sharding import PipelinedAggregator, ShardedFeatures
    gen = torch.Generator(device=dev); gen.manual_seed(1234)
    feat_x = ShardedFeatures(n, D, rank, world, dev)
    feat_g = ShardedFeatures(n, D, rank, world, dev)
    feat_x.full.normal_(generator=gen); feat_g.full.normal_(generator=gen)
    # this rank's block of features / gradients lives inside the full buffers (in-place all-gather)
    x_loc = feat_x.local_view()
    g_loc = feat_g.local_view()
    out_f = torch.empty((r1 - r0, D), device=dev)
    out_b = torch.empty((r1 - r0, D), device=dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)
    gather_events = []
    launches = [0]
    if world == 1 or not args.pipeline:
        tiles = plan.auto_tiles(D) if args.tiles == "auto" else int(args.tiles)
    else:
        tiles = 1                 # the pipeline's stages are already source-blocked
    pipes = {}
    if world > 1 and args.pipeline:
        sched = [[int(k) for k in st.split(",")] for st in args.schedule.split("|")] if args.schedule else None
        px = PipelinedAggregator(plan, feat_x, schedule=sched)
        pipes = {id(feat_x): px,
                 id(feat_g): PipelinedAggregator(plan, feat_g, stage_plans=px.stage_plans, schedule=sched)}

    def one_pass(p, src_loc, feat, out, timed_gather=False):
        if pipes and p is plan:       # all-gather rounds overlapped with the per-stage aggregation
            pipe = pipes[id(feat)]
            pipe.aggregate(None, deg, mode, out)
            launches[0] += pipe.launches
            return
        xs = feat.all_gather(None) if world > 1 else feat.full[:n]
        p.aggregate(xs, deg, mode, out=out, tiles=tiles, gather_events=gather_events if timed_gather else None)
        launches[0] += p.last_launch_count()

    def step(p, timed_gather=False):
        one_pass(p, x_loc, feat_x, out_f, timed_gather)
        one_pass(p, g_loc, feat_g, out_b, timed_gather)

    def timed(p, steps, warmup, timed_gather=False):
        for _ in range(warmup):
            step(p)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        launches[0] = 0
        s, e = ev(), ev()
        w0 = time.time()
        s.record()
        for _ in range(steps):
            step(p, timed_gather)
        e.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        w1 = time.time()
        ms = torch.tensor([s.elapsed_time(e)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()) / steps, w0, w1

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    ms_step, w0, w1 = timed(plan, args.steps, args.warmup, timed_gather=True)
    clocks = sampler.stop(w0, w1) if sampler else None
    n_launch = launches[0]
    value = 2.0 * E / (ms_step / 1e3)

    # dominant kernel: the phase-B gather of this rank's block, timed by events inside the steps
    if not gather_events:             # pipelined run: time this rank's whole-block gather kernel on its own
        xs = feat_x.full[:n]
        for i in range(8):
            e0, e1 = ev(), ev()
            e0.record(); plan.aggregate(xs, deg, mode, out=out_f, phases=2); e1.record()
            if i >= 3:
                gather_events.append((e0, e1))
        torch.cuda.synchronize()
    # one pass = `tiles` phase-B launches (one per source tile); report the pass as one unit
    per_pass = max(tiles, 1) if not pipes else 1
    gms = float(np.sum([a.elapsed_time(b) for a, b in gather_events])) / (len(gather_events) / per_pass)
    info = plan.info
    row_b = 4.0 * D
    gather_bytes = row_b * (info["gather_entries"] + (r1 - r0)) + 4.0 * info["gather_entries"] + 4.0 * (r1 - r0 + 1)
    if mode == "gcn":
        gather_bytes += 4.0 * (info["gather_entries"] - info["partial_entries"])
    achieved = gather_bytes / (gms / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                "traffic": None, "kernel": "gather_rows_kernel (phase B)", "ms_per_launch": gms,
                "launches_per_pass": per_pass,
                "algorithmic_bytes_per_launch": gather_bytes, "peak_kind": f"{peak_kind} copy bandwidth",
                "note": "algorithmic bytes = (gathered rows + written rows) x 4D + 4 per index; hub rows are "
                        "re-read from L2, so achieved can exceed the DRAM peak; see profiles/ for DRAM traffic"}
    if world == 1 and args.scale == 1.0 and args.part_size == WORKLOADS[args.workload][2]:
        roofline["traffic"] = NCU_DRAM_BYTES_PER_LAUNCH.get(f"{args.workload}:D{D}:{mode}")

    extra = {}
    if world == 1 and not args.only_kernel:
        ms_plain, _, _ = timed(plain, max(3, args.steps // 2), 3)
        extra["plain"] = {"ms_per_step": ms_plain, "edges_per_s": 2.0 * E / (ms_plain / 1e3),
                          "algorithmic_GBs": 2 * plain.algorithmic_bytes(D, mode) / ms_plain / 1e6}
        extra["reuse"] = {"ms_per_step": ms_step, "edges_per_s": value,
                          "algorithmic_GBs": 2 * plan.algorithmic_bytes(D, mode) / ms_step / 1e6}

    # ---- end to end through the public API with host buffers -----------------------------------
    def measure_e2e():
        h_x = torch.empty((blk, D), pin_memory=True); h_x.copy_(x_loc)
        h_g = torch.empty((blk, D), pin_memory=True); h_g.copy_(g_loc)
        h_of = torch.empty((r1 - r0, D), pin_memory=True)
        h_ob = torch.empty((r1 - r0, D), pin_memory=True)

        # the caller's own streams around the API: uploads on one copy stream (the gradient's upload
        # overlaps the forward pass), downloads on another (the forward result's download overlaps
        # the backward pass); the aggregation itself runs on the current stream
        cur = torch.cuda.current_stream(dev)
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        up_x, up_g, done_f, done_b, down = (torch.cuda.Event() for _ in range(5))
        done_f.record(cur); done_b.record(cur)

        def e2e_step():
            with torch.cuda.stream(s_in):
                s_in.wait_event(done_f)                    # previous forward pass has read x
                x_loc.copy_(h_x, non_blocking=True); up_x.record(s_in)
                s_in.wait_event(done_b)
                g_loc.copy_(h_g, non_blocking=True); up_g.record(s_in)
            cur.wait_event(up_x)
            one_pass(plan, x_loc, feat_x, out_f); done_f.record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done_f)
                h_of.copy_(out_f, non_blocking=True)
            cur.wait_event(up_g)
            one_pass(plan, g_loc, feat_g, out_b); done_b.record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done_b)
                h_ob.copy_(out_b, non_blocking=True); down.record(s_out)
            cur.wait_event(down)                           # the step ends when both results are on the host

        e2e_steps = max(3, min(args.steps, 10))
        for _ in range(3):
            e2e_step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        s, e = ev(), ev()
        s.record()
        for _ in range(e2e_steps):
            e2e_step()
        e.record()
        torch.cuda.synchronize()
        ms_e2e = torch.tensor([s.elapsed_time(e) / e2e_steps], device=dev)
        if world > 1:
            dist.all_reduce(ms_e2e, op=dist.ReduceOp.MAX)
        ms_e2e = float(ms_e2e.item())
        e2e = {"value": 2.0 * E / (ms_e2e / 1e3), "unit": "edges/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": 2 * blk * D * 4 * world, "d2h_bytes_per_step": 2 * n * D * 4,
               "note": "features and gradients copied from pinned host memory, both results copied back, every step; "
                       "the graph plan stays resident like upstream's inputInfo tensors"}
        return e2e

    e2e = None if args.only_kernel else measure_e2e()

    # ---- width / mode sweep (single GPU only; informational) -----------------------------------
    if world == 1 and not args.no_sweep:
        sweep = []
        for d in (32, 64, 128, 256, 602):
            xs = torch.randn((n, d), device=dev)
            o = torch.empty((n, d), device=dev)
            for m in ("sum", "mean"):
                row = {"D": d, "mode": m}
                for nm, p in (("reuse", plan), ("plain", plain)):
                    t = p.auto_tiles(d)
                    row[nm + "_tiles"] = t
                    for _ in range(3):
                        p.aggregate(xs, deg, m, out=o, tiles=t)
                    s, e = ev(), ev()
                    s.record()
                    for _ in range(5):
                        p.aggregate(xs, deg, m, out=o, tiles=t)
                    e.record(); torch.cuda.synchronize()
                    ms = s.elapsed_time(e) / 5
                    row[nm] = {"ms": round(ms, 4), "gedges_per_s": round(E / ms / 1e6, 3),
                               "algorithmic_GBs": round(p.algorithmic_bytes(d, m) / ms / 1e6, 1)}
                sweep.append(row)
            del xs, o
        extra["sweep_forward_pass"] = sweep

    # ---- one GCN layer through the drop-in layer API (informational: "GCN layer ms") -----------
    if world == 1 and not args.no_sweep:
        from artifact_b200.models import ROF_inputInfo
        from artifact_b200.reuse_conv import ROF_GCNConv
        f_in = {"c2": 602, "c4": 100, "c5": 64}[args.workload]
        t = lambda k: i32(L[k]).to(dev)
        info = ROF_inputInfo(None, None, deg, None, None, args.part_size, 4, None, None, None,
                             t("uniqpart_column_index"), t("uniqpart_pointers"), t("part2Node_ptr"), t("part2Node_col"))
        layer = ROF_GCNConv(f_in, D, add_self_loops=False, kernel_type="ROF_v2").to(dev)
        xin = torch.randn((n, f_in), device=dev, requires_grad=True)

        def layer_step():
            y = layer(xin, info)
            y.backward(feat_g.full[:n])
            xin.grad = None; layer.zero_grad(set_to_none=True)

        for _ in range(3):
            layer_step()
        s, e = ev(), ev()
        s.record()
        for _ in range(5):
            layer_step()
        e.record(); torch.cuda.synchronize()
        ms_layer = s.elapsed_time(e) / 5
        with torch.no_grad():
            w_ = layer.weight.detach()
            s.record()
            for _ in range(5):
                tmp = torch.mm(xin, w_); torch.mm(feat_g.full[:n], w_.t()); torch.mm(xin.t(), feat_g.full[:n])
            e.record(); torch.cuda.synchronize()
        ms_mm = s.elapsed_time(e) / 5
        extra["gcn_layer"] = {"shape": [n, f_in, D], "kernel_type": "ROF_v2", "fwd_bwd_ms": round(ms_layer, 3),
                              "of_which_dense_mm_ms": round(ms_mm, 3),
                              "note": "ROF_GCNConv forward+backward; the three fp32 GEMMs (X.W, dX, dW) stay on cuBLAS"}
        del info, layer, xin

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu:
            cb = cpu_plain(g, D, mode, seconds_budget=20.0, steps=3, warmup=1)
            cpu = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
        line = {
            "metric": "aggregation edges/s", "value": value, "unit": "edges/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(args, g, ratios),
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": n_launch, "clocks": clocks,
            "setup_s": {"graph": round(t_graph, 2), "reuse_search": round(t_search, 2), "plans": round(t_plan, 2)},
            "shard": {"rows": r1 - r0, "edges_rank0": my_edges},
        }
        line.update(extra)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
