"""AggregationPlan: Python handle of a `rof_plan` (include/rof_b200.h).

A plan is built once per graph from upstream's index tensors (the fields of `ROF_inputInfo`,
ROF_evaluation/ROF_main.py:164-174) and then drives every aggregation pass.  torch is used
only to allocate device memory and to name the current stream.
"""
import ctypes
import os

import numpy as np
import torch

from . import _native

MODES = {"gcn": 0, "sum": 1, "mean": 2, "gcn_prescaled": 3}
SCALE_OPS = {"copy": 0, "rsqrt": 1, "reciprocal": 2}
_PHASE_NAMES = {1: "rof:partials", 2: "rof:gather", 4: "rof:segment_reduce", 7: "rof:aggregate"}
# ROF_NVTX=1 brackets every C-ABI aggregation call with an NVTX range (visible to ncu --nvtx)
_NVTX = os.environ.get("ROF_NVTX", "0") not in ("", "0")
ON_HOST, ON_DEVICE = 0, 1


def _as_index(a):
    """-> (keepalive, pointer, length, where) for a torch tensor or numpy array of int32."""
    if isinstance(a, torch.Tensor):
        if a.dtype != torch.int32:
            raise TypeError(f"index tensors must be int32 (upstream casts them at ROF_main.py:143-161), got {a.dtype}")
        if not a.is_contiguous():
            raise RuntimeError("index tensor must be contiguous")
        return a, ctypes.c_void_p(a.data_ptr()), a.numel(), (ON_DEVICE if a.is_cuda else ON_HOST)
    a = np.ascontiguousarray(a)
    if a.dtype != np.int32:
        if a.dtype in (np.uint32, np.int64) and (a.size == 0 or (a.min() >= 0 and a.max() < 2 ** 31)):
            a = a.astype(np.int32)
        else:
            raise TypeError(f"index arrays must be int32, got {a.dtype}")
    return a, ctypes.c_void_p(a.ctypes.data), a.size, ON_HOST


def _same_place(parts):
    wh = {w for (_, _, _, w) in parts}
    if len(wh) != 1:
        raise RuntimeError("all index tensors of one layout must live in the same place (all host or all device)")
    return wh.pop()


def padded_width(dim):
    """leading dimension (floats) that keeps every row of a [*, dim] fp32 matrix 16-byte aligned"""
    return (int(dim) + 3) // 4 * 4


def empty_padded(rows, dim, device):
    """A [rows, dim] fp32 view whose row stride is padded to a multiple of 4 floats, so that the
    gather kernels can use 128-bit loads (and the shared-memory ring) whatever `dim` is."""
    return torch.empty((rows, padded_width(dim)), dtype=torch.float32, device=device)[:, :dim]


def scale_rows(x, degrees, op="rsqrt", out=None):
    """rof_scale_rows(): out[r] = f(degrees[r]) * x[r] (f: 'copy', 'rsqrt', 'reciprocal').  With
    out=None the result goes to a new padded buffer (see empty_padded); out may be x (in place)."""
    if not x.is_cuda or x.dtype != torch.float32 or x.dim() != 2 or (x.stride(1) != 1 and x.size(1) > 1):
        raise RuntimeError("x must be a 2-D float32 CUDA tensor with unit column stride")
    rows, dim = x.shape
    if out is None:
        out = empty_padded(rows, dim, x.device)
    elif (tuple(out.shape) != (rows, dim) or out.dtype != torch.float32 or out.device != x.device
          or (out.stride(1) != 1 and dim > 1)):
        raise RuntimeError("out must be a float32 tensor like x with unit column stride")
    deg_ptr = None
    if SCALE_OPS[op] != 0:
        if (degrees is None or degrees.device != x.device or degrees.dtype != torch.float32
                or not degrees.is_contiguous() or degrees.numel() < rows):
            raise RuntimeError("degrees must be a contiguous float32 tensor on x's device with one entry per row")
        deg_ptr = ctypes.c_void_p(degrees.data_ptr())
    with _device_guard(x.device):
        _native.check(_native.cuda().rof_scale_rows(
            ctypes.c_void_p(x.data_ptr()), x.stride(0) if rows > 1 else dim, dim, deg_ptr, SCALE_OPS[op],
            ctypes.c_void_p(out.data_ptr()), out.stride(0) if rows > 1 else padded_width(dim), rows,
            ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)))
    return out


def probe_read_gbs(nbytes, device, repeats=None, iters=5):
    """Read bandwidth in GB/s of a coalesced 128-bit streaming kernel over a `nbytes` buffer
    (rof_probe_read): L2 -> SM when the buffer fits L2, HBM when it is much larger."""
    buf = torch.zeros(nbytes // 4, dtype=torch.float32, device=device)
    sink = torch.zeros(1, dtype=torch.float32, device=device)
    repeats = repeats or max(1, int(4e9 // nbytes))
    lib = _native.cuda()
    best = 0.0
    with _device_guard(device):
        stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        for i in range(iters + 1):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _native.check(lib.rof_probe_read(ctypes.c_void_p(buf.data_ptr()), nbytes, repeats,
                                             ctypes.c_void_p(sink.data_ptr()), stream))
            e1.record()
            torch.cuda.synchronize(device)
            if i:                                   # the first run warms the cache
                best = max(best, nbytes * repeats / (e0.elapsed_time(e1) / 1e3) / 1e9)
    return best


class AggregationPlan:
    def __init__(self, handle, layout, device, keep):
        self._h = handle
        self.layout = layout
        self.device = device
        self._keep = keep          # index tensors this plan was built from (pins their addresses)
        self._workspace = None
        self._tiled = {}
        self.launches = 0      # kernel launches of the last aggregate() on this plan
        info = _native.PlanInfo()
        _native.check(_native.cuda().rof_plan_get_info(self._h, ctypes.byref(info)))
        self.info = {n: int(getattr(info, n)) for n, _ in _native.PlanInfo._fields_}

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                _native.cuda().rof_plan_destroy(h)
            except Exception:
                pass

    # -- constructors ------------------------------------------------------------------
    @staticmethod
    def _stream(device):
        if device is not None and torch.cuda.is_available():
            return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        return ctypes.c_void_p(0)

    @staticmethod
    def _device_of(keep):
        for t in keep:
            if isinstance(t, torch.Tensor) and t.is_cuda:
                return t.device
        return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else None

    @classmethod
    def from_parts(cls, num_nodes, column_index, part_pointers, part2Node, rows=None, device=None):
        """Original part layout (upstream `SAG` / `GNNA_*`, reuse_conv.cpp:132-205)."""
        ci, pp, pn = map(_as_index, (column_index, part_pointers, part2Node))
        where = _same_place([ci, pp, pn])
        keep = [ci[0], pp[0], pn[0]]
        device = device or cls._device_of(keep)
        r0, r1 = rows if rows is not None else (0, num_nodes)
        h = ctypes.c_void_p()
        with _device_guard(device):
            _native.check(_native.cuda().rof_plan_create_parts(
                ctypes.byref(h), where, num_nodes, r0, r1, ci[1], ci[2], pp[1], pn[1], pn[2], cls._stream(device)))
        return cls(h, "parts", device, keep)

    @classmethod
    def from_v1(cls, num_nodes, column_index, part_pointers, part2Node, part_cache_flagindex,
                part_pointers_cache, column_index_cache, rows=None, device=None):
        """ROF_v1 layout (upstream `reuse_*_v1`, reuse_conv.cpp:208-285)."""
        ci, pp, pn, fl, pc, cc = map(_as_index, (column_index, part_pointers, part2Node, part_cache_flagindex,
                                                  part_pointers_cache, column_index_cache))
        where = _same_place([ci, pp, pn, fl, pc, cc])
        keep = [ci[0], pp[0], pn[0], fl[0], pc[0], cc[0]]
        device = device or cls._device_of(keep)
        r0, r1 = rows if rows is not None else (0, num_nodes)
        groups = max(0, pc[2] - 1)
        h = ctypes.c_void_p()
        with _device_guard(device):
            _native.check(_native.cuda().rof_plan_create_v1(
                ctypes.byref(h), where, num_nodes, r0, r1, ci[1], ci[2], pp[1], pn[1], pn[2], fl[1], pc[1], cc[1],
                groups, cls._stream(device)))
        return cls(h, "v1", device, keep)

    @classmethod
    def from_v2(cls, num_nodes, uniqpart_column_index, uniqpart_pointers, part2Node_ptr, part2Node_col,
                rows=None, device=None):
        """ROF_v2 layout (upstream `reuse_*_v2`, reuse_conv.cpp:288-346)."""
        ci, up, np_, nc = map(_as_index, (uniqpart_column_index, uniqpart_pointers, part2Node_ptr, part2Node_col))
        where = _same_place([ci, up, np_, nc])
        keep = [ci[0], up[0], np_[0], nc[0]]
        device = device or cls._device_of(keep)
        r0, r1 = rows if rows is not None else (0, num_nodes)
        h = ctypes.c_void_p()
        with _device_guard(device):
            _native.check(_native.cuda().rof_plan_create_v2(
                ctypes.byref(h), where, num_nodes, r0, r1, ci[1], ci[2], up[1], np_[1], nc[1], max(0, up[2] - 1),
                cls._stream(device)))
        return cls(h, "v2", device, keep)

    def stages(self, block_rows, stage_of_block):
        """Split this plan for the multi-GPU pipeline (rof_plan_create_stages): feature block b
        (rows [b*block_rows, (b+1)*block_rows)) becomes readable in stage stage_of_block[b].
        Returns the list of per-stage plans; run them in order, all but the first with
        accumulate=True."""
        sob = np.ascontiguousarray(stage_of_block, dtype=np.int32)
        num_stages = int(sob.max()) + 1 if sob.size else 1
        handles = (ctypes.c_void_p * num_stages)()
        with _device_guard(self.device):
            _native.check(_native.cuda().rof_plan_create_stages(
                self._h, int(block_rows), ctypes.c_void_p(sob.ctypes.data), int(sob.size), num_stages, handles,
                self._stream(self.device)))
        return [AggregationPlan(ctypes.c_void_p(h), self.layout + ":stage", self.device, self._keep) for h in handles]

    def stages_by_ranges(self, range_bounds, stage_of_range):
        """Like `stages` for feature rows owned in ranges of any length
        (rof_plan_create_stages_ranges): range r = rows [range_bounds[r], range_bounds[r+1]) becomes
        readable in stage stage_of_range[r]."""
        rb = np.ascontiguousarray(range_bounds, dtype=np.int32)
        sr = np.ascontiguousarray(stage_of_range, dtype=np.int32)
        if rb.size != sr.size + 1:
            raise ValueError("range_bounds needs one more entry than stage_of_range")
        num_stages = int(sr.max()) + 1 if sr.size else 1
        handles = (ctypes.c_void_p * num_stages)()
        with _device_guard(self.device):
            _native.check(_native.cuda().rof_plan_create_stages_ranges(
                self._h, ctypes.c_void_p(rb.ctypes.data), ctypes.c_void_p(sr.ctypes.data), int(sr.size), num_stages,
                handles, self._stream(self.device)))
        return [AggregationPlan(ctypes.c_void_p(h), self.layout + ":stage", self.device, self._keep) for h in handles]

    # -- inspection --------------------------------------------------------------------
    def export(self):
        i = self.info
        rows = i["row_end"] - i["row_begin"]
        out = {
            "row_ptr": np.zeros(rows + 1, np.int64), "col": np.zeros(i["gather_entries"], np.int32),
            "group_ptr": np.zeros(i["num_groups"] + 1, np.int32), "group_col": np.zeros(i["group_sources"], np.int32),
            "items": np.zeros((i["num_items"], 4), np.int32), "split_rows": np.zeros((i["split_rows"], 4), np.int32),
        }
        p = lambda a: ctypes.c_void_p(a.ctypes.data)
        _native.check(_native.cuda().rof_plan_export(self._h, p(out["row_ptr"]), p(out["col"]), p(out["group_ptr"]),
                                                     p(out["group_col"]), p(out["items"]), p(out["split_rows"])))
        return out

    def export_tiles(self):
        """shared-memory tiles of the plan (rof_plan_export_tiles); empty arrays when it has none"""
        i = self.info
        out = {"tiles": np.zeros((i["num_tiles"], 4), np.int32), "titems": np.zeros((i["tile_items"], 4), np.int32),
               "tcol": np.zeros(i["tile_entries"], np.int32), "stage_col": np.zeros(i["num_tiles"] * 64, np.int32)}
        p = lambda a: ctypes.c_void_p(a.ctypes.data)
        _native.check(_native.cuda().rof_plan_export_tiles(self._h, p(out["tiles"]), p(out["titems"]), p(out["tcol"]),
                                                           p(out["stage_col"])))
        return out

    def workspace_bytes(self, dim):
        return int(_native.cuda().rof_plan_workspace_bytes(self._h, int(dim)))

    def algorithmic_bytes(self, dim, mode="gcn"):
        return int(_native.cuda().rof_plan_algorithmic_bytes(self._h, int(dim), MODES[mode]))

    # -- the hot call ------------------------------------------------------------------
    def _get_workspace(self, nbytes, device):
        ws = self._workspace
        if ws is None or ws.numel() < nbytes or ws.device != device:
            # torch's caching allocator returns 512-byte aligned blocks
            ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
            self._workspace = ws
        return ws

    # -- source tiling -----------------------------------------------------------------
    def auto_tiles(self, dim):
        """How many source-row tiles to walk the feature matrix in.  When the matrix is larger
        than L2 (126 MB) and rows are long, summing one L2-sized block of source rows at a time
        (per-tile plans from `stages`, accumulated into `out`) turns DRAM gathers into L2 hits:
        measured on B200, 114.6M-edge graph: D=256 6.9 -> 6.2 ms (4 tiles), D=602 20.0 -> 14.9 ms.
        Short rows lose more to the extra per-row passes than they gain (mean degree 50: 1 tile)."""
        i = self.info
        rows = max(i["row_end"] - i["row_begin"], 1)
        feat_bytes = i["num_nodes"] * dim * 4
        if feat_bytes <= 100e6:
            return 1
        tiles = 1
        while tiles < 8 and feat_bytes / tiles > 64e6:
            tiles *= 2
        while tiles > 1 and i["gather_entries"] / rows / tiles < 48:
            tiles //= 2
        return tiles

    def tile_plans(self, tiles):
        if tiles <= 1:
            return [self]
        tp = self._tiled.get(tiles)
        if tp is None:
            blk = (self.info["num_nodes"] + tiles - 1) // tiles
            tp = self.stages(blk, list(range(tiles)))
            self._tiled[tiles] = tp
        return tp

    def aggregate(self, x, degrees=None, mode="gcn", out=None, cache_result=None, workspace=None, phases=7,
                  accumulate=False, tiles=1, gather_events=None, bias=None, self_x=None, self_scale=1.0,
                  relu=False, _cache_rows=None):
        """out[v] = scale(v) * sum over v's gathered rows; see rof_aggregate() in include/rof_b200.h.
        `x` is [num_nodes, dim] fp32 on the GPU; returns a new [rows, dim] tensor unless `out` is given.
        tiles: 1 = one pass over the whole plan; N > 1 or "auto" = N source tiles (see auto_tiles).
        gather_events: optional list; (start, stop) CUDA events around every phase-B launch are appended.
        bias / self_x / self_scale / relu: fused epilogue out = act(result + self_scale * self_x + bias)
        (rof_aggregate_fused); self_x is [num_nodes, dim] indexed by global row id."""
        if tiles == "auto":
            tiles = self.auto_tiles(x.size(1)) if (phases == 7 and not accumulate) else 1
        if tiles > 1:
            if phases != 7 or accumulate:
                raise RuntimeError("source tiling runs whole passes")
            self.launches = 0
            plans = self.tile_plans(tiles)
            for k, p in enumerate(plans):
                last = k + 1 == len(plans)                 # the epilogue belongs to the last tile only
                # every tile fills the rows of the part_result_cache whose groups it builds
                out = p.aggregate(x, degrees, mode, out=out, cache_result=cache_result, workspace=workspace,
                                  accumulate=k > 0, gather_events=gather_events, bias=bias if last else None,
                                  self_x=self_x if last else None, self_scale=self_scale, relu=relu and last,
                                  _cache_rows=self.info["num_groups"])
                self.launches += p.launches
            return out
        if not x.is_cuda:
            raise RuntimeError("x must be a CUDA tensor")            # upstream CHECK_CUDA, reuse_conv.cpp:121
        if x.dtype != torch.float32 or x.dim() != 2:
            raise RuntimeError("x must be a 2-D float32 tensor")
        if x.stride(1) != 1 and x.size(1) > 1:
            raise RuntimeError("x must be contiguous")               # upstream CHECK_CONTIGUOUS, reuse_conv.cpp:122
        i = self.info
        if x.size(0) != i["num_nodes"]:
            raise RuntimeError(f"x has {x.size(0)} rows, the plan was built for {i['num_nodes']} nodes")
        dim = x.size(1)
        rows = i["row_end"] - i["row_begin"]
        if out is None:
            if accumulate:
                raise RuntimeError("accumulate=True adds to an existing `out`")
            out = torch.empty((rows, dim), dtype=torch.float32, device=x.device)
        else:
            self._check_out(out, rows, dim, x.device)
        m = MODES[mode]
        deg_ptr = None
        if m != MODES["sum"]:
            if (degrees is None or degrees.device != x.device or degrees.dtype != torch.float32
                    or not degrees.is_contiguous()):
                raise RuntimeError("degrees must be a contiguous float32 CUDA tensor on x's device")
            if degrees.numel() != i["num_nodes"]:
                raise RuntimeError("degrees must have one entry per node")
            deg_ptr = ctypes.c_void_p(degrees.data_ptr())
        cache_ptr = None
        if cache_result is not None:
            cache_rows = i["num_groups"] if _cache_rows is None else _cache_rows
            if (not cache_result.is_cuda or cache_result.dtype != torch.float32 or not cache_result.is_contiguous()
                    or tuple(cache_result.shape) != (cache_rows, dim + 1)):
                raise RuntimeError(f"part_result_cache must be a contiguous float32 CUDA tensor of shape "
                                   f"[{cache_rows}, {dim + 1}]")
            cache_ptr = ctypes.c_void_p(cache_result.data_ptr())
        bias_ptr = self_ptr = None
        ld_self = 0
        if bias is not None:
            if not bias.is_cuda or bias.dtype != torch.float32 or not bias.is_contiguous() or bias.numel() != dim:
                raise RuntimeError("bias must be a contiguous float32 CUDA tensor with `dim` entries")
            bias_ptr = ctypes.c_void_p(bias.data_ptr())
        if self_x is not None:
            if (not self_x.is_cuda or self_x.dtype != torch.float32 or self_x.dim() != 2 or self_x.size(1) != dim
                    or self_x.size(0) != i["num_nodes"] or (self_x.stride(1) != 1 and dim > 1)):
                raise RuntimeError("self_x must be a float32 CUDA tensor of shape [num_nodes, dim]")
            self_ptr = ctypes.c_void_p(self_x.data_ptr())
            ld_self = self_x.stride(0) if self_x.size(0) > 1 else dim
        need = self.workspace_bytes(dim)
        ws = workspace if workspace is not None else (self._get_workspace(need, x.device) if need else None)
        ldx = x.stride(0) if x.size(0) > 1 else dim
        ldo = out.stride(0) if rows > 1 else dim
        lib = _native.cuda()
        self.launches = 0
        with _device_guard(x.device):
            stream = ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
            # with gather_events the three phases are issued one by one so that phase B can be bracketed
            for ph in ((1, 2, 4) if (gather_events is not None and phases == 7) else (int(phases),)):
                if gather_events is not None and ph & 2:
                    e0 = torch.cuda.Event(enable_timing=True)
                    e0.record()
                if _NVTX:
                    torch.cuda.nvtx.range_push(_PHASE_NAMES.get(ph, "rof:phases"))
                try:
                    _native.check(lib.rof_aggregate_fused(
                        self._h, ph | (8 if accumulate else 0), m, ctypes.c_void_p(x.data_ptr()), ldx, dim, deg_ptr,
                        ctypes.c_void_p(out.data_ptr()), ldo, cache_ptr,
                        ctypes.c_void_p(ws.data_ptr()) if ws is not None else None,
                        ws.numel() if ws is not None else 0, bias_ptr, self_ptr, ld_self,
                        ctypes.c_float(float(self_scale)), int(bool(relu)), stream))
                finally:
                    if _NVTX:
                        torch.cuda.nvtx.range_pop()
                self.launches += int(lib.rof_last_launch_count())
                if gather_events is not None and ph & 2:
                    e1 = torch.cuda.Event(enable_timing=True)
                    e1.record()
                    gather_events.append((e0, e1))
        return out

    @staticmethod
    def _check_out(out, rows, dim, device):
        if (out.dtype != torch.float32 or out.device != device or out.dim() != 2 or out.size(0) != rows
                or out.size(1) != dim or (out.stride(1) != 1 and dim > 1)):
            raise RuntimeError("out must be a float32 tensor of shape [rows, dim] with unit column stride on x's device")

    def take_status(self):
        """non-zero when a bounded wait inside a kernel of an earlier pass ran out (rof_plan_take_status)"""
        return int(_native.cuda().rof_plan_take_status(self._h))

    def aggregate_static_scratch(self, x, degrees=None, mode="gcn", out=None):
        """rof_aggregate_static_scratch(): the same pass with the library's built-in 32 MiB scratch
        instead of a workspace, for callers that cannot allocate device memory at call time.  Here
        torch still allocates `out` when none is given — pass `out` to allocate nothing at all.
        Raises RofError (ROF_ERR_WORKSPACE) when the pass needs more scratch than is built in."""
        i = self.info
        if not x.is_cuda or x.dtype != torch.float32 or x.dim() != 2 or (x.stride(1) != 1 and x.size(1) > 1):
            raise RuntimeError("x must be a 2-D float32 CUDA tensor with unit column stride")
        if x.size(0) != i["num_nodes"]:
            raise RuntimeError(f"x has {x.size(0)} rows, the plan was built for {i['num_nodes']} nodes")
        dim, rows = x.size(1), i["row_end"] - i["row_begin"]
        if out is None:
            out = torch.empty((rows, dim), dtype=torch.float32, device=x.device)
        else:
            self._check_out(out, rows, dim, x.device)
        deg_ptr = None
        if MODES[mode] != MODES["sum"]:
            if (degrees is None or degrees.device != x.device or degrees.dtype != torch.float32
                    or not degrees.is_contiguous() or degrees.numel() != i["num_nodes"]):
                raise RuntimeError("degrees must be a contiguous float32 tensor on x's device with one entry per node")
            deg_ptr = ctypes.c_void_p(degrees.data_ptr())
        with _device_guard(x.device):
            _native.check(_native.cuda().rof_aggregate_static_scratch(
                self._h, MODES[mode], ctypes.c_void_p(x.data_ptr()), x.stride(0) if x.size(0) > 1 else dim, dim,
                deg_ptr, ctypes.c_void_p(out.data_ptr()), out.stride(0) if rows > 1 else dim,
                ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)))
        return out

    def prepared_call(self, x, degrees, mode, out, accumulate):
        """-> (function, argument list) of the C-ABI call that `aggregate(x, degrees, mode, out=out,
        accumulate=accumulate)` makes, for callers that repeat the very same pass many times and have
        validated it once through `aggregate` (the multi-GPU pipeline: several small launches per pass, where
        the Python-side checks would otherwise be a visible share of the pass).  The last list entry is the
        stream; the caller sets it before every call.  The tensors must outlive the prepared call."""
        dim = x.size(1)
        rows = self.info["row_end"] - self.info["row_begin"]
        need = self.workspace_bytes(dim)
        ws = self._get_workspace(need, x.device) if need else None
        m = MODES[mode]
        args = [self._h, 7 | (8 if accumulate else 0), m, ctypes.c_void_p(x.data_ptr()),
                x.stride(0) if x.size(0) > 1 else dim, dim,
                ctypes.c_void_p(degrees.data_ptr()) if (degrees is not None and m != MODES["sum"]) else None,
                ctypes.c_void_p(out.data_ptr()), out.stride(0) if rows > 1 else dim, None,
                ctypes.c_void_p(ws.data_ptr()) if ws is not None else None, ws.numel() if ws is not None else 0,
                None, None, 0, ctypes.c_float(0.0), 0, None]
        return _native.cuda().rof_aggregate_fused, args

    def last_launch_count(self):
        return self.launches


class _device_guard:
    def __init__(self, device):
        self.device = device
        self.ctx = None

    def __enter__(self):
        if self.device is not None and torch.cuda.is_available():
            self.ctx = torch.cuda.device(self.device)
            self.ctx.__enter__()

    def __exit__(self, *a):
        if self.ctx is not None:
            self.ctx.__exit__(*a)
