"""Row-block sharding of the aggregation over the GPUs of one node.

Destinations are independent, so rank r owns an equal block of destination rows and a plan
built for that block only; what the ranks exchange per pass is the feature matrix: every rank
contributes its block of rows and receives all of them (one all-gather over NCCL / NVLink)
into a full [N, D] buffer in its own HBM.  Kernels only ever read local memory.
Upstream is single-GPU (no collective anywhere in its tree); this module is new.
"""
import torch
import torch.distributed as dist


def row_blocks(num_nodes, world):
    """-> (block_rows, [(r0, r1)] per rank).  Equal-sized blocks (the last may be short or
    empty) so that one all_gather_into_tensor moves the whole matrix."""
    blk = (num_nodes + world - 1) // world if world > 0 else num_nodes
    return blk, [(min(r * blk, num_nodes), min((r + 1) * blk, num_nodes)) for r in range(world)]


class ShardedFeatures:
    """The padded [world*block, D] receive buffer of one feature matrix and its all-gather."""

    def __init__(self, num_nodes, dim, rank, world, device, dtype=torch.float32, group=None):
        self.n, self.dim, self.rank, self.world, self.group = num_nodes, dim, rank, world, group
        self.block, self.blocks = row_blocks(num_nodes, world)
        self.full = torch.zeros((self.block * world, dim), dtype=dtype, device=device)

    @property
    def local_rows(self):
        r0, r1 = self.blocks[self.rank]
        return r1 - r0

    def local_view(self):
        """this rank's block inside the full buffer (block rows, the tail beyond N is padding)"""
        return self.full[self.rank * self.block:(self.rank + 1) * self.block]

    def all_gather(self, x_local=None):
        """x_local: [block, D] (padded) or None to send the rows already in local_view().
        Returns the full [N, D] matrix (a view without the padding rows)."""
        src = self.local_view() if x_local is None else x_local
        if src.shape != (self.block, self.dim):
            raise RuntimeError(f"local block must be [{self.block}, {self.dim}] (padded), got {tuple(src.shape)}")
        if self.world > 1:
            dist.all_gather_into_tensor(self.full, src.contiguous(), group=self.group)
        elif x_local is not None:
            self.full.copy_(src)
        return self.full[:self.n]


class ShardedAggregator:
    """plan for this rank's row block + the all-gather in front of it"""

    def __init__(self, plan, features: ShardedFeatures):
        r0, r1 = features.blocks[features.rank]
        if (plan.info["row_begin"], plan.info["row_end"]) != (r0, r1):
            raise RuntimeError("the plan does not cover this rank's row block")
        self.plan, self.features = plan, features

    def aggregate(self, x_local, degrees, mode, out=None, phases=7):
        x_full = self.features.all_gather(x_local)
        return self.plan.aggregate(x_full, degrees, mode, out=out, phases=phases)


def stage_schedule(world):
    """Which peers' blocks travel in which stage, as lists of ring offsets k (the block of rank
    (r + k) % world).  Stage 0 is the rank's own block; the peers are cut into two groups, the
    nearer (world-1)//2 first, so that a pass is three stages whatever the world size: the
    aggregation of one stage covers the transfer of the next, while the number of kernel launches
    and NCCL calls per pass stays fixed.  [[0], [1, 2, 3], [4, 5, 6, 7]] for 8 ranks, [[0], [1],
    [2, 3]] for 4.  Measured on B200s, 114.6M-edge graph, D=256, ms per forward+backward step —
    8 GPUs: [[0],[1,2,3],[4..7]] 2.57; [[0],[1..7]] 2.66; no overlap 2.77; [[0,1,2,3],[4..7]] 2.77;
    [[0],[1],[2,3,4],[5,6,7]] 3.03; one stage per peer 5.7 (launch-bound);
    4 GPUs: [[0],[1],[2,3]] 3.63; [[0],[1,2,3]] 3.96."""
    if world <= 1:
        return [[0]]
    first = max(1, (world - 1) // 2)
    stages = [[0], list(range(1, 1 + first))]
    if 1 + first < world:
        stages.append(list(range(1 + first, world)))
    return stages


class PipelinedAggregator:
    """All-gather overlapped with aggregation, stage by stage.

    Rank r reads its own block in stage 0 and the blocks of ranks (r + k) % world, k in the
    stage's offsets (see stage_schedule), in the later stages.  Each stage's blocks travel as one
    group of paired sends/receives on a side stream (send the own block to rank r-k, receive the
    block of rank r+k; NVSwitch gives every pair full bandwidth), and the per-stage plans
    (AggregationPlan.stages) run on the compute stream as soon as their blocks have landed,
    adding into `out`.  The result equals the whole-plan aggregate up to the order of the fp32
    adds.  Every kernel reads this GPU's memory only.
    """

    def __init__(self, plan, features: ShardedFeatures, stage_plans=None, schedule=None):
        f = features
        r0, r1 = f.blocks[f.rank]
        if (plan.info["row_begin"], plan.info["row_end"]) != (r0, r1):
            raise RuntimeError("the plan does not cover this rank's row block")
        self.features, self.whole = f, plan
        self.schedule = schedule or stage_schedule(f.world)
        stage_of_offset = {k: s for s, ks in enumerate(self.schedule) for k in ks}
        stage_of_block = [stage_of_offset[(b - f.rank) % f.world] for b in range(f.world)]
        if stage_plans is not None:
            self.stage_plans = stage_plans
        else:
            self.stage_plans = plan.stages(f.block, stage_of_block) if f.world > 1 else [plan]
        dev = f.full.device
        self.comm_stream = torch.cuda.Stream(dev) if f.world > 1 else None
        self.ready = torch.cuda.Event() if f.world > 1 else None
        self.landed = [torch.cuda.Event() for _ in self.schedule]
        self.launches = 0

    def aggregate(self, x_local, degrees, mode, out):
        f = self.features
        R, r, blk = f.world, f.rank, f.block
        cur = torch.cuda.current_stream(f.full.device)
        if x_local is not None:
            f.local_view().copy_(x_local)
        x_full = f.full[:f.n]
        if R > 1:
            self.ready.record(cur)
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(self.ready)
                for s in range(len(self.schedule)):
                    ops = []
                    for k in self.schedule[s]:
                        if k == 0:
                            continue                     # the rank's own block is already in place
                        src = (r + k) % R
                        ops.append(dist.P2POp(dist.isend, f.local_view(), (r - k) % R, group=f.group))
                        ops.append(dist.P2POp(dist.irecv, f.full[src * blk:(src + 1) * blk], src, group=f.group))
                    if ops:
                        for w in dist.batch_isend_irecv(ops):
                            w.wait()
                    self.landed[s].record(self.comm_stream)
        self.launches = 0
        for s, p in enumerate(self.stage_plans):
            if R > 1 and any(k != 0 for k in self.schedule[s]):
                cur.wait_event(self.landed[s])
            p.aggregate(x_full, degrees, mode, out=out, accumulate=s > 0)
            self.launches += p.last_launch_count()
        return out
