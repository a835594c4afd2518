/*
 * rof_b200 — C ABI of the B200 (sm_100a) neighbour-aggregation library.
 *
 * This is the boundary a host program binds instead of upstream's pybind11 module `ROF`
 * (ROF/reuse_conv/reuse_conv.cpp:353-365).  Upstream's seven entry points all reduce to
 * "aggregate a [N, D] fp32 matrix over one of three index layouts"; the dense X.W products
 * around it (reuse_conv_kernel.cu:302, 382-383, 621, 819-820, 971, 1050-1051) stay with the
 * caller's BLAS.  Here that is two steps:
 *
 *   1. build a plan once per graph from the index tensors exactly as upstream's host-side
 *      preprocessor emits them (int32; on the host or already on the device);
 *   2. call rof_aggregate() per layer / per direction with raw device pointers and a stream.
 *
 * No function allocates per call except the plan constructors; rof_aggregate() uses only the
 * caller's workspace.  All functions return a rof_status; none exits the process (upstream
 * prints and calls exit(-1) on a launch error, reuse_conv_kernel.cu:114-118).  All pointers
 * are plain C pointers; `stream` is a cudaStream_t passed as void*.
 */
#ifndef ROF_B200_H_
#define ROF_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct rof_plan rof_plan;

enum rof_status {
  ROF_OK = 0,
  ROF_ERR_BAD_ARGUMENT = 1,   /* null pointer, negative size, unknown enum value, misaligned ld */
  ROF_ERR_BAD_LAYOUT = 2,     /* index tensors violate an invariant of the upstream layouts */
  ROF_ERR_CUDA = 3,           /* a CUDA runtime call failed; see rof_last_error() */
  ROF_ERR_WORKSPACE = 4,      /* workspace missing, misaligned or smaller than rof_plan_workspace_bytes() */
  ROF_ERR_NO_MEMORY = 5,      /* host allocation failed while building a plan, or rof_shared_alloc found no device memory */
  ROF_ERR_WAIT_LIMIT = 6      /* a bounded device-side wait (shared-memory ring copies) gave up */
};

/* What is summed.  Upstream implements GCN (its GNNA / ROF_v1 / ROF_v2 kernels,
 * reuse_conv_kernel.cu:254,270,276-283) and SUM (its SAG kernel, :185); MEAN is
 * SUM followed by 1/degrees[dst] (0 for an empty row). */
enum rof_mode {
  ROF_MODE_GCN = 0,  /* out[v] = rsqrt(deg[v]) * sum_n rsqrt(deg[n]) * x[n] */
  ROF_MODE_SUM = 1,  /* out[v] = sum_n x[n] */
  ROF_MODE_MEAN = 2, /* out[v] = (sum_n x[n]) / deg[v] */
  /* GCN over rows the caller already multiplied by rsqrt(deg[n]) (rof_scale_rows):
   * out[v] = rsqrt(deg[v]) * sum_n x[n].  Same products as ROF_MODE_GCN — upstream multiplies
   * inside its kernels, once per lane per neighbour (reuse_conv_kernel.cu:254, 914) — without
   * the degree load and the rsqrt per gathered row. */
  ROF_MODE_GCN_PRESCALED = 3
};

enum rof_location { ROF_ON_HOST = 0, ROF_ON_DEVICE = 1 };

typedef struct rof_plan_info {
  int64_t num_nodes;        /* N: rows of the feature matrix */
  int64_t row_begin;        /* first destination row this plan produces */
  int64_t row_end;          /* one past the last destination row */
  int64_t num_groups;       /* G: reuse groups whose partial sum is built in phase A */
  int64_t group_sources;    /* rows gathered by phase A (sum of group sizes) */
  int64_t gather_entries;   /* rows gathered by phase B: partial rows + residual source rows */
  int64_t partial_entries;  /* how many of gather_entries are partial rows (sum of fan-outs) */
  int64_t original_edges;   /* edges the same rows hold without reuse */
  int64_t num_items;        /* work items of phase B (rows + segments of split rows) */
  int64_t split_rows;       /* rows cut into segments (second-stage reduce) */
  int64_t num_slots;        /* segment sums held in scratch between phase B and the reduce */
  int64_t segment_edges;    /* maximum entries per work item */
  int64_t num_tiles;            /* shared-memory tiles of short rows (0: the plan has none) */
  int64_t tile_items;           /* rows covered by tiles */
  int64_t tile_entries;         /* their entries */
  int64_t tile_shared_entries;  /* of which are read from shared memory instead of global memory */
  int64_t tile_staged_rows;     /* rows copied into shared memory, summed over the tiles */
} rof_plan_info;

/*
 * Plan constructors.  `where` says whether the int32 index arrays are host or device memory
 * (device arrays are copied to the host once; `stream` orders that copy).  A plan covers the
 * destination rows [row_begin, row_end) — pass 0 and num_nodes for the whole graph; a
 * multi-GPU run gives each rank its own block.  Feature rows are always addressed globally.
 *
 * rof_plan_create_parts — the original part layout used by upstream's `SAG`, `GNNA_forward`
 *   and `GNNA_backward` (reuse_conv.cpp:132-205): column_index[num_column_index],
 *   part_pointers[num_parts+1], part2Node[num_parts].
 */
int rof_plan_create_parts(rof_plan** plan, int where, int num_nodes, int row_begin, int row_end,
                          const int32_t* column_index, int64_t num_column_index,
                          const int32_t* part_pointers, const int32_t* part2Node, int num_parts,
                          void* stream);

/*
 * rof_plan_create_v1 — the ROF_v1 layout of `reuse_forward_v1` / `reuse_backward_v1`
 *   (reuse_conv.cpp:208-285): the reorganised column_index, part_pointers, part2Node, plus
 *   part_cache_flagindex[num_parts] (0, or 1 + group id), part_pointers_cache[num_groups+1]
 *   and column_index_cache[part_pointers_cache[num_groups]].
 */
int rof_plan_create_v1(rof_plan** plan, int where, int num_nodes, int row_begin, int row_end,
                       const int32_t* column_index, int64_t num_column_index,
                       const int32_t* part_pointers, const int32_t* part2Node, int num_parts,
                       const int32_t* part_cache_flagindex, const int32_t* part_pointers_cache,
                       const int32_t* column_index_cache, int num_groups, void* stream);

/*
 * rof_plan_create_v2 — the ROF_v2 layout of `reuse_forward_v2` / `reuse_backward_v2`
 *   (reuse_conv.cpp:288-346): uniqpart_column_index, uniqpart_pointers[num_uniqparts+1],
 *   part2Node_ptr[num_uniqparts+1], part2Node_col[part2Node_ptr[num_uniqparts]].
 */
int rof_plan_create_v2(rof_plan** plan, int where, int num_nodes, int row_begin, int row_end,
                       const int32_t* uniqpart_column_index, int64_t num_column_index,
                       const int32_t* uniqpart_pointers, const int32_t* part2Node_ptr,
                       const int32_t* part2Node_col, int num_uniqparts, void* stream);

void rof_plan_destroy(rof_plan* plan);
int rof_plan_get_info(const rof_plan* plan, rof_plan_info* info);

/*
 * Copy the plan's derived arrays to host memory for inspection (any pointer may be NULL):
 *   row_ptr    [row_end-row_begin+1] int64  entry range of each destination row
 *   col        [gather_entries]      int32  < num_nodes: feature row; >= num_nodes: partial row
 *   group_ptr  [num_groups+1]        int32  source range of each reuse group
 *   group_col  [group_sources]       int32
 *   items      [num_items][4]        int32  (begin, end, dst, mid); dst<0: segment slot -dst-1;
 *                                            entries [begin,mid) are partial rows, [mid,end) feature rows
 *   split_rows [split_rows][4]       int32  (row, first_slot, slot_count, 0)
 * A plan built on a machine without a CUDA device can be exported but not run.
 */
int rof_plan_export(const rof_plan* plan, int64_t* row_ptr, int32_t* col, int32_t* group_ptr,
                    int32_t* group_col, int32_t* items, int32_t* split_rows);

/*
 * Shared-memory tiles of a plan (inspection; any pointer may be NULL).  Where the short rows of a
 * graph share many of their entries — reuse groups fanned out to neighbouring destinations, the
 * regime upstream's partial-sum reuse is built for (reuse_conv_kernel.cu:902-952) — the plan groups
 * 32 consecutive short rows into a tile and lists the entries used at least twice inside it; the
 * tile kernel stages those rows once in shared memory and every destination of the tile adds them
 * from there.
 *   tiles     [num_tiles][4]   int32  (first_item, num_items, stage_begin, stage_count)
 *   titems    [tile_items][4]  int32  (begin, end, dst, mid) into tcol: [begin,mid) slot numbers of
 *                                      the tile's staged rows, [mid,end) global ids (as in `col`)
 *   tcol      [tile_entries]   int32
 *   stage_col [num_tiles * 64] int32  ids of the rows staged by each tile (stage_count valid per tile)
 */
int rof_plan_export_tiles(const rof_plan* plan, int32_t* tiles, int32_t* titems, int32_t* tcol,
                          int32_t* stage_col);

/*
 * Staged plans for the multi-GPU pipeline (no upstream counterpart: upstream is single-GPU).
 * The feature matrix is owned in blocks of `block_rows` consecutive rows; block b becomes
 * available in stage stage_of_block[b] (0 = already local, then the order in which peers'
 * blocks arrive).  `whole` is split into `num_stages` plans over the same destination rows:
 * stage k holds the entries whose source row arrives in stage k, and every reuse group is
 * built in the stage in which its last source arrives.  Running the stages in order — stage 0
 * plain, the others with ROF_PHASE_ACCUMULATE — gives the same sums as `whole`, while stage k
 * only reads blocks that have arrived by then.  stages_out receives num_stages plans.
 */
int rof_plan_create_stages(const rof_plan* whole, int block_rows, const int32_t* stage_of_block,
                           int num_blocks, int num_stages, rof_plan** stages_out, void* stream);

/*
 * The same split for feature rows owned in ranges of any length (row blocks balanced by edge
 * count, a peer's block cut into L2-sized tiles): range r covers feature rows
 * [range_bounds[r], range_bounds[r+1]) and becomes readable in stage stage_of_range[r];
 * range_bounds has num_ranges + 1 ascending entries from 0 to num_nodes.
 */
int rof_plan_create_stages_ranges(const rof_plan* whole, const int32_t* range_bounds,
                                  const int32_t* stage_of_range, int num_ranges, int num_stages,
                                  rof_plan** stages_out, void* stream);

/* Bytes of device scratch rof_aggregate() needs for feature width `dim`: the partial-sum
 * rows of phase A plus the segment sums of split rows.  256-byte aligned memory. */
int64_t rof_plan_workspace_bytes(const rof_plan* plan, int dim);

/* Algorithmic bytes of one rof_aggregate() call at width `dim`: 4*dim per gathered row and
 * per written row (phase A and phase B), plus 4 per index entry read. */
int64_t rof_plan_algorithmic_bytes(const rof_plan* plan, int dim, int mode);

/*
 * One aggregation pass: replaces the kernel launches inside upstream's
 * spmm_forward_cuda_GNNA / reuse_spmm_forward_cuda_v1 / reuse_spmm_forward_cuda_v2 and their
 * backward twins (reuse_conv_kernel.cu:290-386, 603-823, 957-1054).
 *
 *   x        [num_nodes, dim] fp32 device, row stride ldx (elements)
 *   degrees  [num_nodes] fp32 device (in-degrees as upstream passes them); unused for SUM
 *   out      [row_end-row_begin, dim] fp32 device, row stride ldo; every row is written
 *            exactly once (no zero-fill needed, no atomics)
 *   cache_result  optional [num_groups, dim+1] fp32 device: upstream's `part_result_cache`
 *            (ROF_v1 only); when given, phase A also stores each partial row and the 1.0
 *            "ready" flag there like upstream's caching kernel (:479-485).  May be NULL.  A plan made
 *            by rof_plan_create_stages*() fills the rows of the groups it builds, under the ids
 *            those groups have in the plan it was split from: give every stage the same buffer.
 *   workspace / workspace_bytes  device scratch, see rof_plan_workspace_bytes()
 *
 * Work is only enqueued on `stream`; the call does not synchronise.
 */
int rof_aggregate(const rof_plan* plan, int mode, const float* x, int64_t ldx, int dim,
                  const float* degrees, float* out, int64_t ldo, float* cache_result,
                  void* workspace, int64_t workspace_bytes, void* stream);

/*
 * The same pass, one phase at a time, for callers that want to time or overlap the phases:
 * A (ROF_PHASE_PARTIALS) builds the partial-sum rows of the reuse groups into the workspace,
 * B (ROF_PHASE_GATHER) sums every destination row (reads A's rows), C (ROF_PHASE_REDUCE)
 * combines the segment sums of split rows.  Phases must be issued in the order A, B, C on one
 * stream with the same arguments; rof_aggregate() is ROF_PHASE_ALL.  Upstream's counterpart
 * of A and B are the two launches of ROF_v1 (reuse_conv_kernel.cu:665, 692).
 */
enum rof_phase {
  ROF_PHASE_PARTIALS = 1, ROF_PHASE_GATHER = 2, ROF_PHASE_REDUCE = 4, ROF_PHASE_ALL = 7,
  ROF_PHASE_ACCUMULATE = 8 /* modifier: out += result (stage >= 1 of a staged pass) instead of out = result */
};

int rof_aggregate_phases(const rof_plan* plan, int phases, int mode, const float* x, int64_t ldx,
                         int dim, const float* degrees, float* out, int64_t ldo, float* cache_result,
                         void* workspace, int64_t workspace_bytes, void* stream);

/*
 * The same pass with the element-wise work that follows it fused into the store of each output row:
 *     out[v] = act( aggregate(v) + self_scale * self_x[v] + bias ),  act = max(., 0) when relu != 0.
 * `bias` ([dim]) and `self_x` ([num_nodes, dim], row stride ld_self, addressed by global row id) may be
 * NULL.  Covers the bias add that upstream's layer does in a separate pass after the operator
 * (reuse_conv.py:150), the activation its model applies next (ROF_main.py:181), and GIN's
 * (1 + eps) * x + sum over neighbours.  With source tiles or pipeline stages give the epilogue to the
 * LAST stage only (the earlier ones accumulate raw sums).  `phases` as in rof_aggregate_phases().
 */
int rof_aggregate_fused(const rof_plan* plan, int phases, int mode, const float* x, int64_t ldx, int dim,
                        const float* degrees, float* out, int64_t ldo, float* cache_result,
                        void* workspace, int64_t workspace_bytes, const float* bias, const float* self_x,
                        int64_t ld_self, float self_scale, int relu, void* stream);

/*
 * The same pass for callers that cannot allocate device memory (no counterpart in upstream,
 * whose wrappers allocate freely with torch): no workspace argument — the scratch is a fixed
 * array of ROF_STATIC_SCRATCH_BYTES inside the library, reserved on every GPU that loads it
 * until the process exits.  Meant for hosts that gave all of HBM to their own pool at start-up,
 * or that call from a section where a device allocation (a device-wide synchronisation) is not
 * acceptable.  Allocates nothing; no cache_result mirror.
 *   - A pass whose rof_plan_workspace_bytes(plan, dim) exceeds ROF_STATIC_SCRATCH_BYTES returns
 *     ROF_ERR_WORKSPACE and launches nothing.
 *   - The first call on each device looks up the array's device address; make that call during
 *     start-up, with the device current, before any stream capture begins.  With CUDA's lazy
 *     module loading that first call is also where the array gets its 32 MiB of device memory: a
 *     host that hands the rest of HBM to its own pool must make the call before it does so (a full
 *     valid pass — the address is looked up after the arguments have been checked).
 *   - The address is cached per device ordinal for the life of the process.  After
 *     cudaDeviceReset() (or any other teardown of the device's primary context) the cached address
 *     is stale and the entry point must not be used again in that process.
 *   - All calls on a GPU share the array, which keeps the previous call's contents (each pass
 *     writes every scratch row before reading it, so nothing has to be cleared).  Calls that
 *     overlap on the GPU race on it: keep them ordered on one stream.
 */
#define ROF_STATIC_SCRATCH_BYTES (32u << 20)
int rof_aggregate_static_scratch(const rof_plan* plan, int mode, const float* x, int64_t ldx, int dim,
                                 const float* degrees, float* out, int64_t ldo, void* stream);

/*
 * Row scaling pass in front of an aggregation: out[r][0:dim] = f(degrees[r]) * x[r][0:dim] for
 * r in [0, num_rows), f = 1 (ROF_SCALE_COPY), rsqrt (ROF_SCALE_RSQRT) or reciprocal, 0 for a
 * zero degree (ROF_SCALE_RECIPROCAL).  `out` may be `x` itself (in place) or a buffer with a
 * padded leading dimension; columns [dim, min(ldo, dim rounded up to 4)) of out are zeroed.
 * With ROF_SCALE_RSQRT it hoists upstream's per-neighbour factor rsqrt(degrees[n])
 * (reuse_conv_kernel.cu:254, 270) out of the gather: follow with ROF_MODE_GCN_PRESCALED.
 */
enum rof_scale_op { ROF_SCALE_COPY = 0, ROF_SCALE_RSQRT = 1, ROF_SCALE_RECIPROCAL = 2 };
int rof_scale_rows(const float* x, int64_t ldx, int dim, const float* degrees, int op, float* out, int64_t ldo,
                   int64_t num_rows, void* stream);

/*
 * Bandwidth probe (measurement aid, no upstream counterpart): streams `bytes` of device memory
 * `repeats` times through 128-bit loads that bypass L1 and discards the sum.  With a buffer that
 * fits L2 this measures the L2 -> SM read bandwidth the gather kernels are bounded by when the
 * feature rows are L2-resident; with a buffer much larger than L2, the HBM read bandwidth.
 * `sink` is one device float the kernel may write.
 */
int rof_probe_read(const void* buffer, int64_t bytes, int repeats, float* sink, void* stream);

/*
 * One asynchronous copy of `bytes` between two device buffers that this process can address: the
 * current GPU's memory, or a peer GPU's mapped here (CUDA IPC, peer access).  No upstream
 * counterpart (upstream runs on one GPU); it is the transport of the multi-GPU pipeline in which
 * copy engines pull a peer's feature rows over NVLink while this GPU's SMs run the gather, which
 * an SM-driven collective cannot do next to a kernel that saturates HBM.  Ordered on `stream`
 * like any other call of this interface; no kernel is given the peer's memory.
 */
int rof_copy_async(void* dst, const void* src, int64_t bytes, void* stream);

/*
 * Device buffers that other processes of the box can map (one process per GPU): the feature
 * buffer whose rows the peers pull with rof_copy_async.  rof_shared_alloc allocates `bytes` on the
 * current GPU (its own allocation, so that the exported handle covers exactly this buffer) and
 * writes the 64-byte interprocess handle; rof_shared_open maps another process' buffer into the
 * current GPU's address space (peer access is enabled by the driver on first use) and
 * rof_shared_close unmaps it; rof_shared_free releases an own buffer once no peer maps it any more.
 * The handle travels between the processes by any host channel (here: torch.distributed objects).
 */
#define ROF_SHARED_HANDLE_BYTES 64
int rof_shared_alloc(int64_t bytes, void** ptr, unsigned char* handle);
int rof_shared_open(const unsigned char* handle, void** ptr);
int rof_shared_close(void* ptr);
int rof_shared_free(void* ptr);

/* Reads and clears the plan's device status word: non-zero when a bounded wait inside a kernel
 * of an earlier pass ran out (that pass's output is incomplete).  rof_aggregate() checks it on
 * entry and returns ROF_ERR_WAIT_LIMIT. */
int rof_plan_take_status(rof_plan* plan);

/* Number of kernel launches the last rof_aggregate() on this thread enqueued. */
int rof_last_launch_count(void);

/* Message for the last non-OK status returned on this thread (never NULL). */
const char* rof_last_error(void);

/* Library version, and the compute capability the kernels were compiled for (100). */
int rof_version(void);
int rof_compiled_arch(void);

#ifdef __cplusplus
}
#endif
#endif /* ROF_B200_H_ */
