// Internal declarations shared by plan.cu, kernels.cu and api.cu.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "rof_b200.h"

namespace rof {

// One unit of gather work: sum the rows named by col[begin, end) and store the result.
//   dst >= 0 : final output row (global id; the kernel subtracts row_begin), scaled per mode
//   dst <  0 : segment of a split row; the unscaled sum goes to scratch slot (-dst - 1)
struct __align__(16) WorkItem {
  int32_t begin;
  int32_t end;
  int32_t dst;
  int32_t mid;   // entries [begin, mid) name partial rows, [mid, end) feature rows
};

// Second-stage reduce of a split row: out[row] = scale * (slot[first] + ... + slot[first+count-1]).
struct __align__(16) SplitRow {
  int32_t row;
  int32_t first_slot;
  int32_t count;
  int32_t pad;
};

constexpr int kMaxSegmentEdges = 8192;   // longest run of entries one work item sums
constexpr int kMinSegmentEdges = 256;
constexpr double kTargetSegments = 16000.0;  // for wide rows; four times as many for narrow ones
constexpr int kNarrowRowFloats = 32;          // rows up to this width use the finer cut
// Shared-memory tiles: rows of at most kTileMaxRowEntries entries are grouped kTileRows at a time (in
// row order); the entries that occur at least twice inside a tile — partial rows of reuse groups
// and feature rows that several of the tile's destinations gather — are staged once in shared
// memory (at most kTileMaxStage rows) and read from there.
constexpr double kMinReuseSaving = 0.15;      // ROF_v2 plans: reuse groups are used when they save at least this share of the gathered rows
constexpr int kTileRows = 32;
constexpr int kTileMaxRowEntries = 256;
constexpr int kTileMaxStage = 64;
constexpr double kTileMinSaved = 0.25;        // tiles are built when they save at least this share of the global row reads
constexpr int kTileMaxFloats = 256;           // widest feature row the tile kernel covers

}  // namespace rof

namespace rof {
// One shared-memory tile: items [first_item, first_item + num_items) of the tiled item list, and
// the rows to stage, stage_col[stage_begin .. stage_begin + stage_count).
struct __align__(16) TileDesc {
  int32_t first_item;
  int32_t num_items;
  int32_t stage_begin;
  int32_t stage_count;
};
}  // namespace rof

struct rof_plan {
  int device = 0;         // -1: built on a machine without a CUDA device (inspection only)
  int num_nodes = 0;
  int row_begin = 0, row_end = 0;
  int num_groups = 0;
  int64_t group_sources = 0;
  int64_t gather_entries = 0;
  int64_t partial_entries = 0;
  int64_t original_edges = 0;
  int num_items = 0;      // phase B
  int num_split_rows = 0;
  int num_slots = 0;
  int segment_edges = 0;  // rows longer than this are split

  // device arrays
  int32_t* d_col = nullptr;           // [gather_entries + group_sources]: phase-B entries, then group sources
  rof::WorkItem* d_items = nullptr;   // [num_items] phase B, longest first
  rof::WorkItem* d_group_items = nullptr;  // [num_groups] phase A (begin/end index d_col)
  // stage / tile plans: the id each group has in the plan they were split from (the row of the
  // caller's part_result_cache it fills); null for a plan built from index tensors (identity)
  int32_t* d_group_orig = nullptr;
  rof::SplitRow* d_split = nullptr;   // [num_split_rows]
  int32_t* d_slot_owner = nullptr;    // [num_slots]: index into d_split of the row a slot belongs to
  int32_t* d_arrive = nullptr;        // [num_split_rows]: segments of the row seen so far in this pass (0 between passes)
  // written by a kernel whose bounded wait ran out; host-mapped so that the next call sees it
  // without synchronising (0 = fine)
  int* h_status = nullptr;
  int* d_status = nullptr;

  // the same rows cut into shorter segments, used for narrow feature rows (several lane groups
  // per warp need more work items); absent (num_items == 0) when both cuts coincide
  struct FineCut {
    int num_items = 0, num_split_rows = 0, num_slots = 0, segment_edges = 0;
    rof::WorkItem* d_items = nullptr;
    rof::SplitRow* d_split = nullptr;
    int32_t* d_slot_owner = nullptr;
    int32_t* d_arrive = nullptr;
  } fine;

  // shared-memory tiles (absent when num_tiles == 0): the short rows in row order with their
  // entries rewritten as [staged slots | global rows]; the other items of each cut (long rows,
  // segments of split rows) stay with the lane-group kernel
  struct Tiled {
    int num_tiles = 0;
    int num_items = 0;              // rows covered by tiles
    int64_t entries = 0;            // their entries
    int64_t shared_entries = 0;     // of which read from shared memory
    int64_t staged_rows = 0;        // rows copied into shared memory over all tiles
    int32_t* d_tcol = nullptr;      // [entries]: per row, slot numbers first, then global ids (< N feature, >= N partial)
    rof::WorkItem* d_titems = nullptr;  // [num_items]: begin/end into d_tcol, mid = first global entry
    rof::TileDesc* d_tiles = nullptr;   // [num_tiles]
    int32_t* d_stage_col = nullptr;     // [num_tiles * kTileMaxStage]
    rof::WorkItem* d_rest_items = nullptr;  int num_rest = 0;        // coarse cut without the tiled rows
    rof::WorkItem* d_rest_items_fine = nullptr;  int num_rest_fine = 0;
    // host copies for rof_plan_export_tiles()
    std::vector<int32_t> h_tcol, h_stage_col;
    std::vector<rof::WorkItem> h_titems;
    std::vector<rof::TileDesc> h_tiles;
  } tiled;

  // host copies kept for rof_plan_export*(): the small arrays always, the entry arrays
  // only when there is no device to read them back from
  std::vector<int64_t> h_row_ptr;
  std::vector<int32_t> h_group_ptr;
  std::vector<int32_t> h_group_orig;   // host copy of d_group_orig (empty: identity)
  std::vector<rof::WorkItem> h_items;
  std::vector<rof::SplitRow> h_split;
  std::vector<int32_t> h_col;
};

namespace rof {

void set_error(const std::string& msg);
const std::string& last_error();
int cuda_fail(cudaError_t e, const char* what);

// Host-side description of a plan before upload (produced by the three layout readers).
struct HostPlan {
  int num_nodes = 0, row_begin = 0, row_end = 0;
  // destination-major entries of the rows in [row_begin,row_end): row r owns
  // entries [row_ptr[r-row_begin], row_ptr[r-row_begin+1])
  std::vector<int64_t> row_ptr;
  std::vector<int32_t> col;           // < num_nodes: feature row; >= num_nodes: partial row (col - num_nodes)
  std::vector<int32_t> group_ptr;     // [G+1] into group_col
  std::vector<int32_t> group_col;     // sources of each group
  std::vector<int32_t> group_orig;    // optional: id of each group in the plan this one was split from
  int64_t original_edges = 0;
};

int finalize_plan(HostPlan& hp, rof_plan** out, cudaStream_t stream);
double reuse_min_saving();

// Optional fused epilogue of a final output row: out = act(result + self_scale * self_x[row] + bias)
struct Epilogue {
  const float* bias;     // [dim] or null
  const float* self_x;   // [num_nodes, ld_self] rows addressed by global row id, or null
  int64_t ld_self;
  float self_scale;
  int relu;
};

struct GatherArgs {
  const WorkItem* items;
  int num_items;
  const int32_t* col;
  const float* x;        int64_t ldx;        // feature rows (col < num_nodes)
  const float* partials; int64_t ldp;        // partial rows (col >= num_nodes); may be null in phase A
  const float* degrees;
  float* out;            int64_t ldo;        // dst >= 0
  float* slots;          int64_t lds;        // dst < 0
  float* mirror;         int64_t ldm;        // optional second copy of the dst>=0 rows
  int mirror_flag_col;                       // column of `mirror` that receives 1.0f per row, or -1
  const int32_t* mirror_ids;                 // optional: row of `mirror` for each dst (null: dst itself)
  int num_nodes;
  int row_begin;
  int dim;
  int weight_gcn;   // multiply each feature row by rsqrt(degrees[col])
  int scale_mode;   // 0 none, 1 rsqrt(degrees[dst]), 2 1/degrees[dst]
  int accumulate;   // dst >= 0 rows: out += result instead of out = result
  int out_vec;      // set by launch_gather: `out` rows allow stores as wide as the loads
  int out_padded;   // `out` is library scratch with a padded leading dimension: a ragged last vector is stored whole
  int kernel;       // host policy: 0 lane groups, 1 shared-memory ring (used when the buffers allow it)
  int entries_per_item;  // average entries of the launch's items (0: unknown); very short items get narrower lane groups
  // split rows finished by their last-arriving segment (all null: split_reduce_kernel does it)
  const int32_t* slot_owner;
  const SplitRow* split;
  int32_t* arrive;
  int* status;      // plan status word (see rof_plan::h_status), may be null
  Epilogue ep;      // applied to dst >= 0 rows after scaling (and accumulating)
};

struct ReduceArgs {
  const SplitRow* rows;
  int num_rows;
  const float* slots; int64_t lds;
  const float* degrees;
  float* out;         int64_t ldo;
  int row_begin;
  int dim;
  int scale_mode;
  int accumulate;
  Epilogue ep;
};

struct TileArgs {
  const TileDesc* tiles;
  const WorkItem* titems;
  const int32_t* tcol;
  const int32_t* stage_col;
  int num_tiles;
};

// Launchers (kernels.cu).  Return cudaSuccess or the launch error.
// launch_gather_tiles: the tiled rows of a plan (GatherArgs::items / num_items are ignored);
// tiles_supported says whether the buffers and the width allow it.
bool tiles_supported(const GatherArgs& a);
cudaError_t launch_gather_tiles(const GatherArgs& a, const TileArgs& t, cudaStream_t stream, int* launches);
// launch_gather adds the number of kernels it launched to *launches (may be null).
cudaError_t launch_gather(const GatherArgs& a, cudaStream_t stream, int* launches);
// whether launch_gather(a) finishes the split rows itself (arrival counters) so that no
// split-reduce launch is needed afterwards
bool gather_fuses_reduce(const GatherArgs& a);
cudaError_t launch_split_reduce(const ReduceArgs& a, cudaStream_t stream);
cudaError_t launch_scale_rows(const float* x, int64_t ldx, const float* degrees, float* out, int64_t ldo,
                              int num_rows, int dim, int pad_to, int op, cudaStream_t stream);
cudaError_t launch_probe_read(const void* buf, int64_t bytes, int repeats, float* sink, cudaStream_t stream);

}  // namespace rof
