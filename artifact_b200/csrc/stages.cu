// Splits a plan into per-stage plans: stage k only names feature rows that are readable in stage
// k — for the multi-GPU pipeline (a peer's block has arrived) and for source tiling (one L2-sized
// block of source rows at a time); see rof_plan_create_stages* in rof_b200.h.
#include <algorithm>
#include <memory>

#include "rof_internal.h"

using namespace rof;

namespace {

// row_stage[c] = stage in which feature row c becomes readable
int split_by_row_stage(const rof_plan* whole, const std::vector<int32_t>& row_stage, int num_stages,
                       rof_plan** stages_out, cudaStream_t stream) {
  const int n = whole->num_nodes;
  const int rows = whole->row_end - whole->row_begin;
  const int G = whole->num_groups;
  try {
    std::vector<int32_t> col((size_t)whole->gather_entries), gcol((size_t)whole->group_sources);
    int rc = rof_plan_export(whole, nullptr, col.data(), nullptr, gcol.data(), nullptr, nullptr);
    if (rc) return rc;
    const std::vector<int64_t>& row_ptr = whole->h_row_ptr;
    const std::vector<int32_t>& gptr = whole->h_group_ptr;
    auto stage_of = [&](int32_t c) { return row_stage[(size_t)c]; };
    std::vector<int32_t> gstage((size_t)G, 0), glocal((size_t)G, 0);
    std::vector<HostPlan> hp((size_t)num_stages);
    for (int s = 0; s < num_stages; ++s) {
      hp[s].num_nodes = n; hp[s].row_begin = whole->row_begin; hp[s].row_end = whole->row_end;
      hp[s].row_ptr.assign((size_t)rows + 1, 0);
      hp[s].group_ptr.assign(1, 0);
    }
    for (int g = 0; g < G; ++g) {
      int st = 0;
      for (int32_t k = gptr[g]; k < gptr[g + 1]; ++k) st = std::max(st, (int)stage_of(gcol[(size_t)k]));
      gstage[g] = st;
      glocal[g] = (int32_t)hp[st].group_ptr.size() - 1;
      hp[st].group_orig.push_back(whole->h_group_orig.empty() ? g : whole->h_group_orig[(size_t)g]);
      hp[st].group_col.insert(hp[st].group_col.end(), gcol.begin() + gptr[g], gcol.begin() + gptr[g + 1]);
      hp[st].group_ptr.push_back((int32_t)hp[st].group_col.size());
    }
    for (int r = 0; r < rows; ++r)
      for (int64_t k = row_ptr[r]; k < row_ptr[r + 1]; ++k) {
        const int32_t c = col[(size_t)k];
        const int st = c >= n ? gstage[c - n] : stage_of(c);
        hp[st].row_ptr[(size_t)r + 1]++;
        hp[st].original_edges += c >= n ? gptr[c - n + 1] - gptr[c - n] : 1;
      }
    std::vector<std::vector<int64_t>> pos((size_t)num_stages);
    for (int s = 0; s < num_stages; ++s) {
      for (int r = 0; r < rows; ++r) hp[s].row_ptr[(size_t)r + 1] += hp[s].row_ptr[(size_t)r];
      hp[s].col.resize((size_t)hp[s].row_ptr[(size_t)rows]);
      pos[s].assign(hp[s].row_ptr.begin(), hp[s].row_ptr.end() - 1);
    }
    for (int r = 0; r < rows; ++r)
      for (int64_t k = row_ptr[r]; k < row_ptr[r + 1]; ++k) {
        const int32_t c = col[(size_t)k];
        if (c >= n) {
          const int st = gstage[c - n];
          hp[st].col[(size_t)pos[st][(size_t)r]++] = n + glocal[c - n];
        } else {
          const int st = stage_of(c);
          hp[st].col[(size_t)pos[st][(size_t)r]++] = c;
        }
      }
    col.clear(); col.shrink_to_fit();
    for (int s = 0; s < num_stages; ++s) {
      rc = finalize_plan(hp[s], &stages_out[s], stream);
      if (rc) {
        for (int t = 0; t < s; ++t) { rof_plan_destroy(stages_out[t]); stages_out[t] = nullptr; }
        return rc;
      }
      hp[s] = HostPlan();
    }
  } catch (const std::bad_alloc&) {
    set_error("out of host memory while staging the plan");
    return ROF_ERR_NO_MEMORY;
  }
  return ROF_OK;
}

}  // namespace

extern "C" int rof_plan_create_stages(const rof_plan* whole, int block_rows, const int32_t* stage_of_block,
                                      int num_blocks, int num_stages, rof_plan** stages_out, void* stream_) {
  if (!whole || !stage_of_block || !stages_out || block_rows <= 0 || num_blocks <= 0 || num_stages <= 0) {
    set_error("rof_plan_create_stages: bad argument");
    return ROF_ERR_BAD_ARGUMENT;
  }
  for (int s = 0; s < num_stages; ++s) stages_out[s] = nullptr;
  const int n = whole->num_nodes;
  if ((int64_t)block_rows * num_blocks < n) {
    set_error("rof_plan_create_stages: blocks do not cover every feature row");
    return ROF_ERR_BAD_ARGUMENT;
  }
  for (int b = 0; b < num_blocks; ++b)
    if (stage_of_block[b] < 0 || stage_of_block[b] >= num_stages) {
      set_error("rof_plan_create_stages: stage_of_block entry outside [0, num_stages)");
      return ROF_ERR_BAD_ARGUMENT;
    }
  std::vector<int32_t> row_stage;
  try {
    row_stage.resize((size_t)n);
  } catch (const std::bad_alloc&) {
    set_error("out of host memory while staging the plan");
    return ROF_ERR_NO_MEMORY;
  }
  for (int c = 0; c < n; ++c) row_stage[(size_t)c] = stage_of_block[c / block_rows];
  return split_by_row_stage(whole, row_stage, num_stages, stages_out, (cudaStream_t)stream_);
}

extern "C" int rof_plan_create_stages_ranges(const rof_plan* whole, const int32_t* range_bounds,
                                             const int32_t* stage_of_range, int num_ranges, int num_stages,
                                             rof_plan** stages_out, void* stream_) {
  if (!whole || !range_bounds || !stage_of_range || !stages_out || num_ranges <= 0 || num_stages <= 0) {
    set_error("rof_plan_create_stages_ranges: bad argument");
    return ROF_ERR_BAD_ARGUMENT;
  }
  for (int s = 0; s < num_stages; ++s) stages_out[s] = nullptr;
  const int n = whole->num_nodes;
  if (range_bounds[0] != 0 || range_bounds[num_ranges] != n) {
    set_error("rof_plan_create_stages_ranges: the ranges must cover [0, num_nodes)");
    return ROF_ERR_BAD_ARGUMENT;
  }
  for (int r = 0; r < num_ranges; ++r) {
    if (range_bounds[r + 1] < range_bounds[r]) {
      set_error("rof_plan_create_stages_ranges: range bounds must be ascending");
      return ROF_ERR_BAD_ARGUMENT;
    }
    if (stage_of_range[r] < 0 || stage_of_range[r] >= num_stages) {
      set_error("rof_plan_create_stages_ranges: stage_of_range entry outside [0, num_stages)");
      return ROF_ERR_BAD_ARGUMENT;
    }
  }
  std::vector<int32_t> row_stage;
  try {
    row_stage.resize((size_t)n);
  } catch (const std::bad_alloc&) {
    set_error("out of host memory while staging the plan");
    return ROF_ERR_NO_MEMORY;
  }
  for (int r = 0; r < num_ranges; ++r)
    for (int c = range_bounds[r]; c < range_bounds[r + 1]; ++c) row_stage[(size_t)c] = stage_of_range[r];
  return split_by_row_stage(whole, row_stage, num_stages, stages_out, (cudaStream_t)stream_);
}
