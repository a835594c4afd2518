// The per-call entry points of the C ABI: argument checks, workspace carving, launches.
#include "rof_internal.h"

namespace {

thread_local int g_last_launches = 0;

inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// leading dimension of the library's own scratch rows: a multiple of 4 floats so that
// 128-bit loads of partial rows stay aligned whatever the feature width
inline int64_t scratch_ld(int dim) { return round_up(dim, 4); }

struct Workspace {
  int64_t ld;
  int64_t partial_bytes;
  int64_t slot_bytes;
  int64_t total;
};

// narrow rows run on the plan's finer cut (more, shorter work items)
inline bool use_fine_cut(const rof_plan* p, int dim) { return p->fine.num_items > 0 && dim <= rof::kNarrowRowFloats; }

Workspace workspace_for(const rof_plan* p, int dim) {
  Workspace w;
  w.ld = scratch_ld(dim);
  w.partial_bytes = round_up((int64_t)p->num_groups * w.ld * 4, 256);
  w.slot_bytes = round_up((int64_t)(use_fine_cut(p, dim) ? p->fine.num_slots : p->num_slots) * w.ld * 4, 256);
  w.total = w.partial_bytes + w.slot_bytes;
  return w;
}

}  // namespace

using namespace rof;

extern "C" {

int64_t rof_plan_workspace_bytes(const rof_plan* plan, int dim) {
  if (plan == nullptr || dim < 0) return -1;
  return workspace_for(plan, dim).total;
}

int64_t rof_plan_algorithmic_bytes(const rof_plan* p, int dim, int mode) {
  if (p == nullptr || dim < 0) return -1;
  const int64_t rows_out = (int64_t)p->row_end - p->row_begin;
  const int64_t row_bytes = 4LL * dim;
  int64_t b = 0;
  // phase B: gathered rows (partials + residual sources), one written row per destination,
  // one index per entry, one work-item pointer pair per destination
  b += row_bytes * (p->gather_entries + rows_out) + 4 * p->gather_entries + 4 * (rows_out + 1);
  // phase A: group sources in, one partial row out, indices, pointers
  if (p->num_groups > 0) b += row_bytes * (p->group_sources + p->num_groups) + 4 * p->group_sources + 4 * ((int64_t)p->num_groups + 1);
  if (mode == ROF_MODE_GCN) b += 4 * (p->gather_entries - p->partial_entries + p->group_sources);  // degree reads
  if (mode == ROF_MODE_MEAN) b += 4 * rows_out;
  return b;
}

int rof_aggregate(const rof_plan* p, int mode, const float* x, int64_t ldx, int dim,
                  const float* degrees, float* out, int64_t ldo, float* cache_result,
                  void* workspace, int64_t workspace_bytes, void* stream_) {
  return rof_aggregate_phases(p, ROF_PHASE_ALL, mode, x, ldx, dim, degrees, out, ldo, cache_result, workspace,
                              workspace_bytes, stream_);
}

int rof_aggregate_phases(const rof_plan* p, int phases, int mode, const float* x, int64_t ldx, int dim,
                         const float* degrees, float* out, int64_t ldo, float* cache_result,
                         void* workspace, int64_t workspace_bytes, void* stream_) {
  return rof_aggregate_fused(p, phases, mode, x, ldx, dim, degrees, out, ldo, cache_result, workspace, workspace_bytes,
                             nullptr, nullptr, 0, 0.0f, 0, stream_);
}

int rof_aggregate_fused(const rof_plan* p, int phases, int mode, const float* x, int64_t ldx, int dim,
                        const float* degrees, float* out, int64_t ldo, float* cache_result,
                        void* workspace, int64_t workspace_bytes, const float* bias, const float* self_x,
                        int64_t ld_self, float self_scale, int relu, void* stream_) {
  g_last_launches = 0;
  if (self_x != nullptr && ld_self < dim) { set_error("rof_aggregate_fused: ld_self < dim"); return ROF_ERR_BAD_ARGUMENT; }
  const Epilogue ep{bias, self_x, ld_self, self_scale, relu ? 1 : 0};
  if (phases & ~(ROF_PHASE_ALL | ROF_PHASE_ACCUMULATE)) { set_error("rof_aggregate_phases: unknown phase bit"); return ROF_ERR_BAD_ARGUMENT; }
  const int accumulate = (phases & ROF_PHASE_ACCUMULATE) ? 1 : 0;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (p == nullptr) { set_error("rof_aggregate: null plan"); return ROF_ERR_BAD_ARGUMENT; }
  if (mode != ROF_MODE_GCN && mode != ROF_MODE_SUM && mode != ROF_MODE_MEAN) { set_error("rof_aggregate: unknown mode"); return ROF_ERR_BAD_ARGUMENT; }
  if (dim < 0 || ldx < dim || ldo < dim) { set_error("rof_aggregate: dim/ldx/ldo out of order"); return ROF_ERR_BAD_ARGUMENT; }
  const int rows_out = p->row_end - p->row_begin;
  if (rows_out == 0 || dim == 0) return ROF_OK;
  if (out == nullptr) { set_error("rof_aggregate: null out"); return ROF_ERR_BAD_ARGUMENT; }
  if (x == nullptr && (p->gather_entries > 0 || p->group_sources > 0)) { set_error("rof_aggregate: null x"); return ROF_ERR_BAD_ARGUMENT; }
  if (degrees == nullptr && mode != ROF_MODE_SUM) { set_error("rof_aggregate: degrees required for this mode"); return ROF_ERR_BAD_ARGUMENT; }

  const Workspace w = workspace_for(p, dim);
  if (w.total > 0) {
    if (workspace == nullptr || workspace_bytes < w.total || (reinterpret_cast<uintptr_t>(workspace) & 255)) {
      set_error("rof_aggregate: workspace missing, not 256-byte aligned, or smaller than rof_plan_workspace_bytes()");
      return ROF_ERR_WORKSPACE;
    }
  }
  float* partials = p->num_groups ? reinterpret_cast<float*>(workspace) : nullptr;
  const bool fine = use_fine_cut(p, dim);
  const WorkItem* items = fine ? p->fine.d_items : p->d_items;
  const int num_items = fine ? p->fine.num_items : p->num_items;
  const SplitRow* split = fine ? p->fine.d_split : p->d_split;
  const int num_split = fine ? p->fine.num_split_rows : p->num_split_rows;
  const int num_slots = fine ? p->fine.num_slots : p->num_slots;
  float* slots = num_slots ? reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + w.partial_bytes) : nullptr;

  if (p->device < 0) { set_error("rof_aggregate: the plan was built without a CUDA device and cannot run"); return ROF_ERR_CUDA; }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev != p->device) { set_error("rof_aggregate: plan was built on another device"); return ROF_ERR_BAD_ARGUMENT; }

  const int gcn = (mode == ROF_MODE_GCN);
  const int scale_mode = gcn ? 1 : (mode == ROF_MODE_MEAN ? 2 : 0);

  if (p->num_groups > 0 && (phases & ROF_PHASE_PARTIALS)) {  // phase A: one partial row per reuse group
    GatherArgs a{};
    a.items = p->d_group_items; a.num_items = p->num_groups; a.col = p->d_col;
    a.x = x; a.ldx = ldx; a.partials = nullptr; a.ldp = 0; a.degrees = degrees;
    a.out = partials; a.ldo = w.ld; a.slots = nullptr; a.lds = 0;
    a.mirror = cache_result; a.ldm = (int64_t)dim + 1; a.mirror_flag_col = cache_result ? dim : -1;
    a.num_nodes = p->num_nodes; a.row_begin = 0; a.dim = dim; a.weight_gcn = gcn; a.scale_mode = 0;
    e = launch_gather(a, stream);
    if (e != cudaSuccess) return cuda_fail(e, "phase A (group partial sums)");
    g_last_launches += (dim + 2047) / 2048;
  }
  if (phases & ROF_PHASE_GATHER) {  // phase B: one pass over every destination row
    GatherArgs a{};
    a.items = items; a.num_items = num_items; a.col = p->d_col;
    a.x = x; a.ldx = ldx; a.partials = partials; a.ldp = w.ld; a.degrees = degrees;
    a.out = out; a.ldo = ldo; a.slots = slots; a.lds = w.ld;
    a.mirror = nullptr; a.ldm = 0; a.mirror_flag_col = -1;
    a.num_nodes = p->num_nodes; a.row_begin = p->row_begin; a.dim = dim; a.weight_gcn = gcn; a.scale_mode = scale_mode;
    a.accumulate = accumulate;
    a.ep = ep;
    e = launch_gather(a, stream);
    if (e != cudaSuccess) return cuda_fail(e, "phase B (destination gather)");
    g_last_launches += (dim + 2047) / 2048;
  }
  if (num_split > 0 && (phases & ROF_PHASE_REDUCE)) {
    ReduceArgs r{};
    r.rows = split; r.num_rows = num_split; r.slots = slots; r.lds = w.ld; r.degrees = degrees;
    r.out = out; r.ldo = ldo; r.row_begin = p->row_begin; r.dim = dim; r.scale_mode = scale_mode;
    r.accumulate = accumulate;
    r.ep = ep;
    e = launch_split_reduce(r, stream);
    if (e != cudaSuccess) return cuda_fail(e, "segment reduce");
    g_last_launches += 1;
  }
  return ROF_OK;
}

int rof_last_launch_count(void) { return g_last_launches; }

const char* rof_last_error(void) { return rof::last_error().c_str(); }

int rof_version(void) { return 100; }

int rof_compiled_arch(void) { return 100; }

}  // extern "C"
