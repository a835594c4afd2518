// The per-call entry points of the C ABI: argument checks, workspace carving, launches.
#include <algorithm>
#include <cstdlib>
#include <cstring>

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
// ROF_FUSE_REDUCE=0: always combine the segment sums of split rows with a separate launch
inline bool fuse_reduce_enabled() {
  static const bool v = [] {
    const char* e = std::getenv("ROF_FUSE_REDUCE");
    return e == nullptr || std::string(e) != "0";
  }();
  return v;
}

// Host policy for the gather kernels (see kernels.cu): the lane-group kernel (0).  The shared-memory
// ring kernel (1) measured about half as fast on B200 at every width tried (one bulk copy per row of
// at most a few KB does not keep the copy engine busy) and only runs on request (ROF_KERNEL=ring).
constexpr int kDefaultGatherKernel = 0;

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
  if (mode == ROF_MODE_GCN_PRESCALED) b += 4 * rows_out;
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
  if (mode != ROF_MODE_GCN && mode != ROF_MODE_SUM && mode != ROF_MODE_MEAN && mode != ROF_MODE_GCN_PRESCALED) { set_error("rof_aggregate: unknown mode"); return ROF_ERR_BAD_ARGUMENT; }
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
  const int32_t* slot_owner = fine ? p->fine.d_slot_owner : p->d_slot_owner;
  int32_t* arrive = fine ? p->fine.d_arrive : p->d_arrive;

  if (p->device < 0) { set_error("rof_aggregate: the plan was built without a CUDA device and cannot run"); return ROF_ERR_CUDA; }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev != p->device) { set_error("rof_aggregate: plan was built on another device"); return ROF_ERR_BAD_ARGUMENT; }
  if (p->h_status != nullptr && *reinterpret_cast<volatile int*>(p->h_status) != 0) {
    *p->h_status = 0;
    set_error("rof_aggregate: a bounded wait inside an earlier pass on this plan ran out; that pass's output is incomplete");
    return ROF_ERR_WAIT_LIMIT;
  }

  const int gcn = (mode == ROF_MODE_GCN);
  const int scale_mode = (gcn || mode == ROF_MODE_GCN_PRESCALED) ? 1 : (mode == ROF_MODE_MEAN ? 2 : 0);
  bool reduce_done = false;

  if (p->num_groups > 0 && (phases & ROF_PHASE_PARTIALS)) {  // phase A: one partial row per reuse group
    GatherArgs a{};
    a.items = p->d_group_items; a.num_items = p->num_groups; a.col = p->d_col;
    a.x = x; a.ldx = ldx; a.partials = nullptr; a.ldp = 0; a.degrees = degrees;
    a.out = partials; a.ldo = w.ld; a.slots = nullptr; a.lds = 0;
    a.mirror = cache_result; a.ldm = (int64_t)dim + 1; a.mirror_flag_col = cache_result ? dim : -1;
    a.mirror_ids = p->d_group_orig;
    a.num_nodes = p->num_nodes; a.row_begin = 0; a.dim = dim; a.weight_gcn = gcn; a.scale_mode = 0;
    a.out_padded = 1; a.kernel = kDefaultGatherKernel; a.status = p->d_status;
    a.entries_per_item = (int)std::min<int64_t>(p->group_sources / std::max(1, p->num_groups), 1 << 20);
    e = launch_gather(a, stream, &g_last_launches);
    if (e != cudaSuccess) return cuda_fail(e, "phase A (group partial sums)");
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
    a.kernel = kDefaultGatherKernel; a.status = p->d_status;
    a.entries_per_item = (int)std::min<int64_t>(p->gather_entries / std::max(1, num_items), 1 << 20);
    // short rows that share entries: staged once per tile in shared memory; the other items
    // (long rows, segments of split rows) follow with the lane-group kernel
    const bool tiled = p->tiled.num_tiles > 0 && tiles_supported(a);
    if (tiled) {
      TileArgs t{p->tiled.d_tiles, p->tiled.d_titems, p->tiled.d_tcol, p->tiled.d_stage_col, p->tiled.num_tiles};
      e = launch_gather_tiles(a, t, stream, &g_last_launches);
      if (e != cudaSuccess) return cuda_fail(e, "phase B (shared-memory tiles)");
      a.items = fine ? p->tiled.d_rest_items_fine : p->tiled.d_rest_items;
      a.num_items = fine ? p->tiled.num_rest_fine : p->tiled.num_rest;
      a.kernel = kDefaultGatherKernel;
      a.entries_per_item = 0;   // what the tiles left: long rows and segments
    }
    // when the caller wants the whole pass, the last segment of a split row to arrive finishes it
    if (num_split > 0 && (phases & ROF_PHASE_REDUCE) && fuse_reduce_enabled()) {
      a.slot_owner = slot_owner; a.split = split; a.arrive = arrive;
      reduce_done = gather_fuses_reduce(a);
      if (!reduce_done) a.arrive = nullptr;
    }
    e = launch_gather(a, stream, &g_last_launches);
    if (e != cudaSuccess) return cuda_fail(e, "phase B (destination gather)");
  }
  if (num_split > 0 && (phases & ROF_PHASE_REDUCE) && !reduce_done) {
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

int rof_scale_rows(const float* x, int64_t ldx, int dim, const float* degrees, int op, float* out, int64_t ldo,
                   int64_t num_rows, void* stream_) {
  if (num_rows < 0 || num_rows > 0x7fffffffLL || dim < 0 || ldx < dim || ldo < dim || op < 0 || op > 2) {
    set_error("rof_scale_rows: sizes out of order or unknown op");
    return ROF_ERR_BAD_ARGUMENT;
  }
  if (num_rows == 0 || dim == 0) return ROF_OK;
  if (x == nullptr || out == nullptr || (op != ROF_SCALE_COPY && degrees == nullptr)) {
    set_error("rof_scale_rows: null pointer");
    return ROF_ERR_BAD_ARGUMENT;
  }
  // the padding columns up to the next multiple of 4 floats are zeroed when the row has room for them
  const int pad_to = (int)std::min<int64_t>(round_up(dim, 4), ldo);
  const cudaError_t e = launch_scale_rows(x, ldx, degrees, out, ldo, (int)num_rows, dim, pad_to, op, (cudaStream_t)stream_);
  return e == cudaSuccess ? ROF_OK : cuda_fail(e, "rof_scale_rows");
}

int rof_copy_async(void* dst, const void* src, int64_t bytes, void* stream_) {
  if (bytes < 0 || (bytes > 0 && (dst == nullptr || src == nullptr))) {
    set_error("rof_copy_async: null pointer or negative size");
    return ROF_ERR_BAD_ARGUMENT;
  }
  if (bytes == 0) return ROF_OK;
  const cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDefault, (cudaStream_t)stream_);
  return e == cudaSuccess ? ROF_OK : cuda_fail(e, "rof_copy_async");
}

static_assert(sizeof(cudaIpcMemHandle_t) == ROF_SHARED_HANDLE_BYTES, "interprocess handle size");

int rof_shared_alloc(int64_t bytes, void** ptr, unsigned char* handle) {
  if (bytes <= 0 || ptr == nullptr || handle == nullptr) {
    set_error("rof_shared_alloc: bad argument");
    return ROF_ERR_BAD_ARGUMENT;
  }
  *ptr = nullptr;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) { cudaGetLastError(); set_error("rof_shared_alloc: out of device memory"); return ROF_ERR_NO_MEMORY; }
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) { cudaFree(p); return cuda_fail(e, "cudaIpcGetMemHandle"); }
  std::memcpy(handle, &h, sizeof(h));
  *ptr = p;
  return ROF_OK;
}

int rof_shared_open(const unsigned char* handle, void** ptr) {
  if (handle == nullptr || ptr == nullptr) { set_error("rof_shared_open: null pointer"); return ROF_ERR_BAD_ARGUMENT; }
  *ptr = nullptr;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  const cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? ROF_OK : cuda_fail(e, "cudaIpcOpenMemHandle");
}

int rof_shared_close(void* ptr) {
  if (ptr == nullptr) return ROF_OK;
  const cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? ROF_OK : cuda_fail(e, "cudaIpcCloseMemHandle");
}

int rof_shared_free(void* ptr) {
  if (ptr == nullptr) return ROF_OK;
  const cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? ROF_OK : cuda_fail(e, "cudaFree");
}

int rof_probe_read(const void* buffer, int64_t bytes, int repeats, float* sink, void* stream_) {
  if (buffer == nullptr || sink == nullptr || bytes < 0 || repeats < 0 || (reinterpret_cast<uintptr_t>(buffer) & 15)) {
    set_error("rof_probe_read: null or misaligned buffer");
    return ROF_ERR_BAD_ARGUMENT;
  }
  const cudaError_t e = launch_probe_read(buffer, bytes, repeats, sink, (cudaStream_t)stream_);
  return e == cudaSuccess ? ROF_OK : cuda_fail(e, "rof_probe_read");
}

int rof_plan_take_status(rof_plan* p) {
  if (p == nullptr || p->h_status == nullptr) return 0;
  const int v = *reinterpret_cast<volatile int*>(p->h_status);
  *p->h_status = 0;
  return v;
}

int rof_last_launch_count(void) { return g_last_launches; }

const char* rof_last_error(void) { return rof::last_error().c_str(); }

int rof_version(void) { return 100; }

int rof_compiled_arch(void) { return 100; }

}  // extern "C"
