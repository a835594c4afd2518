// Plan builder: turns upstream's three part-major index layouts into one destination-major
// work list.
//
// Upstream runs one warp per *part* and adds every part's sum into its destination row with
// atomics (reuse_conv_kernel.cu:230-285, 521-600, 879-953).  Here the same index tensors are
// transposed once, on the host, into rows of entries: an entry < N names a feature row, an
// entry >= N names the partial sum of reuse group (entry - N).  Rows longer than
// the segment length are cut into segments whose sums are combined by a second small kernel in a
// fixed order, so the result is deterministic.  Work items are ordered longest first so the
// hardware block scheduler balances the power-law tail.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <numeric>

#include "rof_internal.h"

namespace rof {

static thread_local std::string g_error = "";

void set_error(const std::string& msg) { g_error = msg; }

int cuda_fail(cudaError_t e, const char* what) {
  set_error(std::string(what) + ": " + cudaGetErrorString(e));
  return ROF_ERR_CUDA;
}

const std::string& last_error() { return g_error; }

namespace {

// Host view of an int32 index array that may live on the device.
struct HostArray {
  std::vector<int32_t> owned;
  const int32_t* ptr = nullptr;
  int64_t n = 0;
  int fetch(const int32_t* src, int64_t count, int where, cudaStream_t stream, const char* name) {
    n = count;
    if (count < 0) { set_error(std::string(name) + ": negative length"); return ROF_ERR_BAD_ARGUMENT; }
    if (count == 0) { ptr = nullptr; return ROF_OK; }
    if (src == nullptr) { set_error(std::string(name) + ": null pointer"); return ROF_ERR_BAD_ARGUMENT; }
    if (where == ROF_ON_HOST) { ptr = src; return ROF_OK; }
    try { owned.resize((size_t)count); } catch (...) { set_error("out of host memory"); return ROF_ERR_NO_MEMORY; }
    cudaError_t e = cudaMemcpyAsync(owned.data(), src, sizeof(int32_t) * (size_t)count, cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return cuda_fail(e, name);
    ptr = owned.data();
    return ROF_OK;
  }
};

int bad_layout(const std::string& msg) {
  set_error("bad layout: " + msg);
  return ROF_ERR_BAD_LAYOUT;
}

int check_common(rof_plan** plan, int where, int num_nodes, int row_begin, int row_end) {
  if (plan == nullptr) { set_error("plan: null output pointer"); return ROF_ERR_BAD_ARGUMENT; }
  *plan = nullptr;
  if (where != ROF_ON_HOST && where != ROF_ON_DEVICE) { set_error("where: unknown location"); return ROF_ERR_BAD_ARGUMENT; }
  if (num_nodes < 0 || row_begin < 0 || row_end < row_begin || row_end > num_nodes) {
    set_error("num_nodes / row range out of order");
    return ROF_ERR_BAD_ARGUMENT;
  }
  return ROF_OK;
}

// pointers[count+1] must be non-decreasing and stay inside [0, limit]
int check_pointers(const int32_t* p, int64_t count, int64_t limit, const char* name) {
  if (count == 0) return ROF_OK;
  for (int64_t i = 0; i <= count; ++i) {
    if (p[i] < 0 || p[i] > limit) return bad_layout(std::string(name) + " leaves its index array");
    if (i > 0 && p[i] < p[i - 1]) return bad_layout(std::string(name) + " is not non-decreasing");
  }
  return ROF_OK;
}

int check_ids(const int32_t* p, int64_t count, int64_t limit, const char* name) {
  for (int64_t i = 0; i < count; ++i)
    if (p[i] < 0 || p[i] >= limit) return bad_layout(std::string(name) + " holds an id outside [0, num_nodes)");
  return ROF_OK;
}

int sync_if_device(int where, cudaStream_t stream) {
  if (where != ROF_ON_DEVICE) return ROF_OK;
  cudaError_t e = cudaStreamSynchronize(stream);
  return e == cudaSuccess ? ROF_OK : cuda_fail(e, "copy of index tensors to the host");
}

}  // namespace

// ---------------------------------------------------------------------------------------
// shared-memory tiles
// ---------------------------------------------------------------------------------------
namespace {

struct HostTiles {
  std::vector<int32_t> tcol, stage_col;
  std::vector<WorkItem> titems;
  std::vector<TileDesc> tiles;
  int64_t entries = 0, shared_entries = 0, staged_rows = 0;
};

// The ids that occur at least twice among `ents`, most frequent first (ties: smaller id first),
// at most kTileMaxStage of them.  `sorted` is scratch.  Returns how many global row reads staging
// them saves: sum over kept ids of (occurrences - 1).
int64_t shared_ids_of_tile(const std::vector<int32_t>& ents, std::vector<int32_t>& sorted,
                           std::vector<std::pair<int32_t, int32_t>>& kept) {
  sorted = ents;
  std::sort(sorted.begin(), sorted.end());
  kept.clear();
  for (size_t i = 0; i < sorted.size();) {
    size_t j = i + 1;
    while (j < sorted.size() && sorted[j] == sorted[i]) ++j;
    if (j - i >= 2) kept.emplace_back((int32_t)(j - i), sorted[i]);   // (count, id)
    i = j;
  }
  std::sort(kept.begin(), kept.end(), [](const std::pair<int32_t, int32_t>& a, const std::pair<int32_t, int32_t>& b) {
    return a.first != b.first ? a.first > b.first : a.second < b.second;
  });
  if ((int)kept.size() > kTileMaxStage) kept.resize(kTileMaxStage);
  int64_t saved = 0;
  for (const auto& k : kept) saved += k.first - 1;
  return saved;
}

}  // namespace

// Smallest share of the gathered rows that reuse groups must save for a ROF_v2 plan to use them
// (ROF_REUSE_MIN overrides, e.g. 0 to always use the groups the search found).
double reuse_min_saving() {
  const char* e = std::getenv("ROF_REUSE_MIN");
  if (e != nullptr && e[0] != '\0') return std::atof(e);
  return kMinReuseSaving;
}

namespace {

// ROF_TILES=0 never builds tiles, ROF_TILES=1 always does (when there are eligible rows); unset:
// tiles are built when a sample of them saves at least kTileMinSaved of the global row reads.
int tiles_override() {
  const char* e = std::getenv("ROF_TILES");
  if (e == nullptr || e[0] == '\0') return -1;
  return e[0] == '0' ? 0 : 1;
}

// Groups the short rows of `hp`, in row order, into tiles and rewrites their entries.  Returns
// false (and leaves `out` empty) when tiling does not pay.
bool build_tiles(const HostPlan& hp, HostTiles& out) {
  const int rows = hp.row_end - hp.row_begin;
  const int ov = tiles_override();
  if (ov == 0 || rows == 0) return false;
  std::vector<int32_t> elig;
  elig.reserve((size_t)rows);
  int64_t elig_entries = 0;
  for (int r = 0; r < rows; ++r) {
    const int64_t len = hp.row_ptr[r + 1] - hp.row_ptr[r];
    if (len <= kTileMaxRowEntries) { elig.push_back(r); elig_entries += len; }
  }
  if (elig.empty() || elig_entries == 0) return false;
  const int num_tiles = (int)((elig.size() + kTileRows - 1) / kTileRows);
  auto tile_entries = [&](int t, std::vector<int32_t>& ents) {
    ents.clear();
    const size_t e0 = (size_t)t * kTileRows, e1 = std::min(elig.size(), e0 + kTileRows);
    for (size_t k = e0; k < e1; ++k) {
      const int r = elig[k];
      ents.insert(ents.end(), hp.col.begin() + hp.row_ptr[r], hp.col.begin() + hp.row_ptr[r + 1]);
    }
  };
  if (ov < 0) {   // sample up to 256 tiles, evenly spread
    std::vector<int32_t> ents, sorted;
    std::vector<std::pair<int32_t, int32_t>> kept;
    const int step = std::max(1, num_tiles / 256);
    int64_t saved = 0, total = 0;
    for (int t = 0; t < num_tiles; t += step) {
      tile_entries(t, ents);
      saved += shared_ids_of_tile(ents, sorted, kept);
      total += (int64_t)ents.size();
    }
    if (total == 0 || (double)saved < kTileMinSaved * (double)total) return false;
  }

  std::vector<int64_t> tptr(elig.size() + 1, 0);   // entry offsets of the tiled rows
  for (size_t k = 0; k < elig.size(); ++k) tptr[k + 1] = tptr[k] + (hp.row_ptr[elig[k] + 1] - hp.row_ptr[elig[k]]);
  out.entries = elig_entries;
  out.tcol.resize((size_t)elig_entries);
  out.titems.resize(elig.size());
  out.tiles.resize((size_t)num_tiles);
  out.stage_col.assign((size_t)num_tiles * kTileMaxStage, 0);
  int64_t shared_total = 0, staged_total = 0;
#pragma omp parallel reduction(+ : shared_total, staged_total)
  {
    std::vector<int32_t> ents, sorted;
    std::vector<std::pair<int32_t, int32_t>> kept, by_id;
#pragma omp for schedule(dynamic, 64)
    for (int t = 0; t < num_tiles; ++t) {
      tile_entries(t, ents);
      shared_ids_of_tile(ents, sorted, kept);
      by_id.clear();
      for (int sidx = 0; sidx < (int)kept.size(); ++sidx) {
        out.stage_col[(size_t)t * kTileMaxStage + sidx] = kept[sidx].second;
        by_id.emplace_back(kept[sidx].second, sidx);   // (id, slot)
      }
      std::sort(by_id.begin(), by_id.end());
      auto slot_of = [&](int32_t c) {
        auto it = std::lower_bound(by_id.begin(), by_id.end(), std::make_pair(c, (int32_t)-1));
        return (it != by_id.end() && it->first == c) ? it->second : -1;
      };
      const size_t e0 = (size_t)t * kTileRows, e1 = std::min(elig.size(), e0 + kTileRows);
      out.tiles[(size_t)t] = TileDesc{(int32_t)e0, (int32_t)(e1 - e0), (int32_t)(t * kTileMaxStage), (int32_t)kept.size()};
      staged_total += (int64_t)kept.size();
      for (size_t k = e0; k < e1; ++k) {
        const int r = elig[k];
        int64_t w = tptr[k];
        for (int64_t q = hp.row_ptr[r]; q < hp.row_ptr[r + 1]; ++q) {   // staged slots first ...
          const int sl = slot_of(hp.col[(size_t)q]);
          if (sl >= 0) out.tcol[(size_t)w++] = sl;
        }
        const int64_t mid = w;
        for (int64_t q = hp.row_ptr[r]; q < hp.row_ptr[r + 1]; ++q)     // ... then the rows read from global memory
          if (slot_of(hp.col[(size_t)q]) < 0) out.tcol[(size_t)w++] = hp.col[(size_t)q];
        shared_total += mid - tptr[k];
        out.titems[k] = WorkItem{(int32_t)tptr[k], (int32_t)tptr[k + 1], hp.row_begin + r, (int32_t)mid};
      }
    }
  }
  out.shared_entries = shared_total;
  out.staged_rows = staged_total;
  return true;
}

}  // namespace

// ---------------------------------------------------------------------------------------
// finalize: row lists -> sorted work items -> device
// ---------------------------------------------------------------------------------------
static int finalize_plan_impl(HostPlan& hp, rof_plan** out, cudaStream_t stream);

int finalize_plan(HostPlan& hp, rof_plan** out, cudaStream_t stream) {
  try {
    return finalize_plan_impl(hp, out, stream);
  } catch (const std::bad_alloc&) {  // never let an exception cross the C ABI
    set_error("out of host memory while building the plan");
    return ROF_ERR_NO_MEMORY;
  }
}

static int finalize_plan_impl(HostPlan& hp, rof_plan** out, cudaStream_t stream) {
  const int rows = hp.row_end - hp.row_begin;
  const int64_t entries = (int64_t)hp.col.size();
  const int64_t gsrc = (int64_t)hp.group_col.size();
  const int groups = (int)hp.group_ptr.size() - 1;
  if (entries + gsrc >= (int64_t)INT32_MAX) {
    set_error("more than 2^31-1 gather entries in one plan; shard the rows");
    return ROF_ERR_BAD_ARGUMENT;
  }

  std::unique_ptr<rof_plan> p(new rof_plan());
  cudaError_t e = cudaGetDevice(&p->device);
  if (e != cudaSuccess) {
    // No usable device: keep the plan on the host so that it can still be inspected with
    // rof_plan_export(); rof_aggregate() refuses such a plan.
    (void)cudaGetLastError();
    p->device = -1;
  }
  p->num_nodes = hp.num_nodes;
  p->row_begin = hp.row_begin;
  p->row_end = hp.row_end;
  p->num_groups = groups < 0 ? 0 : groups;
  p->group_sources = gsrc;
  p->gather_entries = entries;
  p->original_edges = hp.original_edges;
  // Every row lists its partial rows first, then its feature rows (the order the v1 / v2
  // layouts already produce), so the kernel walks two ranges with one base pointer each.
  std::vector<int64_t> row_mid((size_t)rows);
  const int32_t n_nodes = hp.num_nodes;
#pragma omp parallel for schedule(static, 1024)
  for (int r = 0; r < rows; ++r) {
    auto b = hp.col.begin() + hp.row_ptr[r], e = hp.col.begin() + hp.row_ptr[r + 1];
    auto m = std::stable_partition(b, e, [n_nodes](int32_t c) { return c >= n_nodes; });
    row_mid[(size_t)r] = m - hp.col.begin();
    // ascending ids inside each range: the reorganised layouts list a row's group sources first, and rows
    // that sweep the feature matrix in the same direction share more cache lines (114.6M-edge graph, D=256:
    // 11.9 ms per step in layout order, 11.4 ms sorted)
    std::sort(b, m);
    std::sort(m, e);
  }
  for (int r = 0; r < rows; ++r) p->partial_entries += row_mid[(size_t)r] - hp.row_ptr[r];

  // rows ordered by length, longest first (stable: equal lengths keep ascending row id)
  std::vector<int32_t> order((size_t)rows);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) {
    return (hp.row_ptr[a + 1] - hp.row_ptr[a]) > (hp.row_ptr[b + 1] - hp.row_ptr[b]);
  });

  // Segment length.  Long segments are cheaper (fewer segment sums to store and re-read, less
  // per-item overhead: on the 114.6M-edge graph 8192-entry segments beat 256-entry ones by 18 %
  // at width 256), but too few of them leave SMs idle at the end (one eighth of that graph:
  // 0.95 ms with 1024, 1.5 ms with 4096).  The sweet spot is a few segments per resident lane
  // group — ~16k for wide rows (one group per warp on 148 SMs x 32 warps), four times as many
  // for rows of at most 32 floats (4 or 8 groups per warp: 0.96 ms vs 1.20 ms there) — so the
  // plan carries two cuts of the same rows and rof_aggregate() picks by feature width.
  auto segment_length = [&](double target) {
    int seg = kMinSegmentEdges;
    while (seg < kMaxSegmentEdges && (double)entries / target > 1.4142 * seg) seg *= 2;
    return seg;
  };
  auto cut = [&](int seg, std::vector<WorkItem>& items, std::vector<SplitRow>& split) {
    items.clear(); split.clear();
    items.reserve((size_t)rows + (size_t)(entries / seg) + 1);
    int slots = 0;
    for (int32_t r : order) {
      const int64_t b = hp.row_ptr[r], en = hp.row_ptr[r + 1];
      const int64_t len = en - b;
      if (len <= seg) {
        items.push_back(WorkItem{(int32_t)b, (int32_t)en, hp.row_begin + r, (int32_t)row_mid[(size_t)r]});
      } else {
        const int nseg = (int)((len + seg - 1) / seg);
        split.push_back(SplitRow{hp.row_begin + r, slots, nseg, 0});
        for (int s = 0; s < nseg; ++s) {
          const int64_t sb = b + (int64_t)s * seg;
          const int64_t se = std::min(en, sb + seg);
          const int64_t sm = std::min(se, std::max(sb, row_mid[(size_t)r]));
          items.push_back(WorkItem{(int32_t)sb, (int32_t)se, -(slots + s) - 1, (int32_t)sm});
        }
        slots += nseg;
      }
    }
    // full segments first, then everything else by length (split rows' short tails included)
    std::stable_sort(items.begin(), items.end(),
                     [](const WorkItem& a, const WorkItem& b) { return (a.end - a.begin) > (b.end - b.begin); });
    return slots;
  };
  std::vector<WorkItem> items, fine_items;
  std::vector<SplitRow> split, fine_split;
  p->segment_edges = segment_length(kTargetSegments);
  p->num_slots = cut(p->segment_edges, items, split);
  p->num_items = (int)items.size();
  p->num_split_rows = (int)split.size();
  p->fine.segment_edges = segment_length(4.0 * kTargetSegments);
  if (p->fine.segment_edges != p->segment_edges) {
    p->fine.num_slots = cut(p->fine.segment_edges, fine_items, fine_split);
    p->fine.num_items = (int)fine_items.size();
    p->fine.num_split_rows = (int)fine_split.size();
  }

  std::vector<WorkItem> gitems((size_t)p->num_groups);
  for (int g = 0; g < p->num_groups; ++g)
    gitems[g] = WorkItem{(int32_t)(entries + hp.group_ptr[g]), (int32_t)(entries + hp.group_ptr[g + 1]), g,
                         (int32_t)(entries + hp.group_ptr[g])};

  // shared-memory tiles for the short rows, and the items each cut keeps for the lane-group kernel
  HostTiles ht;
  std::vector<WorkItem> rest, rest_fine;
  if (build_tiles(hp, ht)) {
    auto keep_rest = [](const std::vector<WorkItem>& all, std::vector<WorkItem>& out_items) {
      out_items.clear();
      for (const WorkItem& w : all)
        if (w.dst < 0 || w.end - w.begin > kTileMaxRowEntries) out_items.push_back(w);
    };
    keep_rest(items, rest);
    keep_rest(fine_items, rest_fine);
    p->tiled.num_tiles = (int)ht.tiles.size();
    p->tiled.num_items = (int)ht.titems.size();
    p->tiled.entries = ht.entries;
    p->tiled.shared_entries = ht.shared_entries;
    p->tiled.staged_rows = ht.staged_rows;
    p->tiled.num_rest = (int)rest.size();
    p->tiled.num_rest_fine = (int)rest_fine.size();
    p->tiled.h_tiles = ht.tiles;
    p->tiled.h_titems = ht.titems;
    p->tiled.h_tcol = ht.tcol;
    p->tiled.h_stage_col = ht.stage_col;
  }

  p->h_row_ptr = hp.row_ptr;
  p->h_group_ptr = hp.group_ptr;
  if ((int)hp.group_orig.size() == p->num_groups) p->h_group_orig = hp.group_orig;
  p->h_items = items;
  p->h_split = split;
  if (p->device < 0) {
    p->h_col = hp.col;
    p->h_col.insert(p->h_col.end(), hp.group_col.begin(), hp.group_col.end());
    *out = p.release();
    return ROF_OK;
  }

  auto upload = [&](void** dptr, const void* src, size_t bytes, const char* what) -> int {
    *dptr = nullptr;
    if (bytes == 0) return ROF_OK;
    cudaError_t err = cudaMalloc(dptr, bytes);
    if (err != cudaSuccess) return cuda_fail(err, what);
    err = cudaMemcpyAsync(*dptr, src, bytes, cudaMemcpyHostToDevice, stream);
    if (err != cudaSuccess) return cuda_fail(err, what);
    return ROF_OK;
  };
  int rc = ROF_OK;
  {
    size_t bytes = sizeof(int32_t) * (size_t)(entries + gsrc);
    if (bytes) {
      e = cudaMalloc((void**)&p->d_col, bytes);
      if (e != cudaSuccess) rc = cuda_fail(e, "cudaMalloc(col)");
      if (rc == ROF_OK && entries) {
        e = cudaMemcpyAsync(p->d_col, hp.col.data(), sizeof(int32_t) * (size_t)entries, cudaMemcpyHostToDevice, stream);
        if (e != cudaSuccess) rc = cuda_fail(e, "upload col");
      }
      if (rc == ROF_OK && gsrc) {
        e = cudaMemcpyAsync(p->d_col + entries, hp.group_col.data(), sizeof(int32_t) * (size_t)gsrc,
                            cudaMemcpyHostToDevice, stream);
        if (e != cudaSuccess) rc = cuda_fail(e, "upload group sources");
      }
    }
  }
  if (rc == ROF_OK) rc = upload((void**)&p->d_items, items.data(), sizeof(WorkItem) * items.size(), "upload work items");
  if (rc == ROF_OK) rc = upload((void**)&p->d_group_items, gitems.data(), sizeof(WorkItem) * gitems.size(), "upload group items");
  if (rc == ROF_OK) rc = upload((void**)&p->d_split, split.data(), sizeof(SplitRow) * split.size(), "upload split rows");
  if (rc == ROF_OK && (int)hp.group_orig.size() == p->num_groups)
    rc = upload((void**)&p->d_group_orig, hp.group_orig.data(), sizeof(int32_t) * hp.group_orig.size(), "upload group ids");
  if (rc == ROF_OK) rc = upload((void**)&p->fine.d_items, fine_items.data(), sizeof(WorkItem) * fine_items.size(), "upload work items (narrow rows)");
  if (rc == ROF_OK) rc = upload((void**)&p->fine.d_split, fine_split.data(), sizeof(SplitRow) * fine_split.size(), "upload split rows (narrow rows)");
  // which split row every scratch slot belongs to, and the rows' arrival counters (zero between passes)
  auto owners_of = [](const std::vector<SplitRow>& sp, int slots) {
    std::vector<int32_t> o((size_t)slots);
    for (size_t i = 0; i < sp.size(); ++i)
      for (int k = 0; k < sp[i].count; ++k) o[(size_t)sp[i].first_slot + k] = (int32_t)i;
    return o;
  };
  auto counters = [&](int32_t** dptr, size_t n) -> int {
    *dptr = nullptr;
    if (n == 0) return ROF_OK;
    cudaError_t err = cudaMalloc((void**)dptr, sizeof(int32_t) * n);
    if (err != cudaSuccess) return cuda_fail(err, "cudaMalloc(arrival counters)");
    err = cudaMemsetAsync(*dptr, 0, sizeof(int32_t) * n, stream);
    return err == cudaSuccess ? ROF_OK : cuda_fail(err, "clear arrival counters");
  };
  const std::vector<int32_t> owners = owners_of(split, p->num_slots), fine_owners = owners_of(fine_split, p->fine.num_slots);
  if (rc == ROF_OK) rc = upload((void**)&p->d_slot_owner, owners.data(), sizeof(int32_t) * owners.size(), "upload slot owners");
  if (rc == ROF_OK) rc = upload((void**)&p->fine.d_slot_owner, fine_owners.data(), sizeof(int32_t) * fine_owners.size(), "upload slot owners (narrow rows)");
  if (p->tiled.num_tiles > 0) {
    if (rc == ROF_OK) rc = upload((void**)&p->tiled.d_tcol, ht.tcol.data(), sizeof(int32_t) * ht.tcol.size(), "upload tile entries");
    if (rc == ROF_OK) rc = upload((void**)&p->tiled.d_titems, ht.titems.data(), sizeof(WorkItem) * ht.titems.size(), "upload tile items");
    if (rc == ROF_OK) rc = upload((void**)&p->tiled.d_tiles, ht.tiles.data(), sizeof(TileDesc) * ht.tiles.size(), "upload tiles");
    if (rc == ROF_OK) rc = upload((void**)&p->tiled.d_stage_col, ht.stage_col.data(), sizeof(int32_t) * ht.stage_col.size(), "upload tile stage lists");
    if (rc == ROF_OK) rc = upload((void**)&p->tiled.d_rest_items, rest.data(), sizeof(WorkItem) * rest.size(), "upload untiled items");
    if (rc == ROF_OK) rc = upload((void**)&p->tiled.d_rest_items_fine, rest_fine.data(), sizeof(WorkItem) * rest_fine.size(), "upload untiled items (narrow rows)");
  }
  if (rc == ROF_OK) rc = counters(&p->d_arrive, split.size());
  if (rc == ROF_OK) rc = counters(&p->fine.d_arrive, fine_split.size());
  if (rc == ROF_OK) {
    e = cudaHostAlloc((void**)&p->h_status, sizeof(int), cudaHostAllocMapped);
    if (e == cudaSuccess) {
      *p->h_status = 0;
      e = cudaHostGetDevicePointer((void**)&p->d_status, p->h_status, 0);
    }
    if (e != cudaSuccess) rc = cuda_fail(e, "status word");
  }
  if (rc == ROF_OK) {
    e = cudaStreamSynchronize(stream);  // the host vectors die at return
    if (e != cudaSuccess) rc = cuda_fail(e, "plan upload");
  }
  if (rc != ROF_OK) {
    rof_plan_destroy(p.release());
    return rc;
  }
  *out = p.release();
  return ROF_OK;
}

}  // namespace rof

using namespace rof;

extern "C" {

int rof_plan_create_parts(rof_plan** plan, int where, int num_nodes, int row_begin, int row_end,
                          const int32_t* column_index, int64_t num_column_index,
                          const int32_t* part_pointers, const int32_t* part2Node, int num_parts,
                          void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  int rc = check_common(plan, where, num_nodes, row_begin, row_end);
  if (rc) return rc;
  if (num_parts < 0) { set_error("num_parts < 0"); return ROF_ERR_BAD_ARGUMENT; }
  HostArray col, pp, p2n;
  if ((rc = col.fetch(column_index, num_column_index, where, stream, "column_index"))) return rc;
  if ((rc = pp.fetch(part_pointers, num_parts ? (int64_t)num_parts + 1 : 0, where, stream, "part_pointers"))) return rc;
  if ((rc = p2n.fetch(part2Node, num_parts, where, stream, "part2Node"))) return rc;
  if ((rc = sync_if_device(where, stream))) return rc;
  if ((rc = check_pointers(pp.ptr, num_parts, num_column_index, "part_pointers"))) return rc;
  if ((rc = check_ids(p2n.ptr, num_parts, num_nodes, "part2Node"))) return rc;
  if ((rc = check_ids(col.ptr, num_column_index, num_nodes, "column_index"))) return rc;

  HostPlan hp;
  hp.num_nodes = num_nodes; hp.row_begin = row_begin; hp.row_end = row_end;
  const int rows = row_end - row_begin;
  try {
    hp.row_ptr.assign((size_t)rows + 1, 0);
    for (int p = 0; p < num_parts; ++p) {
      int v = p2n.ptr[p];
      if (v >= row_begin && v < row_end) hp.row_ptr[(size_t)(v - row_begin) + 1] += pp.ptr[p + 1] - pp.ptr[p];
    }
    for (int r = 0; r < rows; ++r) hp.row_ptr[r + 1] += hp.row_ptr[r];
    hp.col.resize((size_t)hp.row_ptr[rows]);
    std::vector<int64_t> pos(hp.row_ptr.begin(), hp.row_ptr.end() - 1);
    for (int p = 0; p < num_parts; ++p) {
      int v = p2n.ptr[p];
      if (v < row_begin || v >= row_end) continue;
      int64_t& w = pos[(size_t)(v - row_begin)];
      for (int32_t k = pp.ptr[p]; k < pp.ptr[p + 1]; ++k) hp.col[(size_t)w++] = col.ptr[k];
    }
    hp.group_ptr.assign(1, 0);
    hp.original_edges = hp.row_ptr[rows];
  } catch (const std::bad_alloc&) {
    set_error("out of host memory while building the plan");
    return ROF_ERR_NO_MEMORY;
  }
  return finalize_plan(hp, plan, stream);
}

int rof_plan_create_v1(rof_plan** plan, int where, int num_nodes, int row_begin, int row_end,
                       const int32_t* column_index, int64_t num_column_index,
                       const int32_t* part_pointers, const int32_t* part2Node, int num_parts,
                       const int32_t* part_cache_flagindex, const int32_t* part_pointers_cache,
                       const int32_t* column_index_cache, int num_groups, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  int rc = check_common(plan, where, num_nodes, row_begin, row_end);
  if (rc) return rc;
  if (num_parts < 0 || num_groups < 0) { set_error("num_parts / num_groups < 0"); return ROF_ERR_BAD_ARGUMENT; }
  HostArray col, pp, p2n, flag, ppc, cic;
  if ((rc = col.fetch(column_index, num_column_index, where, stream, "column_index"))) return rc;
  if ((rc = pp.fetch(part_pointers, num_parts ? (int64_t)num_parts + 1 : 0, where, stream, "part_pointers"))) return rc;
  if ((rc = p2n.fetch(part2Node, num_parts, where, stream, "part2Node"))) return rc;
  if ((rc = flag.fetch(part_cache_flagindex, num_parts, where, stream, "part_cache_flagindex"))) return rc;
  if ((rc = ppc.fetch(part_pointers_cache, num_groups ? (int64_t)num_groups + 1 : 0, where, stream, "part_pointers_cache"))) return rc;
  if ((rc = sync_if_device(where, stream))) return rc;
  int64_t n_cic = num_groups ? ppc.ptr[num_groups] : 0;
  if (n_cic < 0) return bad_layout("part_pointers_cache ends below zero");
  if ((rc = cic.fetch(column_index_cache, n_cic, where, stream, "column_index_cache"))) return rc;
  if ((rc = sync_if_device(where, stream))) return rc;
  if ((rc = check_pointers(pp.ptr, num_parts, num_column_index, "part_pointers"))) return rc;
  if ((rc = check_pointers(ppc.ptr, num_groups, n_cic, "part_pointers_cache"))) return rc;
  if ((rc = check_ids(p2n.ptr, num_parts, num_nodes, "part2Node"))) return rc;
  if ((rc = check_ids(col.ptr, num_column_index, num_nodes, "column_index"))) return rc;
  if ((rc = check_ids(cic.ptr, n_cic, num_nodes, "column_index_cache"))) return rc;
  for (int p = 0; p < num_parts; ++p)
    if (flag.ptr[p] < 0 || flag.ptr[p] > num_groups) return bad_layout("part_cache_flagindex names a group that does not exist");

  HostPlan hp;
  hp.num_nodes = num_nodes; hp.row_begin = row_begin; hp.row_end = row_end;
  const int rows = row_end - row_begin;
  try {
    hp.row_ptr.assign((size_t)rows + 1, 0);
    for (int p = 0; p < num_parts; ++p) {
      int v = p2n.ptr[p];
      if (v < row_begin || v >= row_end) continue;
      hp.row_ptr[(size_t)(v - row_begin) + 1] += flag.ptr[p] > 0 ? 1 : pp.ptr[p + 1] - pp.ptr[p];
      hp.original_edges += pp.ptr[p + 1] - pp.ptr[p];
    }
    for (int r = 0; r < rows; ++r) hp.row_ptr[r + 1] += hp.row_ptr[r];
    hp.col.resize((size_t)hp.row_ptr[rows]);
    std::vector<int64_t> pos(hp.row_ptr.begin(), hp.row_ptr.end() - 1);
    for (int p = 0; p < num_parts; ++p) {
      int v = p2n.ptr[p];
      if (v < row_begin || v >= row_end) continue;
      int64_t& w = pos[(size_t)(v - row_begin)];
      if (flag.ptr[p] > 0) {
        hp.col[(size_t)w++] = num_nodes + (flag.ptr[p] - 1);
      } else {
        for (int32_t k = pp.ptr[p]; k < pp.ptr[p + 1]; ++k) hp.col[(size_t)w++] = col.ptr[k];
      }
    }
    // every group keeps its id: upstream's caching kernel fills all rows of the caller's
    // part_result_cache (reuse_conv_kernel.cu:427-486), used or not
    if (num_groups > 0) {
      hp.group_ptr.assign(ppc.ptr, ppc.ptr + num_groups + 1);
      hp.group_col.assign(cic.ptr, cic.ptr + n_cic);
    } else {
      hp.group_ptr.assign(1, 0);
    }
  } catch (const std::bad_alloc&) {
    set_error("out of host memory while building the plan");
    return ROF_ERR_NO_MEMORY;
  }
  return finalize_plan(hp, plan, stream);
}

int rof_plan_create_v2(rof_plan** plan, int where, int num_nodes, int row_begin, int row_end,
                       const int32_t* uniqpart_column_index, int64_t num_column_index,
                       const int32_t* uniqpart_pointers, const int32_t* part2Node_ptr,
                       const int32_t* part2Node_col, int num_uniqparts, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  int rc = check_common(plan, where, num_nodes, row_begin, row_end);
  if (rc) return rc;
  if (num_uniqparts < 0) { set_error("num_uniqparts < 0"); return ROF_ERR_BAD_ARGUMENT; }
  HostArray col, up, np_, nc;
  const int64_t nptr = num_uniqparts ? (int64_t)num_uniqparts + 1 : 0;
  if ((rc = col.fetch(uniqpart_column_index, num_column_index, where, stream, "uniqpart_column_index"))) return rc;
  if ((rc = up.fetch(uniqpart_pointers, nptr, where, stream, "uniqpart_pointers"))) return rc;
  if ((rc = np_.fetch(part2Node_ptr, nptr, where, stream, "part2Node_ptr"))) return rc;
  if ((rc = sync_if_device(where, stream))) return rc;
  const int64_t n_nc = num_uniqparts ? np_.ptr[num_uniqparts] : 0;
  if (n_nc < 0) return bad_layout("part2Node_ptr ends below zero");
  if ((rc = nc.fetch(part2Node_col, n_nc, where, stream, "part2Node_col"))) return rc;
  if ((rc = sync_if_device(where, stream))) return rc;
  if ((rc = check_pointers(up.ptr, num_uniqparts, num_column_index, "uniqpart_pointers"))) return rc;
  if ((rc = check_pointers(np_.ptr, num_uniqparts, n_nc, "part2Node_ptr"))) return rc;
  if ((rc = check_ids(col.ptr, num_column_index, num_nodes, "uniqpart_column_index"))) return rc;
  if ((rc = check_ids(nc.ptr, n_nc, num_nodes, "part2Node_col"))) return rc;

  HostPlan hp;
  hp.num_nodes = num_nodes; hp.row_begin = row_begin; hp.row_end = row_end;
  const int rows = row_end - row_begin;
  try {
    // A unique part becomes a reuse group — its partial sum is built once in phase A and read as
    // one row by each of its destinations — when that saves row traffic inside this plan's row
    // block: `local` destinations read 1 row instead of `len`, at the price of `len` reads and one
    // write in phase A.  Otherwise its sources are listed inline in the destination's row.
    // And reuse is used at all only when it saves a worthwhile share of the gathered rows
    // (reuse_min_saving(): below that the partial rows cost more L2 than the reads they replace;
    // measured on the 114.6M- and 123.8M-edge power-law graphs, 6.5 % and 2.8 % saved: 1-2 % slower).
    // With ROF_REUSE_MIN <= 0 every part shared by two local destinations is a group, as the search
    // picked them.
    const double min_saving = reuse_min_saving();
    auto worth = [min_saving](int local, int32_t len) {
      if (local < 2 || len < 2) return false;
      return min_saving <= 0.0 || (int64_t)local * (len - 1) > len + 1;
    };
    std::vector<int32_t> group_of((size_t)num_uniqparts, -1);
    std::vector<int32_t> local_of((size_t)num_uniqparts, 0);
    int64_t saved = 0, total = 0;
    for (int u = 0; u < num_uniqparts; ++u) {
      const int32_t len = up.ptr[u + 1] - up.ptr[u];
      int local = 0;
      for (int32_t k = np_.ptr[u]; k < np_.ptr[u + 1]; ++k) local += (nc.ptr[k] >= row_begin && nc.ptr[k] < row_end);
      local_of[(size_t)u] = local;
      total += (int64_t)local * len;
      if (worth(local, len)) saved += (int64_t)local * (len - 1) - (len + 1);
    }
    const bool use_groups = total > 0 && (min_saving <= 0.0 || (double)saved >= min_saving * (double)total);
    hp.group_ptr.assign(1, 0);
    hp.row_ptr.assign((size_t)rows + 1, 0);
    for (int u = 0; u < num_uniqparts; ++u) {
      const int32_t len = up.ptr[u + 1] - up.ptr[u];
      const int local = local_of[(size_t)u];
      if (local == 0 || len == 0) continue;
      const bool grouped = use_groups && worth(local, len);
      if (grouped) {
        group_of[u] = (int32_t)hp.group_ptr.size() - 1;
        hp.group_col.insert(hp.group_col.end(), col.ptr + up.ptr[u], col.ptr + up.ptr[u + 1]);
        hp.group_ptr.push_back((int32_t)hp.group_col.size());
      }
      for (int32_t k = np_.ptr[u]; k < np_.ptr[u + 1]; ++k) {
        int v = nc.ptr[k];
        if (v < row_begin || v >= row_end) continue;
        hp.row_ptr[(size_t)(v - row_begin) + 1] += grouped ? 1 : len;
        hp.original_edges += len;
      }
    }
    for (int r = 0; r < rows; ++r) hp.row_ptr[r + 1] += hp.row_ptr[r];
    hp.col.resize((size_t)hp.row_ptr[rows]);
    std::vector<int64_t> pos(hp.row_ptr.begin(), hp.row_ptr.end() - 1);
    for (int u = 0; u < num_uniqparts; ++u) {
      const int32_t len = up.ptr[u + 1] - up.ptr[u];
      if (len == 0) continue;
      for (int32_t k = np_.ptr[u]; k < np_.ptr[u + 1]; ++k) {
        int v = nc.ptr[k];
        if (v < row_begin || v >= row_end) continue;
        int64_t& w = pos[(size_t)(v - row_begin)];
        if (group_of[u] >= 0) {
          hp.col[(size_t)w++] = num_nodes + group_of[u];
        } else {
          for (int32_t s = up.ptr[u]; s < up.ptr[u + 1]; ++s) hp.col[(size_t)w++] = col.ptr[s];
        }
      }
    }
  } catch (const std::bad_alloc&) {
    set_error("out of host memory while building the plan");
    return ROF_ERR_NO_MEMORY;
  }
  return finalize_plan(hp, plan, stream);
}

int rof_plan_export(const rof_plan* p, int64_t* row_ptr, int32_t* col, int32_t* group_ptr, int32_t* group_col,
                    int32_t* items, int32_t* split_rows) {
  if (p == nullptr) { set_error("rof_plan_export: null plan"); return ROF_ERR_BAD_ARGUMENT; }
  if (row_ptr) std::memcpy(row_ptr, p->h_row_ptr.data(), sizeof(int64_t) * p->h_row_ptr.size());
  if (group_ptr) std::memcpy(group_ptr, p->h_group_ptr.data(), sizeof(int32_t) * p->h_group_ptr.size());
  if (items) std::memcpy(items, p->h_items.data(), sizeof(WorkItem) * p->h_items.size());
  if (split_rows) std::memcpy(split_rows, p->h_split.data(), sizeof(SplitRow) * p->h_split.size());
  const size_t nb = sizeof(int32_t) * (size_t)p->gather_entries, ng = sizeof(int32_t) * (size_t)p->group_sources;
  if (p->device < 0) {
    if (col && nb) std::memcpy(col, p->h_col.data(), nb);
    if (group_col && ng) std::memcpy(group_col, p->h_col.data() + p->gather_entries, ng);
    return ROF_OK;
  }
  cudaError_t e = cudaSuccess;
  if (col && nb) e = cudaMemcpy(col, p->d_col, nb, cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && group_col && ng) e = cudaMemcpy(group_col, p->d_col + p->gather_entries, ng, cudaMemcpyDeviceToHost);
  return e == cudaSuccess ? ROF_OK : cuda_fail(e, "rof_plan_export");
}

int rof_plan_export_tiles(const rof_plan* p, int32_t* tiles, int32_t* titems, int32_t* tcol, int32_t* stage_col) {
  if (p == nullptr) { set_error("rof_plan_export_tiles: null plan"); return ROF_ERR_BAD_ARGUMENT; }
  const auto& t = p->tiled;
  if (tiles) std::memcpy(tiles, t.h_tiles.data(), sizeof(TileDesc) * t.h_tiles.size());
  if (titems) std::memcpy(titems, t.h_titems.data(), sizeof(WorkItem) * t.h_titems.size());
  if (tcol) std::memcpy(tcol, t.h_tcol.data(), sizeof(int32_t) * t.h_tcol.size());
  if (stage_col) std::memcpy(stage_col, t.h_stage_col.data(), sizeof(int32_t) * t.h_stage_col.size());
  return ROF_OK;
}

void rof_plan_destroy(rof_plan* p) {
  if (p == nullptr) return;
  cudaFree(p->d_col);
  cudaFree(p->d_items);
  cudaFree(p->d_group_items);
  cudaFree(p->d_group_orig);
  cudaFree(p->d_split);
  cudaFree(p->fine.d_items);
  cudaFree(p->fine.d_split);
  cudaFree(p->tiled.d_tcol);
  cudaFree(p->tiled.d_titems);
  cudaFree(p->tiled.d_tiles);
  cudaFree(p->tiled.d_stage_col);
  cudaFree(p->tiled.d_rest_items);
  cudaFree(p->tiled.d_rest_items_fine);
  cudaFree(p->d_slot_owner);
  cudaFree(p->d_arrive);
  cudaFree(p->fine.d_slot_owner);
  cudaFree(p->fine.d_arrive);
  if (p->h_status) cudaFreeHost(p->h_status);
  delete p;
}

int rof_plan_get_info(const rof_plan* p, rof_plan_info* info) {
  if (p == nullptr || info == nullptr) { set_error("rof_plan_get_info: null argument"); return ROF_ERR_BAD_ARGUMENT; }
  info->num_nodes = p->num_nodes;
  info->row_begin = p->row_begin;
  info->row_end = p->row_end;
  info->num_groups = p->num_groups;
  info->group_sources = p->group_sources;
  info->gather_entries = p->gather_entries;
  info->partial_entries = p->partial_entries;
  info->original_edges = p->original_edges;
  info->num_items = p->num_items;
  info->split_rows = p->num_split_rows;
  info->num_slots = p->num_slots;
  info->segment_edges = p->segment_edges;
  info->num_tiles = p->tiled.num_tiles;
  info->tile_items = p->tiled.num_items;
  info->tile_entries = p->tiled.entries;
  info->tile_shared_entries = p->tiled.shared_entries;
  info->tile_staged_rows = p->tiled.staged_rows;
  return ROF_OK;
}

}  // extern "C"
