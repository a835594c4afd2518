// Reuse-group search: a from-scratch, parallel implementation of the host-side
// preprocessing pipeline whose *outputs* are identical, array for array, to upstream's
// reuse_search_ext (ROF/reuse_search_ext/src/reuse_search_ext.h):
//
//   split_part                  (:82-148)   fixed-size chunks ("parts") of every in-neighbour list
//   get_part_intersect          (:152-228)  for each full part, the destinations containing all its sources
//   greedy_max_reuse            (:232-303)  fan-out-descending greedy pick of source-disjoint parts
//   reorganize_indices          (:409-505)  ROF_v1 layout
//   reorganize_indices_uniquely (:507-640)  ROF_v2 layout
//
// Upstream's algorithms are quadratic in places (a std::set per source per part, a linear
// find+swap per group per destination) and need hours and tens of GB at 10^8 edges.  The
// same results are computed here differently:
//   * intersections are counted with bitmaps (AND + popcount, or probes) for high-out-degree
//     sources and galloping searches otherwise; only the picked parts' lists are materialised;
//   * the pick order needs upstream's exact tie-breaking, which comes from std::sort on an
//     identity permutation with a "greater fan-out" comparator — reproduced by making the
//     same std::sort call on the same data;
//   * the row reorganisation is done per destination row in parallel (rows are independent:
//     only the pick order of the groups containing a row matters), with a position map in
//     place of the linear find.
// tests/test_search_cpu.py checks every output array against upstream's own module.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <parallel/algorithm>
#include <vector>
#include <omp.h>

namespace {

using u32 = uint32_t;

struct Csr {
  int n;
  const int64_t* ptr;
  const int32_t* idx;
  int64_t deg(int v) const { return ptr[v + 1] - ptr[v]; }
  const int32_t* row(int v) const { return idx + ptr[v]; }
};

struct Bitmaps {
  int words = 0;                       // 64-bit words per bitmap
  std::vector<int32_t> slot;           // node -> bitmap index or -1
  std::vector<uint64_t> bits;
  const uint64_t* of(int node) const { return slot[node] < 0 ? nullptr : bits.data() + (size_t)slot[node] * words; }
};

// Bitmaps for the highest-out-degree sources, within a memory budget.
void build_bitmaps(const Csr& out, int64_t budget_bytes, Bitmaps& bm) {
  const int n = out.n;
  bm.words = (n + 63) / 64;
  bm.slot.assign((size_t)n, -1);
  const int64_t per = (int64_t)bm.words * 8;
  int64_t max_maps = per > 0 ? budget_bytes / per : 0;
  if (max_maps <= 0) return;
  // a bitmap pays off only when the list is long relative to a probe/merge
  const int64_t min_deg = std::max<int64_t>(256, bm.words / 4);
  std::vector<int32_t> cand;
  for (int v = 0; v < n; ++v)
    if (out.deg(v) >= min_deg) cand.push_back(v);
  if ((int64_t)cand.size() > max_maps) {
    std::nth_element(cand.begin(), cand.begin() + max_maps, cand.end(),
                     [&](int32_t a, int32_t b) { return out.deg(a) > out.deg(b); });
    cand.resize((size_t)max_maps);
  }
  bm.bits.assign((size_t)cand.size() * bm.words, 0);
  for (size_t i = 0; i < cand.size(); ++i) bm.slot[cand[i]] = (int32_t)i;
#pragma omp parallel for schedule(dynamic, 16)
  for (int64_t i = 0; i < (int64_t)cand.size(); ++i) {
    uint64_t* b = bm.bits.data() + (size_t)i * bm.words;
    const int v = cand[i];
    for (int64_t k = out.ptr[v]; k < out.ptr[v + 1]; ++k) {
      const int32_t u = out.idx[k];
      b[u >> 6] |= 1ull << (u & 63);
    }
  }
}

// first position in [lo, hi) with a[pos] >= key, found by galloping from lo
inline int64_t gallop(const int32_t* a, int64_t lo, int64_t hi, int32_t key) {
  int64_t step = 1, l = lo;
  while (l + step < hi && a[l + step] < key) { l += step; step <<= 1; }
  int64_t r = std::min(hi, l + step + 1);
  return std::lower_bound(a + l, a + r, key) - a;
}

// Destinations that contain every source of the part: intersection of the sources' out-lists.
// Returns the count; when `out_list` is given also appends the members (ascending).
int64_t intersect_part(const Csr& out, const Bitmaps& bm, const int32_t* src, int ps, std::vector<u32>* out_list) {
  int order[16];
  for (int i = 0; i < ps; ++i) order[i] = i;
  std::sort(order, order + ps, [&](int a, int b) { return out.deg(src[a]) < out.deg(src[b]); });
  const int s0 = src[order[0]];
  const int64_t d0 = out.deg(s0);
  if (d0 == 0) return 0;

  bool all_bitmaps = true;
  for (int i = 0; i < ps; ++i) all_bitmaps &= (bm.of(src[i]) != nullptr);
  if (all_bitmaps && (int64_t)bm.words * ps < d0 * 2 * (ps - 1) + 64) {
    const uint64_t* maps[16];
    for (int i = 0; i < ps; ++i) maps[i] = bm.of(src[i]);
    int64_t cnt = 0;
    for (int w = 0; w < bm.words; ++w) {
      uint64_t x = maps[0][w];
      for (int i = 1; i < ps && x; ++i) x &= maps[i][w];
      if (!x) continue;
      cnt += __builtin_popcountll(x);
      if (out_list)
        while (x) {
          out_list->push_back((u32)(w * 64 + __builtin_ctzll(x)));
          x &= x - 1;
        }
    }
    return cnt;
  }

  const int32_t* a = out.row(s0);
  const uint64_t* maps[16];
  const int32_t* rows[16];
  int64_t cur[16], len[16];
  for (int i = 1; i < ps; ++i) {
    const int s = src[order[i]];
    maps[i] = bm.of(s);
    rows[i] = out.row(s);
    cur[i] = 0;
    len[i] = out.deg(s);
  }
  int64_t cnt = 0;
  bool others_mapped = true;
  for (int i = 1; i < ps; ++i) others_mapped &= (maps[i] != nullptr);
  if (!out_list && others_mapped) {  // count only, every other list as a bitmap: branch-free probes
    for (int64_t k = 0; k < d0; ++k) {
      const int32_t u = a[k];
      uint64_t bit = 1;
      for (int i = 1; i < ps; ++i) bit &= maps[i][u >> 6] >> (u & 63);
      cnt += (int64_t)(bit & 1);
    }
    return cnt;
  }
  for (int64_t k = 0; k < d0; ++k) {
    const int32_t u = a[k];
    bool in_all = true;
    for (int i = 1; i < ps; ++i) {
      if (maps[i]) {
        if (!((maps[i][u >> 6] >> (u & 63)) & 1)) { in_all = false; break; }
      } else {
        cur[i] = gallop(rows[i], cur[i], len[i], u);
        if (cur[i] >= len[i]) {  // this list is exhausted: nothing further can match
          in_all = false;
          k = d0;
          break;
        }
        if (rows[i][cur[i]] != u) { in_all = false; break; }
      }
    }
    if (in_all) {
      ++cnt;
      if (out_list) out_list->push_back((u32)u);
    }
  }
  return cnt;
}

bool rows_sorted_unique(const Csr& c) {
  bool ok = true;
#pragma omp parallel for schedule(static, 4096) reduction(&& : ok)
  for (int v = 0; v < c.n; ++v)
    for (int64_t k = c.ptr[v] + 1; k < c.ptr[v + 1]; ++k) ok = ok && (c.idx[k - 1] < c.idx[k]);
  return ok;
}

}  // namespace

extern "C" {

enum rofh_search_array {
  ROFH_PART_POINTERS = 0, ROFH_PART2NODE, ROFH_NUM_PARTS_PER_NODE_ACC, ROFH_INTERSECTION_NUM, ROFH_INDEX_PICKED,
  ROFH_PICKED_FANOUT, ROFH_COLUMN_INDEX, ROFH_PART_POINTERS_CACHE, ROFH_COLUMN_INDEX_CACHE,
  ROFH_PART_CACHE_FLAGINDEX, ROFH_UNIQPART_COLUMN_INDEX, ROFH_UNIQPART_POINTERS, ROFH_PART2NODE_PTR,
  ROFH_PART2NODE_COL, ROFH_NUM_ARRAYS
};

struct rofh_search {
  std::vector<int32_t> arr[ROFH_NUM_ARRAYS];
  double seconds[6] = {0, 0, 0, 0, 0, 0};  // split, count, pick, lists, reorganise, assemble
};

// Inputs: destination-major CSR (indptr_dst, indices_src) and its transpose (indptr_src,
// indices_dst), rows ascending without duplicates, as upstream's scripts build them with
// scipy (ROF_evaluation/cuda/middle-main.py:184-198).  Returns nullptr on bad arguments.
rofh_search* rofh_reuse_search(int n, const int64_t* indptr_dst, const int32_t* indices_src,
                               const int64_t* indptr_src, const int32_t* indices_dst, int part_size,
                               int num_threads, int64_t bitmap_budget_bytes) {
  if (n < 0 || part_size < 1 || part_size > 16) return nullptr;
  if (num_threads > 0) omp_set_num_threads(num_threads);
  const Csr in{n, indptr_dst, indices_src};
  const Csr outg{n, indptr_src, indices_dst};
  const int64_t E = n ? indptr_dst[n] : 0;
  if (E >= INT32_MAX) return nullptr;
  if (!rows_sorted_unique(in) || !rows_sorted_unique(outg)) return nullptr;
  const int ps = part_size;
  rofh_search* S = new rofh_search();
  double t0 = omp_get_wtime();

  // ---- split_part -------------------------------------------------------------------
  std::vector<int32_t>& acc = S->arr[ROFH_NUM_PARTS_PER_NODE_ACC];
  acc.resize((size_t)n);
  int64_t run = 0;
  for (int v = 0; v < n; ++v) {
    run += (in.deg(v) + ps - 1) / ps;
    acc[v] = (int32_t)run;
  }
  const int64_t P = run;
  std::vector<int32_t>& part_ptr = S->arr[ROFH_PART_POINTERS];
  std::vector<int32_t>& part2node = S->arr[ROFH_PART2NODE];
  part_ptr.resize((size_t)P + 1);
  part2node.resize((size_t)P);
  part_ptr[0] = 0;
#pragma omp parallel for schedule(static, 1024)
  for (int v = 0; v < n; ++v) {
    const int64_t base = v ? acc[v - 1] : 0, np = acc[v] - base;
    for (int64_t j = 0; j < np; ++j) {
      part2node[(size_t)(base + j)] = v;
      part_ptr[(size_t)(base + j + 1)] = (int32_t)(j == np - 1 ? indptr_dst[v + 1] : indptr_dst[v] + (j + 1) * ps);
    }
  }
  S->seconds[0] = omp_get_wtime() - t0; t0 = omp_get_wtime();

  // ---- get_part_intersect (sizes only; discard_remainder_part = true) ------------------
  Bitmaps bm;
  build_bitmaps(outg, bitmap_budget_bytes, bm);
  std::vector<int32_t>& nums = S->arr[ROFH_INTERSECTION_NUM];
  nums.assign((size_t)P, 0);
  {
    // Many parts hold the same source tuple (hub pairs recur in thousands of rows) and the
    // expensive ones are exactly those: count each distinct tuple once.  Parts are grouped
    // by sorting a 64-bit key (highest-out-degree source of the tuple, 32-bit hash of the
    // tuple): equal tuples become neighbours (confirmed by comparing the tuples), and
    // consecutive tuples share their longest out-list, which then stays in cache.
    struct Key { uint64_t h; u32 p; bool operator<(const Key& o) const { return h < o.h || (h == o.h && p < o.p); } };
    std::vector<Key> keys((size_t)P);
#pragma omp parallel for schedule(static, 4096)
    for (int64_t p = 0; p < P; ++p) {
      if (part_ptr[(size_t)p + 1] - part_ptr[(size_t)p] != ps) {
        keys[(size_t)p] = Key{~0ull, (u32)p};  // partial parts sort to the end and are dropped
        continue;
      }
      const int32_t* t = indices_src + part_ptr[(size_t)p];
      uint64_t h = 0x9E3779B97F4A7C15ull;
      int32_t big = t[0];
      for (int k = 0; k < ps; ++k) {
        h ^= (uint64_t)(u32)t[k] + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
        h *= 0xBF58476D1CE4E5B9ull;
        if (outg.deg(t[k]) > outg.deg(big)) big = t[k];
      }
      keys[(size_t)p] = Key{((uint64_t)(u32)big << 32) | (h >> 32), (u32)p};
    }
    __gnu_parallel::sort(keys.begin(), keys.end());
    while (!keys.empty() && keys.back().h == ~0ull &&
           part_ptr[(size_t)keys.back().p + 1] - part_ptr[(size_t)keys.back().p] != ps)
      keys.pop_back();
    const int64_t F = (int64_t)keys.size();
    auto same_tuple = [&](u32 a, u32 b) {
      return std::memcmp(indices_src + part_ptr[a], indices_src + part_ptr[b], sizeof(int32_t) * (size_t)ps) == 0;
    };
    // run starts: a new run begins where the hash changes; inside a run of equal hashes
    // (almost always one tuple) every part is compared with the run's representatives
    std::vector<int64_t> run_start;
    for (int64_t i = 0; i < F; ++i)
      if (i == 0 || keys[(size_t)i].h != keys[(size_t)i - 1].h) run_start.push_back(i);
    run_start.push_back(F);
    const int64_t R = (int64_t)run_start.size() - 1;
#pragma omp parallel
    {
      std::vector<std::pair<u32, int32_t>> reps;  // (representative part, its count) within one run
#pragma omp for schedule(dynamic, 512)
      for (int64_t r = 0; r < R; ++r) {
        reps.clear();
        for (int64_t i = run_start[(size_t)r]; i < run_start[(size_t)r + 1]; ++i) {
          const u32 p = keys[(size_t)i].p;
          int32_t cnt = -1;
          for (auto& rp : reps)
            if (same_tuple(rp.first, p)) { cnt = rp.second; break; }
          if (cnt < 0) {
            cnt = (int32_t)intersect_part(outg, bm, indices_src + part_ptr[p], ps, nullptr);
            reps.emplace_back(p, cnt);
          }
          nums[p] = cnt;
        }
      }
    }
  }
  S->seconds[1] = omp_get_wtime() - t0; t0 = omp_get_wtime();

  // ---- greedy_max_reuse --------------------------------------------------------------
  // The same call upstream makes (:245-264): std::sort over an identity permutation of
  // uint32 with this comparator.  Ties are broken by the library's introsort; making the
  // identical call on identical data is what reproduces upstream's order.
  // std::sort's result depends only on the outcomes of its comparisons, so sorting
  // (fan-out, index) pairs by fan-out walks through the same comparisons and moves as upstream's
  // sort of bare indices with a look-up comparator, without the cache miss per comparison.
  struct Keyed { u32 num; u32 idx; };
  std::vector<u32> unums(nums.begin(), nums.end());
  std::vector<Keyed> keyed((size_t)P);
#pragma omp parallel for schedule(static, 1 << 16)
  for (int64_t i = 0; i < P; ++i) keyed[(size_t)i] = Keyed{unums[(size_t)i], (u32)i};
  std::sort(keyed.begin(), keyed.end(), [](const Keyed& a, const Keyed& b) { return a.num > b.num; });
  std::vector<u32> index_ordered((size_t)P);
#pragma omp parallel for schedule(static, 1 << 16)
  for (int64_t i = 0; i < P; ++i) index_ordered[(size_t)i] = keyed[(size_t)i].idx;
  keyed.clear(); keyed.shrink_to_fit();
  std::vector<int32_t>& picked = S->arr[ROFH_INDEX_PICKED];
  std::vector<uint8_t> taken((size_t)n, 0);
  for (int64_t i = 0; i < P; ++i) {
    const u32 p = index_ordered[(size_t)i];
    if (unums[p] < 2) break;
    bool conflict = false;
    for (int32_t k = part_ptr[p]; k < part_ptr[p + 1]; ++k) conflict |= taken[(size_t)indices_src[k]] != 0;
    if (conflict) continue;
    picked.push_back((int32_t)p);
    for (int32_t k = part_ptr[p]; k < part_ptr[p + 1]; ++k) taken[(size_t)indices_src[k]] = 1;
  }
  const int64_t G = (int64_t)picked.size();
  S->seconds[2] = omp_get_wtime() - t0; t0 = omp_get_wtime();

  // ---- destination lists of the picked parts -------------------------------------------
  std::vector<std::vector<u32>> lists((size_t)G);
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t g = 0; g < G; ++g) {
    lists[(size_t)g].reserve((size_t)nums[(size_t)picked[(size_t)g]]);
    intersect_part(outg, bm, indices_src + part_ptr[(size_t)picked[(size_t)g]], ps, &lists[(size_t)g]);
  }
  std::vector<int32_t>& fan = S->arr[ROFH_PICKED_FANOUT];
  fan.resize((size_t)G);
  std::vector<int32_t>& p2n_ptr = S->arr[ROFH_PART2NODE_PTR];
  std::vector<int32_t>& p2n_col = S->arr[ROFH_PART2NODE_COL];
  p2n_ptr.assign(1, 0);
  for (int64_t g = 0; g < G; ++g) {
    fan[(size_t)g] = (int32_t)lists[(size_t)g].size();
    p2n_ptr.push_back(p2n_ptr.back() + fan[(size_t)g]);
  }
  S->seconds[3] = omp_get_wtime() - t0; t0 = omp_get_wtime();

  // groups of each destination, in pick order (transpose of `lists`)
  std::vector<int64_t> gptr((size_t)n + 1, 0);
  for (int64_t g = 0; g < G; ++g)
    for (u32 v : lists[(size_t)g]) gptr[(size_t)v + 1]++;
  for (int v = 0; v < n; ++v) gptr[(size_t)v + 1] += gptr[(size_t)v];
  std::vector<int32_t> gof((size_t)gptr[(size_t)n]);
  {
    std::vector<int64_t> pos(gptr.begin(), gptr.end() - 1);
    for (int64_t g = 0; g < G; ++g)
      for (u32 v : lists[(size_t)g]) gof[(size_t)pos[v]++] = (int32_t)g;
  }

  // ---- reorganise every row (v1 column_index + flags) -----------------------------------
  // Upstream, per picked part in pick order and per destination: linear-find each source in
  // the not-yet-reorganised tail of the row and swap it to the front of that tail (:464-472).
  // Per row that is the sequence below; `where`/`who` replace the linear find.
  std::vector<int32_t>& col1 = S->arr[ROFH_COLUMN_INDEX];
  col1.assign(indices_src, indices_src + E);
  std::vector<int32_t>& flag = S->arr[ROFH_PART_CACHE_FLAGINDEX];
  flag.assign((size_t)P, 0);
  std::vector<int32_t> done((size_t)n, 0);  // entries moved to the front of each row
#pragma omp parallel
  {
    std::vector<int32_t> where, who;  // original rank -> position, position -> original rank
#pragma omp for schedule(dynamic, 256)
    for (int v = 0; v < n; ++v) {
      const int64_t ng = gptr[(size_t)v + 1] - gptr[(size_t)v];
      if (ng == 0) continue;
      const int64_t b = indptr_dst[v], d = in.deg(v);
      const int32_t* orig = indices_src + b;
      int32_t* row = col1.data() + b;
      where.resize((size_t)d);
      who.resize((size_t)d);
      std::iota(where.begin(), where.end(), 0);
      std::iota(who.begin(), who.end(), 0);
      int64_t front = 0;
      const int64_t part_base = v ? acc[(size_t)v - 1] : 0;
      for (int64_t t = 0; t < ng; ++t) {
        const int32_t g = gof[(size_t)(gptr[(size_t)v] + t)];
        const int32_t p = picked[(size_t)g];
        for (int32_t k = part_ptr[(size_t)p]; k < part_ptr[(size_t)p + 1]; ++k) {
          const int32_t s = indices_src[k];
          const int64_t rank = std::lower_bound(orig, orig + d, s) - orig;
          if (rank >= d || orig[rank] != s) continue;           // upstream's "impossible error"
          const int64_t at = where[(size_t)rank];
          if (at < front) continue;
          const int32_t other = who[(size_t)front];
          std::swap(row[at], row[front]);
          who[(size_t)at] = other; where[(size_t)other] = (int32_t)at;
          who[(size_t)front] = (int32_t)rank; where[(size_t)rank] = (int32_t)front;
          ++front;
        }
        flag[(size_t)(part_base + t)] = g + 1;
      }
      done[(size_t)v] = (int32_t)front;
    }
  }
  S->seconds[4] = omp_get_wtime() - t0; t0 = omp_get_wtime();

  // ---- assemble v1 cache arrays and the v2 layout ---------------------------------------
  std::vector<int32_t>& ppc = S->arr[ROFH_PART_POINTERS_CACHE];
  std::vector<int32_t>& cic = S->arr[ROFH_COLUMN_INDEX_CACHE];
  ppc.assign(1, 0);
  cic.reserve((size_t)G * ps);
  for (int64_t g = 0; g < G; ++g) {
    const int32_t p = picked[(size_t)g];
    cic.insert(cic.end(), indices_src + part_ptr[(size_t)p], indices_src + part_ptr[(size_t)p + 1]);
    ppc.push_back((int32_t)cic.size());
  }
  p2n_col.resize((size_t)p2n_ptr.back());
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t g = 0; g < G; ++g)
    std::copy(lists[(size_t)g].begin(), lists[(size_t)g].end(), p2n_col.begin() + p2n_ptr[(size_t)g]);

  // residual chunks, node by node (:607-636)
  std::vector<int64_t> res_parts((size_t)n + 1, 0), res_cols((size_t)n + 1, 0);
  for (int v = 0; v < n; ++v) {
    const int64_t r = in.deg(v) - done[(size_t)v];
    res_cols[(size_t)v + 1] = res_cols[(size_t)v] + r;
    res_parts[(size_t)v + 1] = res_parts[(size_t)v] + (r + ps - 1) / ps;
  }
  std::vector<int32_t>& ucol = S->arr[ROFH_UNIQPART_COLUMN_INDEX];
  std::vector<int32_t>& uptr = S->arr[ROFH_UNIQPART_POINTERS];
  const int64_t gcols = (int64_t)cic.size();
  ucol.resize((size_t)(gcols + res_cols[(size_t)n]));
  uptr.resize((size_t)(G + 1 + res_parts[(size_t)n]));
  std::copy(cic.begin(), cic.end(), ucol.begin());
  std::copy(ppc.begin(), ppc.end(), uptr.begin());
  const int64_t fan_total = p2n_ptr.back();
  p2n_ptr.resize((size_t)(G + 1 + res_parts[(size_t)n]));
  p2n_col.resize((size_t)(fan_total + res_parts[(size_t)n]));
#pragma omp parallel for schedule(static, 1024)
  for (int v = 0; v < n; ++v) {
    const int64_t r = in.deg(v) - done[(size_t)v];
    if (r == 0) continue;
    const int64_t cbase = gcols + res_cols[(size_t)v];
    std::copy(col1.begin() + indptr_dst[v] + done[(size_t)v], col1.begin() + indptr_dst[v + 1], ucol.begin() + cbase);
    const int64_t np = (r + ps - 1) / ps;
    for (int64_t j = 0; j < np; ++j) {
      const int64_t u = G + res_parts[(size_t)v] + j;  // unique-part id
      uptr[(size_t)u + 1] = (int32_t)(j == np - 1 ? cbase + r : cbase + (j + 1) * ps);
      p2n_col[(size_t)(fan_total + res_parts[(size_t)v] + j)] = v;
      p2n_ptr[(size_t)u + 1] = (int32_t)(fan_total + res_parts[(size_t)v] + j + 1);
    }
  }
  S->seconds[5] = omp_get_wtime() - t0;
  return S;
}

int64_t rofh_search_size(const rofh_search* s, int which) {
  if (!s || which < 0 || which >= ROFH_NUM_ARRAYS) return -1;
  return (int64_t)s->arr[which].size();
}

void rofh_search_fetch(const rofh_search* s, int which, int32_t* out) {
  if (!s || which < 0 || which >= ROFH_NUM_ARRAYS) return;
  if (!s->arr[which].empty()) std::memcpy(out, s->arr[which].data(), sizeof(int32_t) * s->arr[which].size());
}

double rofh_search_seconds(const rofh_search* s, int stage) { return (s && stage >= 0 && stage < 6) ? s->seconds[stage] : -1.0; }

void rofh_search_free(rofh_search* s) { delete s; }

}  // extern "C"
