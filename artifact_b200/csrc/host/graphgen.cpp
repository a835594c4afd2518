// Seeded synthetic graph generators (host, OpenMP).
//
// The benchmark configurations are named by shape only (node count, edge count, degree
// exponent, cap); no dataset is available, so graphs of those shapes are drawn here.
// Everything is a pure function of (parameters, seed): each destination row owns a
// counter-based random stream, so the result does not depend on the thread count.
//
// Output format is the one the reuse preprocessor consumes: a CSR over destinations
// (`indptr_dst[n+1]`, `indices_src[]`, each row sorted ascending, no duplicates), i.e. the
// arrays upstream builds with scipy in ROF_evaluation/cuda/middle-main.py:184-198.
#include <algorithm>
#include <climits>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <omp.h>

namespace {

struct SplitMix64 {
  uint64_t s;
  explicit SplitMix64(uint64_t seed) : s(seed) {}
  uint64_t next() {
    uint64_t z = (s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
  // uniform in (0,1): never 0, so log() is finite
  double uniform() { return ((next() >> 11) + 0.5) * (1.0 / 9007199254740992.0); }
  uint64_t below(uint64_t n) { return (uint64_t)(((__uint128_t)next() * n) >> 64); }
};

inline uint64_t mix_seed(uint64_t seed, uint64_t row) {
  SplitMix64 g(seed ^ (row * 0xD6E8FEB86659FD93ull + 0x2545F4914F6CDD1Dull));
  g.next();
  return g.next();
}

struct RowStore {
  // per-thread append buffers + per-row (thread, offset, length)
  std::vector<std::vector<int32_t>> buf;
  std::vector<int32_t> row_thread;
  std::vector<int64_t> row_off;
  std::vector<int32_t> row_len;
  int n = 0;
};

}  // namespace

extern "C" {

struct rofh_graph {
  RowStore st;
};

// Directed Chung-Lu graph, one row per destination.
//   a_desc[n]   : source (out-) weights sorted in DESCENDING order
//   src_id[n]   : node id of the source holding a_desc[k]
//   b[n]        : destination (in-) weight of node v, indexed by node id
//   S           : normaliser; P(u -> v) = min(1, a_u * b_v / S)
// Sampling uses geometric skipping over the descending weight list (Miller & Hagberg,
// "Efficient generation of networks with given expected degrees", 2011), O(n + edges).
rofh_graph* rofh_chung_lu_rows(int n, const double* a_desc, const int32_t* src_id, const double* b,
                               double S, uint64_t seed, int allow_self_loops) {
  rofh_graph* g = new rofh_graph();
  RowStore& st = g->st;
  st.n = n;
  int nt = omp_get_max_threads();
  st.buf.resize(nt);
  st.row_thread.assign(n, 0);
  st.row_off.assign(n, 0);
  st.row_len.assign(n, 0);
#pragma omp parallel
  {
    int t = omp_get_thread_num();
    std::vector<int32_t>& out = st.buf[t];
#pragma omp for schedule(dynamic, 256)
    for (int v = 0; v < n; ++v) {
      SplitMix64 rng(mix_seed(seed, (uint64_t)v));
      const double bv = b[v] / S;
      size_t start = out.size();
      int64_t u = 0;
      double p = std::min(1.0, a_desc[0] * bv);
      while (u < n && p > 0.0) {
        if (p < 1.0) {
          double r = rng.uniform();
          double skip = std::floor(std::log(r) / std::log1p(-p));
          if (skip >= (double)(n - u)) break;
          u += (int64_t)skip;
        }
        if (u >= n) break;
        double q = std::min(1.0, a_desc[u] * bv);
        double r = rng.uniform();
        if (r < q / p) {
          int32_t s = src_id[u];
          if (allow_self_loops || s != v) out.push_back(s);
        }
        p = q;
        ++u;
      }
      std::sort(out.begin() + start, out.end());
      st.row_thread[v] = t;
      st.row_off[v] = (int64_t)start;
      st.row_len[v] = (int32_t)(out.size() - start);
    }
  }
  return g;
}

// Community graph: n nodes in clusters of `cluster` consecutive ids.  Every node of a
// cluster has the same `pool` in-neighbours (drawn once per cluster from its own members)
// plus `extra` distinct uniform random in-neighbours outside that pool.
rofh_graph* rofh_community_rows(int n, int cluster, int pool, int extra, uint64_t seed) {
  rofh_graph* g = new rofh_graph();
  RowStore& st = g->st;
  st.n = n;
  int nt = omp_get_max_threads();
  st.buf.resize(nt);
  st.row_thread.assign(n, 0);
  st.row_off.assign(n, 0);
  st.row_len.assign(n, 0);
  int nclusters = (n + cluster - 1) / cluster;
#pragma omp parallel
  {
    int t = omp_get_thread_num();
    std::vector<int32_t>& out = st.buf[t];
    std::vector<int32_t> members, poolv;
#pragma omp for schedule(dynamic, 64)
    for (int c = 0; c < nclusters; ++c) {
      int lo = c * cluster, hi = std::min(n, lo + cluster);
      members.resize(hi - lo);
      for (int i = lo; i < hi; ++i) members[i - lo] = i;
      SplitMix64 crng(mix_seed(seed ^ 0xC1A5C1A5ull, (uint64_t)c));
      int m = (int)members.size();
      int take = std::min(pool, m);
      for (int i = 0; i < take; ++i) {  // partial Fisher-Yates
        int j = i + (int)crng.below((uint64_t)(m - i));
        std::swap(members[i], members[j]);
      }
      poolv.assign(members.begin(), members.begin() + take);
      std::sort(poolv.begin(), poolv.end());
      for (int v = lo; v < hi; ++v) {
        SplitMix64 rng(mix_seed(seed, (uint64_t)v));
        size_t start = out.size();
        out.insert(out.end(), poolv.begin(), poolv.end());
        int got = 0;
        while (got < extra && (int)(out.size() - start) < n) {
          int32_t s = (int32_t)rng.below((uint64_t)n);
          bool dup = false;
          for (size_t k = start; k < out.size(); ++k)
            if (out[k] == s) { dup = true; break; }
          if (!dup) { out.push_back(s); ++got; }
        }
        std::sort(out.begin() + start, out.end());
        st.row_thread[v] = t;
        st.row_off[v] = (int64_t)start;
        st.row_len[v] = (int32_t)(out.size() - start);
      }
    }
  }
  return g;
}

int64_t rofh_graph_num_edges(const rofh_graph* g) {
  int64_t e = 0;
  for (int v = 0; v < g->st.n; ++v) e += g->st.row_len[v];
  return e;
}

// indptr has n+1 int64 entries, indices has num_edges int32 entries.
void rofh_graph_fetch(const rofh_graph* g, int64_t* indptr, int32_t* indices) {
  const RowStore& st = g->st;
  indptr[0] = 0;
  for (int v = 0; v < st.n; ++v) indptr[v + 1] = indptr[v] + st.row_len[v];
#pragma omp parallel for schedule(static, 1024)
  for (int v = 0; v < st.n; ++v) {
    if (st.row_len[v])
      std::memcpy(indices + indptr[v], st.buf[st.row_thread[v]].data() + st.row_off[v],
                  sizeof(int32_t) * (size_t)st.row_len[v]);
  }
}

void rofh_graph_free(rofh_graph* g) { delete g; }

// Thread count of every later OpenMP region of this library (launchers such as torchrun export
// OMP_NUM_THREADS=1, which would make the generators and the search single-threaded).
void rofh_set_num_threads(int n) { if (n > 0) omp_set_num_threads(n); }
int rofh_max_threads(void) { return omp_get_max_threads(); }

// Transpose a CSR over destinations into a CSR over sources (rows sorted ascending):
// the second CSR upstream builds from the swapped COO (middle-main.py:187-198).
void rofh_transpose_csr(int n, const int64_t* indptr, const int32_t* indices, int64_t* t_indptr,
                        int32_t* t_indices) {
  std::vector<int64_t> cnt((size_t)n + 1, 0);
  int64_t e = indptr[n];
  for (int64_t k = 0; k < e; ++k) cnt[(size_t)indices[k] + 1]++;
  t_indptr[0] = 0;
  for (int i = 0; i < n; ++i) t_indptr[i + 1] = t_indptr[i] + cnt[(size_t)i + 1];
  std::vector<int64_t> pos(t_indptr, t_indptr + n);
  for (int v = 0; v < n; ++v)  // ascending v => each output row is ascending
    for (int64_t k = indptr[v]; k < indptr[v + 1]; ++k) t_indices[pos[indices[k]]++] = v;
}

// Row-wise union of a CSR with its transpose (both with ascending rows), optionally with
// the diagonal: the symmetrised graph.  Two calls: out_indices == nullptr only fills
// out_indptr (n+1 entries); the second call fills out_indices.
void rofh_symmetrize(int n, const int64_t* indptr, const int32_t* indices, const int64_t* t_indptr,
                     const int32_t* t_indices, int add_self_loops, int64_t* out_indptr,
                     int32_t* out_indices) {
  const bool fill = out_indices != nullptr;
  if (!fill) out_indptr[0] = 0;
#pragma omp parallel for schedule(dynamic, 1024)
  for (int v = 0; v < n; ++v) {
    const int32_t* a = indices + indptr[v];
    const int32_t* ae = indices + indptr[v + 1];
    const int32_t* b = t_indices + t_indptr[v];
    const int32_t* be = t_indices + t_indptr[v + 1];
    bool self_pending = add_self_loops != 0;
    int64_t cnt = 0;
    int32_t* out = fill ? out_indices + out_indptr[v] : nullptr;
    while (a < ae || b < be || self_pending) {
      int64_t x = a < ae ? *a : INT64_MAX;
      int64_t y = b < be ? *b : INT64_MAX;
      int64_t z = self_pending ? v : INT64_MAX;
      int64_t m = std::min(x, std::min(y, z));
      if (x == m) ++a;
      if (y == m) ++b;
      if (z == m) self_pending = false;
      if (fill) out[cnt] = (int32_t)m;
      ++cnt;
    }
    if (!fill) out_indptr[v + 1] = cnt;
  }
  if (!fill)
    for (int v = 0; v < n; ++v) out_indptr[v + 1] += out_indptr[v];
}

}  // extern "C"
