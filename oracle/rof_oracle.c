/*
 * CPU ORACLE — TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the arithmetic of upstream's five aggregation kernels
 * (ROF/reuse_conv/reuse_conv_kernel.cu), written part-major exactly as upstream walks its
 * index tensors, so that it shares nothing with the destination-major plan the CUDA
 * library builds.  Nothing in the product may call this file; it is used by tests/,
 * by __graft_entry__.smoke() and by bench.py's cpu_baseline / reference arm.
 *
 * Parity status: upstream ships no tests, golden vectors or CPU implementation of this path
 * (four "TODO: CPU version" markers, reuse_conv.cpp:238,278,310,341), so the restatement is
 * pinned by (1) a dense D^-1/2 A D^-1/2 X check on small graphs, (2) agreement of the three
 * layouts on the same graph, and (3) upstream's own CUDA kernels compiled unmodified for
 * sm_100a and run on the GPU by the GPU test-suite (tests/test_gpu_reference_kernels.py).
 *
 * Every function takes `exact64`: 0 = emulate the fp32 kernel (each product and each add
 * rounded to float, products never fused: __fmul_rn, reuse_conv_kernel.cu:270) in the
 * sequential part order 0..P-1 (one admissible order of upstream's atomics); 1 = the same
 * sums in double with an exact 1/sqrt, the truth that tolerances are measured against.
 *
 * `mode`: 0 = GCN symmetric norm (upstream's GNNA / ROF_v1 / ROF_v2 kernels),
 *         1 = plain sum (upstream's SAG kernel, reuse_conv_kernel.cu:149-195),
 *         2 = mean (sum, then 1/deg[dst]; no upstream kernel — benchmark extension).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { MODE_GCN = 0, MODE_SUM = 1, MODE_MEAN = 2 };

/* round-to-nearest 1/sqrt(x) in fp32, the result __frsqrt_rn gives (reuse_conv_kernel.cu:254) */
static float rsqrt_rn_f32(float x) {
  long double r = 1.0L / sqrtl((long double)x);
  return (float)r;
}

static inline double rnd(double v, int exact64) { return exact64 ? v : (double)(float)v; }

static inline double src_weight(const float* degrees, int n, int mode, int exact64) {
  if (mode != MODE_GCN) return 1.0;
  return exact64 ? 1.0 / sqrt((double)degrees[n]) : (double)rsqrt_rn_f32(degrees[n]);
}

static inline double dst_scale(const float* degrees, int v, int mode, int exact64) {
  if (mode == MODE_SUM) return 1.0;
  if (mode == MODE_MEAN) {
    float d = degrees[v];
    if (d == 0.0f) return 0.0;
    return exact64 ? 1.0 / (double)d : (double)(1.0f / d);
  }
  return src_weight(degrees, v, MODE_GCN, exact64);
}

/* partial[d] = sum_{k in [beg,end)} w(col[k]) * x[col[k]][d]   (kernel inner loop, e.g. :250-274) */
static void part_sum(double* partial, const float* x, int64_t ldx, int dim, const int32_t* col,
                     int64_t beg, int64_t end, const float* degrees, int mode, int exact64) {
  for (int d = 0; d < dim; ++d) partial[d] = 0.0;
  for (int64_t k = beg; k < end; ++k) {
    int n = col[k];
    double w = src_weight(degrees, n, mode, exact64);
    const float* row = x + (int64_t)n * ldx;
    if (mode == MODE_GCN)
      for (int d = 0; d < dim; ++d) partial[d] = rnd(partial[d] + rnd(w * (double)row[d], exact64), exact64);
    else
      for (int d = 0; d < dim; ++d) partial[d] = rnd(partial[d] + (double)row[d], exact64);
  }
}

static void flush_part(double* out_row, const double* partial, int dim, double scale, int mode, int exact64) {
  if (mode == MODE_SUM)
    for (int d = 0; d < dim; ++d) out_row[d] = rnd(out_row[d] + partial[d], exact64);
  else
    for (int d = 0; d < dim; ++d) out_row[d] = rnd(out_row[d] + rnd(partial[d] * scale, exact64), exact64);
}

static void store_out(float* out, int64_t ldo, const double* acc, int num_nodes, int dim) {
  for (int v = 0; v < num_nodes; ++v)
    for (int d = 0; d < dim; ++d) out[(int64_t)v * ldo + d] = (float)acc[(int64_t)v * dim + d];
}

/* For MODE_MEAN the scale is applied once per row at the end (sum, then divide), for GCN it
 * is applied per part like upstream (reuse_conv_kernel.cu:276-283). */
static void finish_mean(double* acc, const float* degrees, int num_nodes, int dim, int exact64) {
  for (int v = 0; v < num_nodes; ++v) {
    double s = dst_scale(degrees, v, MODE_MEAN, exact64);
    for (int d = 0; d < dim; ++d) acc[(int64_t)v * dim + d] = rnd(acc[(int64_t)v * dim + d] * s, exact64);
  }
}

/*
 * Original part layout, no reuse.  mode GCN follows spmm_forward_cuda_kernel_GNNA
 * (reuse_conv_kernel.cu:230-285); mode SUM follows SAG_cuda_kernel (:149-195).
 */
int oracle_parts(float* out, int64_t ldo, const float* x, int64_t ldx, int num_nodes, int dim,
                 const int32_t* column_index, const float* degrees, const int32_t* part_pointers,
                 const int32_t* part2Node, int num_parts, int mode, int exact64) {
  double* acc = (double*)calloc((size_t)num_nodes * dim + 1, sizeof(double));
  double* partial = (double*)malloc(sizeof(double) * (dim + 1));
  if (!acc || !partial) return 1;
  for (int p = 0; p < num_parts; ++p) {
    int v = part2Node[p];
    part_sum(partial, x, ldx, dim, column_index, part_pointers[p], part_pointers[p + 1], degrees, mode, exact64);
    flush_part(acc + (int64_t)v * dim, partial, dim, dst_scale(degrees, v, mode == MODE_GCN ? MODE_GCN : MODE_SUM, exact64),
               mode == MODE_GCN ? MODE_GCN : MODE_SUM, exact64);
  }
  if (mode == MODE_MEAN) finish_mean(acc, degrees, num_nodes, dim, exact64);
  store_out(out, ldo, acc, num_nodes, dim);
  free(acc);
  free(partial);
  return 0;
}

/*
 * ROF v1: caching kernel then reusing kernel.
 *   phase A  spmm_forward_cuda_kernel_caching (:427-486): cache_result[g][0:dim] = partial of
 *            group g, cache_result[g][dim] = 1 (the "ready" flag kept in an extra float column);
 *   phase B  spmm_forward_cuda_kernel_reusing (:521-600): a part with flag>0 whose cache row is
 *            ready adds cache_result[flag-1] * scale(dst); any other part is recomputed.
 * `cache_result` is the caller's [num_groups, dim+1] buffer and is written like upstream does.
 */
int oracle_v1(float* out, int64_t ldo, const float* x, int64_t ldx, int num_nodes, int dim,
              const int32_t* column_index, const float* degrees, const int32_t* part_pointers,
              const int32_t* part2Node, int num_parts, float* cache_result, int num_groups,
              const int32_t* part_cache_flagindex, const int32_t* part_pointers_cache,
              const int32_t* column_index_cache, int mode, int exact64) {
  double* acc = (double*)calloc((size_t)num_nodes * dim + 1, sizeof(double));
  double* partial = (double*)malloc(sizeof(double) * (dim + 1));
  double* cache = (double*)malloc(sizeof(double) * ((size_t)num_groups * dim + 1));
  if (!acc || !partial || !cache) return 1;
  int pm = mode == MODE_GCN ? MODE_GCN : MODE_SUM;
  for (int g = 0; g < num_groups; ++g) {
    part_sum(cache + (int64_t)g * dim, x, ldx, dim, column_index_cache, part_pointers_cache[g],
             part_pointers_cache[g + 1], degrees, mode, exact64);
    for (int d = 0; d < dim; ++d) cache_result[(int64_t)g * (dim + 1) + d] = (float)cache[(int64_t)g * dim + d];
    cache_result[(int64_t)g * (dim + 1) + dim] = 1.0f;
  }
  for (int p = 0; p < num_parts; ++p) {
    int v = part2Node[p];
    int flag = part_cache_flagindex[p];
    int ready = flag > 0 && cache_result[(int64_t)(flag - 1) * (dim + 1) + dim] != 0.0f;
    double s = dst_scale(degrees, v, pm, exact64);
    if (!ready) {
      part_sum(partial, x, ldx, dim, column_index, part_pointers[p], part_pointers[p + 1], degrees, mode, exact64);
      flush_part(acc + (int64_t)v * dim, partial, dim, s, pm, exact64);
    } else {
      flush_part(acc + (int64_t)v * dim, cache + (int64_t)(flag - 1) * dim, dim, s, pm, exact64);
    }
  }
  if (mode == MODE_MEAN) finish_mean(acc, degrees, num_nodes, dim, exact64);
  store_out(out, ldo, acc, num_nodes, dim);
  free(acc);
  free(partial);
  free(cache);
  return 0;
}

/*
 * ROF v2: spmm_forward_cuda_kernel_fuse (:879-953): one partial per unique part, added to
 * every destination in part2Node_col[part2Node_ptr[u] : part2Node_ptr[u+1]].
 */
int oracle_v2(float* out, int64_t ldo, const float* x, int64_t ldx, int num_nodes, int dim,
              const int32_t* uniqpart_column_index, const float* degrees, const int32_t* uniqpart_pointers,
              const int32_t* part2Node_ptr, const int32_t* part2Node_col, int num_uniqparts, int mode,
              int exact64) {
  double* acc = (double*)calloc((size_t)num_nodes * dim + 1, sizeof(double));
  double* partial = (double*)malloc(sizeof(double) * (dim + 1));
  if (!acc || !partial) return 1;
  int pm = mode == MODE_GCN ? MODE_GCN : MODE_SUM;
  for (int u = 0; u < num_uniqparts; ++u) {
    part_sum(partial, x, ldx, dim, uniqpart_column_index, uniqpart_pointers[u], uniqpart_pointers[u + 1],
             degrees, mode, exact64);
    for (int k = part2Node_ptr[u]; k < part2Node_ptr[u + 1]; ++k) {
      int v = part2Node_col[k];
      flush_part(acc + (int64_t)v * dim, partial, dim, dst_scale(degrees, v, pm, exact64), pm, exact64);
    }
  }
  if (mode == MODE_MEAN) finish_mean(acc, degrees, num_nodes, dim, exact64);
  store_out(out, ldo, acc, num_nodes, dim);
  free(acc);
  free(partial);
  return 0;
}

/*
 * Plain (reuse-free) CSR aggregation over destinations with OpenMP — the operation the
 * benchmark names as the CPU comparison path (a CSR gather-sum as torch_scatter /
 * torch_sparse would compute it).  fp32 accumulation, one row per loop iteration.
 * Used as the timed CPU baseline; numerically it is oracle_parts with one part per row.
 */
int oracle_plain_csr(float* out, int64_t ldo, const float* x, int64_t ldx, int row_begin, int row_end,
                     int dim, const int64_t* indptr, const int32_t* indices, const float* degrees, int mode,
                     int num_threads) {
#ifdef _OPENMP
  if (num_threads > 0) omp_set_num_threads(num_threads);
#endif
#pragma omp parallel
  {
    float* acc = (float*)malloc(sizeof(float) * (dim + 1));
#pragma omp for schedule(dynamic, 64)
    for (int v = row_begin; v < row_end; ++v) {
      for (int d = 0; d < dim; ++d) acc[d] = 0.0f;
      for (int64_t k = indptr[v]; k < indptr[v + 1]; ++k) {
        int n = indices[k];
        const float* row = x + (int64_t)n * ldx;
        if (mode == MODE_GCN) {
          float w = rsqrt_rn_f32(degrees[n]);
          for (int d = 0; d < dim; ++d) acc[d] += w * row[d];
        } else {
          for (int d = 0; d < dim; ++d) acc[d] += row[d];
        }
      }
      float s = (float)dst_scale(degrees, v, mode, 0);
      float* o = out + (int64_t)v * ldo;
      if (mode == MODE_SUM)
        for (int d = 0; d < dim; ++d) o[d] = acc[d];
      else
        for (int d = 0; d < dim; ++d) o[d] = acc[d] * s;
    }
    free(acc);
  }
  return 0;
}

float oracle_rsqrt_rn(float x) { return rsqrt_rn_f32(x); }

int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
