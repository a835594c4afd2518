/* A torch-free C host of the library: plan from host index arrays, device buffers from the CUDA
 * runtime, one aggregation pass, check on the host.  Built and run by tests/test_gpu_c_host.py. */
#include <cuda_runtime_api.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include "rof_b200.h"

#define N 64
#define D 12
#define CHECK_CUDA(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA: %s\n", cudaGetErrorString(e_)); return 2; } } while (0)
#define CHECK_ROF(x) do { int s_ = (x); if (s_ != ROF_OK) { printf("rof status %d: %s\n", s_, rof_last_error()); return 3; } } while (0)

int main(void) {
  /* ring graph: node v aggregates v+1, v+2 and v+5 (mod N); one part of size 3 per node */
  int32_t col[3 * N], part_ptr[N + 1], part2node[N];
  for (int v = 0; v < N; ++v) {
    col[3 * v] = (v + 1) % N; col[3 * v + 1] = (v + 2) % N; col[3 * v + 2] = (v + 5) % N;
    part_ptr[v] = 3 * v; part2node[v] = v;
  }
  part_ptr[N] = 3 * N;
  static float x[N * D], deg[N], out[N * D];
  for (int n = 0; n < N; ++n) { deg[n] = 3.0f; for (int d = 0; d < D; ++d) x[n * D + d] = (float)n + 0.125f * (float)d; }

  rof_plan* plan = NULL;
  CHECK_ROF(rof_plan_create_parts(&plan, ROF_ON_HOST, N, 0, N, col, 3 * N, part_ptr, part2node, N, NULL));
  rof_plan_info info;
  CHECK_ROF(rof_plan_get_info(plan, &info));
  if (info.gather_entries != 3 * N || info.num_groups != 0) { printf("unexpected plan\n"); return 4; }

  float *d_x, *d_deg, *d_out; void* d_ws = NULL;
  int64_t ws_bytes = rof_plan_workspace_bytes(plan, D);
  CHECK_CUDA(cudaMalloc((void**)&d_x, sizeof x)); CHECK_CUDA(cudaMalloc((void**)&d_deg, sizeof deg));
  CHECK_CUDA(cudaMalloc((void**)&d_out, sizeof out));
  if (ws_bytes > 0) CHECK_CUDA(cudaMalloc(&d_ws, (size_t)ws_bytes));
  CHECK_CUDA(cudaMemcpy(d_x, x, sizeof x, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(d_deg, deg, sizeof deg, cudaMemcpyHostToDevice));
  cudaStream_t stream;
  CHECK_CUDA(cudaStreamCreate(&stream));

  int bad = 0;
  for (int mode = ROF_MODE_GCN; mode <= ROF_MODE_MEAN; ++mode) {
    CHECK_ROF(rof_aggregate(plan, mode, d_x, D, D, d_deg, d_out, D, NULL, d_ws, ws_bytes, stream));
    CHECK_CUDA(cudaMemcpyAsync(out, d_out, sizeof out, cudaMemcpyDeviceToHost, stream));
    CHECK_CUDA(cudaStreamSynchronize(stream));
    for (int v = 0; v < N; ++v)
      for (int d = 0; d < D; ++d) {
        double s = (double)x[((v + 1) % N) * D + d] + x[((v + 2) % N) * D + d] + x[((v + 5) % N) * D + d];
        double want = mode == ROF_MODE_SUM ? s : s / 3.0;          /* gcn: rsqrt(3)*rsqrt(3) = 1/3 too */
        if (fabs((double)out[v * D + d] - want) > 1e-6 + 1e-5 * fabs(want)) ++bad;
      }
  }
  /* status instead of a crash on a bad call */
  if (rof_aggregate(plan, 7, d_x, D, D, d_deg, d_out, D, NULL, d_ws, ws_bytes, stream) != ROF_ERR_BAD_ARGUMENT) ++bad;
  if (rof_aggregate(plan, ROF_MODE_SUM, d_x, D - 1, D, d_deg, d_out, D, NULL, d_ws, ws_bytes, stream) != ROF_ERR_BAD_ARGUMENT) ++bad;

  rof_plan_destroy(plan);
  cudaFree(d_x); cudaFree(d_deg); cudaFree(d_out); cudaFree(d_ws); cudaStreamDestroy(stream);
  printf(bad ? "MISMATCH %d\n" : "OK %d\n", bad ? bad : rof_last_launch_count());
  return bad ? 1 : 0;
}
