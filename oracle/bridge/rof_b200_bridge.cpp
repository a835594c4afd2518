// Reference-side binding of librof_b200 (test infrastructure; built by oracle/build_bridge.py).
//
// Upstream's pybind layer (ROF/reuse_conv/reuse_conv.cpp:1-118 declarations, :132-346 checked
// wrappers, :353-365 module) calls seven functions that upstream defines in
// reuse_conv_kernel.cu.  This file defines the same seven functions on top of the C ABI of
// include/rof_b200.h, so that upstream's reuse_conv.cpp — compiled unmodified, from where it
// lies — links against the new kernels instead of its own: the swap a maintainer of upstream
// would make.  torch stays in charge of memory, streams and the dense products, as in upstream
// (reuse_conv_kernel.cu:302, 382-383, 621, 819-820, 971, 1050-1051).
#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>

#include <map>
#include <mutex>
#include <vector>

#include "rof_b200.h"

namespace {

void ok(int rc, const char* what) { TORCH_CHECK(rc == ROF_OK, what, ": ", rof_last_error()); }

// One plan per distinct set of index tensors (keyed by address, length and version counter; the
// cache keeps the tensors alive so that an address cannot be reused while its entry exists).
struct Entry {
  rof_plan* plan;
  std::vector<torch::Tensor> keep;
};
std::mutex g_mutex;
std::map<std::vector<int64_t>, Entry> g_plans;

std::vector<int64_t> key_of(int layout, int64_t n, const std::vector<torch::Tensor>& t) {
  std::vector<int64_t> k{layout, n};
  for (const auto& x : t) {
    k.push_back(reinterpret_cast<int64_t>(x.data_ptr()));
    k.push_back(x.numel());
    k.push_back((int64_t)x._version());
  }
  return k;
}

const int32_t* i32(const torch::Tensor& t) {
  TORCH_CHECK(t.scalar_type() == torch::kInt32, "index tensors must be int32 (ROF_main.py:143-161)");
  return t.data_ptr<int32_t>();
}

void* stream() { return (void*)at::cuda::getCurrentCUDAStream().stream(); }

rof_plan* plan_parts(int64_t n, const torch::Tensor& col, const torch::Tensor& pp, const torch::Tensor& p2n) {
  std::lock_guard<std::mutex> lock(g_mutex);
  auto key = key_of(0, n, {col, pp, p2n});
  auto it = g_plans.find(key);
  if (it != g_plans.end()) return it->second.plan;
  rof_plan* p = nullptr;
  ok(rof_plan_create_parts(&p, ROF_ON_DEVICE, (int)n, 0, (int)n, i32(col), col.numel(), i32(pp), i32(p2n),
                           (int)p2n.numel(), stream()),
     "rof_plan_create_parts");
  g_plans[key] = Entry{p, {col, pp, p2n}};
  return p;
}

rof_plan* plan_v1(int64_t n, const torch::Tensor& col, const torch::Tensor& pp, const torch::Tensor& p2n,
                  const torch::Tensor& flag, const torch::Tensor& ppc, const torch::Tensor& cic) {
  std::lock_guard<std::mutex> lock(g_mutex);
  auto key = key_of(1, n, {col, pp, p2n, flag, ppc, cic});
  auto it = g_plans.find(key);
  if (it != g_plans.end()) return it->second.plan;
  rof_plan* p = nullptr;
  const int groups = ppc.numel() > 0 ? (int)ppc.numel() - 1 : 0;
  ok(rof_plan_create_v1(&p, ROF_ON_DEVICE, (int)n, 0, (int)n, i32(col), col.numel(), i32(pp), i32(p2n),
                        (int)p2n.numel(), i32(flag), i32(ppc), i32(cic), groups, stream()),
     "rof_plan_create_v1");
  g_plans[key] = Entry{p, {col, pp, p2n, flag, ppc, cic}};
  return p;
}

rof_plan* plan_v2(int64_t n, const torch::Tensor& col, const torch::Tensor& up, const torch::Tensor& nptr,
                  const torch::Tensor& ncol) {
  std::lock_guard<std::mutex> lock(g_mutex);
  auto key = key_of(2, n, {col, up, nptr, ncol});
  auto it = g_plans.find(key);
  if (it != g_plans.end()) return it->second.plan;
  rof_plan* p = nullptr;
  const int uniq = up.numel() > 0 ? (int)up.numel() - 1 : 0;
  ok(rof_plan_create_v2(&p, ROF_ON_DEVICE, (int)n, 0, (int)n, i32(col), col.numel(), i32(up), i32(nptr), i32(ncol), uniq,
                        stream()),
     "rof_plan_create_v2");
  g_plans[key] = Entry{p, {col, up, nptr, ncol}};
  return p;
}

// out = aggregate(x) over the plan; `cache` is upstream's part_result_cache ([G, D+1]) or undefined
torch::Tensor aggregate(rof_plan* p, int mode, const torch::Tensor& x, const torch::Tensor& degrees,
                        const torch::Tensor* cache) {
  TORCH_CHECK(x.scalar_type() == torch::kFloat32 && x.dim() == 2, "features must be a 2-D float32 tensor");
  const int64_t n = x.size(0), d = x.size(1);
  auto out = torch::empty({n, d}, x.options());
  const int64_t need = rof_plan_workspace_bytes(p, (int)d);
  auto ws = torch::empty({std::max<int64_t>(need, 256)}, x.options().dtype(torch::kUInt8));
  float* cache_ptr = nullptr;
  if (cache != nullptr && cache->defined() && cache->numel() > 0) {
    rof_plan_info info;
    ok(rof_plan_get_info(p, &info), "rof_plan_get_info");
    TORCH_CHECK(cache->size(0) == info.num_groups && cache->size(1) == d + 1,
                "part_result_cache must be [reuse_size, out_channels + 1]");
    cache_ptr = cache->data_ptr<float>();
  }
  ok(rof_aggregate(p, mode, x.data_ptr<float>(), n > 1 ? x.stride(0) : d, (int)d,
                   degrees.defined() ? degrees.data_ptr<float>() : nullptr, out.data_ptr<float>(), d, cache_ptr,
                   ws.data_ptr(), ws.numel(), stream()),
     "rof_aggregate");
  return out;
}

std::vector<torch::Tensor> backward_tail(const torch::Tensor& d_prime, const torch::Tensor& X, const torch::Tensor& W) {
  return {torch::mm(d_prime, W.transpose(0, 1)), torch::mm(X.transpose(0, 1), d_prime)};
}

}  // namespace

// reuse_conv.cpp:11-20
torch::Tensor SAG_cuda(torch::Tensor input, torch::Tensor row_pointers, torch::Tensor column_index,
                       torch::Tensor degrees, torch::Tensor part_pointers, torch::Tensor part2Node, int partSize,
                       int dimWorker, int warpPerBlock) {
  (void)row_pointers; (void)partSize; (void)dimWorker; (void)warpPerBlock;
  return aggregate(plan_parts(input.size(0), column_index, part_pointers, part2Node), ROF_MODE_SUM, input, degrees,
                   nullptr);
}

// reuse_conv.cpp:23-33
std::vector<torch::Tensor> spmm_forward_cuda_GNNA(torch::Tensor input, torch::Tensor weight, torch::Tensor column_index,
                                                  torch::Tensor degrees, torch::Tensor part_pointers,
                                                  torch::Tensor part2Node, int partSize, int dimWorker,
                                                  int warpPerBlock) {
  (void)partSize; (void)dimWorker; (void)warpPerBlock;
  auto tmp = torch::mm(input, weight);
  return {aggregate(plan_parts(input.size(0), column_index, part_pointers, part2Node), ROF_MODE_GCN, tmp, degrees,
                    nullptr)};
}

// reuse_conv.cpp:36-47
std::vector<torch::Tensor> spmm_backward_cuda_GNNA(torch::Tensor d_output, torch::Tensor X, torch::Tensor weight,
                                                   torch::Tensor column_index, torch::Tensor degrees,
                                                   torch::Tensor part_pointers, torch::Tensor part2Node, int partSize,
                                                   int dimWorker, int warpPerBlock) {
  (void)partSize; (void)dimWorker; (void)warpPerBlock;
  auto dp = aggregate(plan_parts(d_output.size(0), column_index, part_pointers, part2Node), ROF_MODE_GCN, d_output,
                      degrees, nullptr);
  return backward_tail(dp, X, weight);
}

// reuse_conv.cpp:50-65
std::vector<torch::Tensor> reuse_spmm_forward_cuda_v1(torch::Tensor input, torch::Tensor weight,
                                                      torch::Tensor column_index, torch::Tensor degrees,
                                                      torch::Tensor part_pointers, torch::Tensor part2Node,
                                                      int partSize, int dimWorker, int warpPerBlock,
                                                      torch::Tensor part_result_cache,
                                                      torch::Tensor part_cache_flagindex,
                                                      torch::Tensor part_pointers_cache,
                                                      torch::Tensor column_index_cache) {
  (void)partSize; (void)dimWorker; (void)warpPerBlock;
  auto tmp = torch::mm(input, weight);
  rof_plan* p = plan_v1(input.size(0), column_index, part_pointers, part2Node, part_cache_flagindex,
                        part_pointers_cache, column_index_cache);
  return {aggregate(p, ROF_MODE_GCN, tmp, degrees, &part_result_cache)};
}

// reuse_conv.cpp:68-85
std::vector<torch::Tensor> reuse_spmm_backward_cuda_v1(torch::Tensor d_output, torch::Tensor X, torch::Tensor weight,
                                                       torch::Tensor column_index, torch::Tensor degrees,
                                                       torch::Tensor part_pointers, torch::Tensor part2Node,
                                                       int partSize, int dimWorker, int warpPerBlock,
                                                       torch::Tensor cache_result, torch::Tensor part_cache_flag,
                                                       torch::Tensor part_pointers_cache,
                                                       torch::Tensor column_index_cache) {
  (void)partSize; (void)dimWorker; (void)warpPerBlock;
  rof_plan* p = plan_v1(d_output.size(0), column_index, part_pointers, part2Node, part_cache_flag,
                        part_pointers_cache, column_index_cache);
  return backward_tail(aggregate(p, ROF_MODE_GCN, d_output, degrees, &cache_result), X, weight);
}

// reuse_conv.cpp:89-101
std::vector<torch::Tensor> reuse_spmm_forward_cuda_v2(torch::Tensor input, torch::Tensor weight,
                                                      torch::Tensor uniqpart_column_index, torch::Tensor degrees,
                                                      torch::Tensor uniqpart_pointers, torch::Tensor part2Node_ptr,
                                                      torch::Tensor part2Node_col, int partSize, int dimWorker,
                                                      int warpPerBlock) {
  (void)partSize; (void)dimWorker; (void)warpPerBlock;
  auto tmp = torch::mm(input, weight);
  rof_plan* p = plan_v2(input.size(0), uniqpart_column_index, uniqpart_pointers, part2Node_ptr, part2Node_col);
  return {aggregate(p, ROF_MODE_GCN, tmp, degrees, nullptr)};
}

// reuse_conv.cpp:105-118
std::vector<torch::Tensor> reuse_spmm_backward_cuda_v2(torch::Tensor d_output, torch::Tensor X, torch::Tensor weight,
                                                       torch::Tensor uniqpart_column_index, torch::Tensor degrees,
                                                       torch::Tensor uniqpart_pointers, torch::Tensor part2Node_ptr,
                                                       torch::Tensor part2Node_col, int partSize, int dimWorker,
                                                       int warpPerBlock) {
  (void)partSize; (void)dimWorker; (void)warpPerBlock;
  rof_plan* p = plan_v2(d_output.size(0), uniqpart_column_index, uniqpart_pointers, part2Node_ptr, part2Node_col);
  return backward_tail(aggregate(p, ROF_MODE_GCN, d_output, degrees, nullptr), X, weight);
}
