// rof_aggregate_static_scratch: the aggregation pass for hosts that must not allocate.
//
// Some processes that load this library cannot give rof_aggregate() a workspace because they
// cannot obtain device memory at the time of the call: a serving process that handed all of
// HBM to its own pool at start-up and has no spare block to lend, or a caller sitting in a
// latency-critical section where a device allocation (which synchronises the whole device)
// is not acceptable.  For them the scratch that phase A (partial-sum rows of the reuse groups)
// and phase B (segment sums of split rows) need lives in the fixed device array below, which
// every GPU that loads the library reserves once and keeps until the process exits.
//
// The price is the fixed size, ROF_STATIC_SCRATCH_BYTES (32 MiB): a pass whose
// rof_plan_workspace_bytes(plan, dim) is larger is refused with ROF_ERR_WORKSPACE and nothing
// is launched.  All calls on one GPU share the array and it keeps whatever the last call left
// in it; a pass writes every scratch row before it reads it, so nothing needs clearing, but two
// passes that overlap on the GPU (different streams, or the same plan from two threads) would
// overwrite each other's rows — callers must keep such calls ordered.
//
// Set-up: the array's name is a host-side stand-in, not a device address, so the address is
// looked up with cudaGetSymbolAddress — once per device, with that device current, on the
// first call made on that device.  That first call should therefore be made during start-up,
// before any stream capture begins — and, because CUDA loads this module lazily, before the host
// gives the rest of HBM away: the lookup is what makes the driver back the array with memory.
// The address is cached per device ordinal for the life of the process; it does not survive a
// cudaDeviceReset().
#include <mutex>

#include "rof_internal.h"

namespace {

constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_scratch[ROF_STATIC_SCRATCH_BYTES];

std::mutex g_lookup_mutex;
void* g_scratch_address[kMaxDevices] = {nullptr};

// Device address of g_static_scratch on the current device (looked up once per device).
int static_scratch_address(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return rof::cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) {
    rof::set_error("rof_aggregate_static_scratch: device ordinal beyond the supported range");
    return ROF_ERR_BAD_ARGUMENT;
  }
  std::lock_guard<std::mutex> lock(g_lookup_mutex);
  if (g_scratch_address[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return rof::cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
    if (p == nullptr || (reinterpret_cast<uintptr_t>(p) & 255)) {
      rof::set_error("rof_aggregate_static_scratch: the static scratch has no usable device address");
      return ROF_ERR_CUDA;
    }
    g_scratch_address[dev] = p;
  }
  *out = g_scratch_address[dev];
  return ROF_OK;
}

}  // namespace

extern "C" int rof_aggregate_static_scratch(const rof_plan* plan, int mode, const float* x, int64_t ldx, int dim,
                                            const float* degrees, float* out, int64_t ldo, void* stream) {
  if (plan == nullptr || dim < 0) {
    rof::set_error("rof_aggregate_static_scratch: null plan or negative dim");
    return ROF_ERR_BAD_ARGUMENT;
  }
  const int64_t need = rof_plan_workspace_bytes(plan, dim);
  if (need < 0 || need > (int64_t)ROF_STATIC_SCRATCH_BYTES) {
    rof::set_error("rof_aggregate_static_scratch: this pass needs " + std::to_string(need) +
                   " bytes of scratch but the built-in scratch holds " + std::to_string((int64_t)ROF_STATIC_SCRATCH_BYTES) +
                   "; use rof_aggregate() with a caller-provided workspace");
    return ROF_ERR_WORKSPACE;
  }
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != ROF_OK) return rc;
  return rof_aggregate_phases(plan, ROF_PHASE_ALL, mode, x, ldx, dim, degrees, out, ldo, nullptr, scratch,
                              (int64_t)ROF_STATIC_SCRATCH_BYTES, stream);
}
