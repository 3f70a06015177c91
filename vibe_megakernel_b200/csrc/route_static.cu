// moe_route_static: the router for callers that may not allocate device memory.
//
// moe_route needs a caller-provided workspace for its logits and selection arrays. Some hosts of
// this library cannot supply one: a plugin that is handed only its input and output buffers and
// whose host forbids cudaMalloc once serving has started (an allocation synchronises the device
// and can fail under a capped memory pool), or a thin FFI wrapper that has no allocator at all.
// For them the same kernels run with their scratch in an array that is part of this library's
// device image: every GPU that loads the library holds kStaticBytes of it until the process
// exits, whether or not this entry point is ever called.
//
// What follows from that:
//   * sizes are capped (MOE_STATIC_ROUTE_MAX_TOKENS tokens, MOE_STATIC_ROUTE_MAX_EXPERTS experts, MOE_MAX_TOPK
//     picks); larger requests are refused with MOE_ERR_TOO_LARGE, nothing is launched;
//   * all calls on one GPU share the array. It keeps whatever the previous call left; the router
//     writes every element it later reads, so nothing has to be cleared first. Two calls whose
//     kernels can overlap on the GPU (different streams, or different host threads) race on it:
//     keep calls to this entry point on one stream, or order them yourself;
//   * the first call on each device looks the array's device address up (set-up, below). Make
//     that first call outside any stream capture.
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace {

constexpr size_t kLogitFloats = static_cast<size_t>(MOE_STATIC_ROUTE_MAX_TOKENS) * MOE_STATIC_ROUTE_MAX_EXPERTS;
constexpr size_t kPickWords = static_cast<size_t>(MOE_STATIC_ROUTE_MAX_TOKENS) * MOE_MAX_TOPK;
constexpr size_t kStaticBytes = (kLogitFloats + 2 * kPickWords) * 4;     // 557,056 bytes

// In host code this name is only a handle for the runtime: it is not a device address and must
// never be passed to a kernel. The address comes from cudaGetSymbolAddress, per device.
static __device__ __align__(256) unsigned char g_route_scratch[kStaticBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_lock;
void* g_scratch_on_device[kMaxDevices] = {};

// Once per device, with that device current: ask the runtime where this device's copy lives.
int scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return MOE_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> hold(g_setup_lock);
  if (!g_scratch_on_device[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_route_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (!ptr) return MOE_ERR_DRIVER;
    g_scratch_on_device[dev] = ptr;
  }
  *out = g_scratch_on_device[dev];
  return MOE_OK;
}

}  // namespace

extern "C" int moe_route_static(const moe_config_t* cfg, const void* x_bf16, const float* router,
                                const float* router_bias, int32_t tokens, int64_t* expert_ids, float* weights,
                                void* stream) {
  if (!cfg || !x_bf16 || !router) return MOE_ERR_BAD_ARG;
  if (tokens < 1) return MOE_ERR_BAD_ARG;
  if (tokens > MOE_STATIC_ROUTE_MAX_TOKENS || cfg->n_experts > MOE_STATIC_ROUTE_MAX_EXPERTS || cfg->topk > MOE_MAX_TOPK)
    return MOE_ERR_TOO_LARGE;
  const int rc = moe_workspace_layout(cfg, tokens, nullptr);   // same geometry checks as moe_route
  if (rc != MOE_OK) return rc;
  void* base = nullptr;
  const int sc = scratch_for_current_device(&base);
  if (sc != MOE_OK) return sc;
  float* logits = static_cast<float*>(base);
  int32_t* ids32 = reinterpret_cast<int32_t*>(logits + kLogitFloats);
  float* picked = reinterpret_cast<float*>(ids32 + kPickWords);
  int launches = 0;
  const cudaError_t e = moe::launch_router(*cfg, static_cast<const __nv_bfloat16*>(x_bf16), router, router_bias,
                                           tokens, logits, ids32, picked, expert_ids, weights,
                                           static_cast<cudaStream_t>(stream), &launches);
  return e == cudaSuccess ? MOE_OK : static_cast<int>(e);
}
