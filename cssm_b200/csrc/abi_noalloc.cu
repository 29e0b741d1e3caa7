// cssm_gated_forward_static: the gated block for callers that cannot allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: a plugin called from inside
// another framework's execution of a step (where the framework's allocator owns all device
// memory and a driver allocation would stall or fragment it), or a real-time / sandboxed
// service that is only allowed to launch work.  For them the scratch memory of the block
// (the planar x_main/z planes, the plane sums and the gate maps) lives in one fixed
// array that is part of the loaded library image on every GPU that loads it.
#include <mutex>
#include "common.cuh"

namespace cssm {

constexpr size_t STATIC_SCRATCH_BYTES = (size_t)64 << 20;   // 64 MiB per GPU, held until exit

// File-scope device array.  In host code this name is only a handle for the runtime, never a
// device address: the address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
static std::mutex g_mu;
static void* g_scratch_ptr[MAX_DEVICES] = {nullptr};

// Device address of the scratch array on the CURRENT device; resolved once per device and kept
// for the life of the process.  The address belongs to the device's primary context: after
// cudaDeviceReset (or after a host framework has destroyed and re-created that context) it is
// stale and this entry point must not be called again in that process.
static int static_scratch(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  if (dev < 0 || dev >= MAX_DEVICES) return CSSM_ERR_SIZE_LIMIT;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
    if (p == nullptr) return CSSM_ERR_CUDA;
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return CSSM_OK;
}

}  // namespace cssm

using namespace cssm;

extern "C" {

size_t cssm_static_scratch_bytes(void) { return STATIC_SCRATCH_BYTES; }

int cssm_gated_forward_static(const cssm_gated_desc* d, const cssm_gated_weights* w,
                              const void* plan, const float* x, float* y, void* stream) {
  if (!d) return CSSM_ERR_NULL;
  const size_t need = cssm_gated_workspace_bytes(d);
  if (need == 0) {
    cssm_gated_ws_layout l;
    return cssm_gated_workspace_layout(d, &l);     // reports why the descriptor is rejected
  }
  if (need > STATIC_SCRATCH_BYTES) return CSSM_ERR_SIZE_LIMIT;
  void* scratch = nullptr;
  const int s = static_scratch(&scratch);
  if (s != CSSM_OK) return s;
  // Every part of the scratch (planes, plane sums, gate maps) is fully written by the block's
  // own kernels before it is read, so nothing has to be cleared between calls.
  return cssm_gated_forward(d, w, plan, x, y, scratch, STATIC_SCRATCH_BYTES, stream);
}

}  // extern "C"
