// fwd_eb_forward_static_scratch: the split-bag pooling path for hosts that are
// not allowed to allocate device memory.
//
// Some embedders hand this library a fixed set of buffers and forbid every
// allocation afterwards: a TensorRT plugin built with getWorkspaceSize() == 0
// (the reference plugin's contract, embedding_bag_plugin.cpp:129-133) gets no
// workspace pointer in enqueue(), and a serving loop that has frozen its
// memory pool, or runs inside a region where cudaMalloc would synchronise the
// device, cannot ask for one either.  For them the scratch the split strategy
// needs lives in a fixed array inside this library's device image.
//
// The array is file-scope device memory: each GPU that loads the library
// carries its own 8 MiB copy from module load until the process exits.  In host
// code the array's name is only a handle for the runtime, not an address a
// kernel may use, so the device address is looked up once per device with
// cudaGetSymbolAddress (that device being current) and cached.
#include <mutex>

#include "eb_internal.h"
#include "fwd_eb.h"

namespace {

static __device__ __align__(256) unsigned char g_static_scratch[FWD_EB_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_lock;
void* g_scratch_ptr[kMaxDevices] = {};

// Device address of g_static_scratch on the current device (cached per ordinal).
int scratch_address(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fwd_eb::cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices)
    return fwd_eb::fail(FWD_EB_ETOOBIG, "device ordinal %d beyond the %d this entry point tracks",
                        dev, kMaxDevices);
  std::lock_guard<std::mutex> hold(g_lock);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return fwd_eb::cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
    if (!p) return fwd_eb::fail(FWD_EB_EINVAL, "static scratch has no device address");
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace

extern "C" int fwd_eb_forward_static_scratch(const fwd_eb_params* p, void* stream) {
  if (!p) return fwd_eb::fail(FWD_EB_EINVAL, "params is null");
  if (p->mode == FWD_EB_MODE_GATHER)
    return fwd_eb::fail(FWD_EB_EINVAL, "GATHER pools nothing and needs no scratch: use fwd_eb_forward");
  fwd_eb_params q = *p;
  q.strategy = FWD_EB_STRATEGY_SPLIT;
  q.workspace = nullptr;
  q.workspace_bytes = 0;
  // Size check first: pure host arithmetic, so an oversized call is refused before any CUDA call.
  const size_t need = fwd_eb_workspace_size(&q);
  if (need > (size_t)FWD_EB_STATIC_SCRATCH_BYTES)
    return fwd_eb::fail(FWD_EB_ETOOBIG,
                        "call needs %zu bytes of split scratch but the built-in array holds %zu: "
                        "use fewer or narrower bags per call, or fwd_eb_forward with your own workspace",
                        need, (size_t)FWD_EB_STATIC_SCRATCH_BYTES);
  void* scratch = nullptr;
  int rc = scratch_address(&scratch);
  if (rc) return rc;
  q.workspace = scratch;
  q.workspace_bytes = FWD_EB_STATIC_SCRATCH_BYTES;
  return fwd_eb_forward(&q, stream);
}

extern "C" int fwd_eb_static_scratch_prepare(void) {
  void* scratch = nullptr;
  return scratch_address(&scratch);
}
