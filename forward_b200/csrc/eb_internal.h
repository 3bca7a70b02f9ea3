// Shared by the translation units of libfwd_eb.so; not part of the public ABI.
#pragma once

#include <cuda_runtime.h>

#include <nvtx3/nvToolsExt.h>   // header-only: no library to link, calls are no-ops without a tool attached

#include <cstdlib>

struct fwd_eb_params;

namespace fwd_eb {

// Record the calling thread's error text and hand back `code`.
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
void clear_error();
void count_launch();

// A named NVTX range around a host-side entry point (what a timeline tool shows around the
// launches it queues), only when FWD_EB_NVTX=1 is set in the environment (read once).
inline bool nvtx_on() {
  static const bool on = [] {
    const char* e = std::getenv("FWD_EB_NVTX");
    return e && e[0] == '1';
  }();
  return on;
}
struct NvtxRange {
  explicit NvtxRange(const char* name) : on_(nvtx_on()) {
    if (on_) nvtxRangePushA(name);
  }
  ~NvtxRange() {
    if (on_) nvtxRangePop();
  }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
  bool on_;
};

struct PoolArgs;
// Validate `p` and fill the kernel arguments for the lane-group strategy (shared by the
// single-GPU launcher and the row-shard push).  vec / cpl / tiles describe the chosen shape.
// *stream = 1 when the streaming kernel (eb_stream.cuh) should run the shape (args->stream_k is
// then set), 2 for the lean kernel (eb_lite.cuh), 0 for eb_pool_group_kernel.
int plan_group(const struct ::fwd_eb_params* p, PoolArgs* args, int* vec, int* cpl, int* tiles, int* stream);
int sm_count();

}  // namespace fwd_eb
