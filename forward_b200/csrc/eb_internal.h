// Shared by the translation units of libfwd_eb.so; not part of the public ABI.
#pragma once

#include <cuda_runtime.h>

struct fwd_eb_params;

namespace fwd_eb {

// Record the calling thread's error text and hand back `code`.
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
void clear_error();
void count_launch();

struct PoolArgs;
// Validate `p` and fill the kernel arguments for the lane-group strategy (shared by the
// single-GPU launcher and the row-shard push).  vec / cpl / tiles describe the chosen shape.
// *stream = 1 when the streaming kernel (eb_stream.cuh) should run the shape (args->stream_k is
// then set), 2 for the lean kernel (eb_lite.cuh), 0 for eb_pool_group_kernel.
int plan_group(const struct ::fwd_eb_params* p, PoolArgs* args, int* vec, int* cpl, int* tiles, int* stream);
int sm_count();

}  // namespace fwd_eb
