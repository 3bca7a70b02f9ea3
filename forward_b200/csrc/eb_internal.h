// Shared by the translation units of libfwd_eb.so; not part of the public ABI.
#pragma once

#include <cuda_runtime.h>

namespace fwd_eb {

// Record the calling thread's error text and hand back `code`.
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
void clear_error();
void count_launch();

}  // namespace fwd_eb
