// C entry points around the reference's own launchers, so tests and the bench can run the
// unmodified reference kernels (compiled from the reference tree where it lies) next to ours.
// TEST INFRASTRUCTURE: built only where the reference tree is mounted, output goes to
// oracle/_ref/ and is never committed.
#include <cuda_runtime.h>

#include "trt_engine/trt_network_crt/plugins/embedding_bag_plugin/embedding_bag_plugin.h"

extern "C" {

int ref_eb_bag(const int* input, const int* offsets, float* output, int input_size, int num_bags,
               const float* data, int count, int dim, int data_offset, int op, void* stream) {
  fwd::trt_::EmbeddingBag(input, offsets, output, input_size, num_bags, data, count, dim, data_offset,
                          op, static_cast<cudaStream_t>(stream));
  return (int)cudaGetLastError();
}

int ref_eb_bag_fixed(const int* input, float* output, int batch, int len, const float* data,
                     int count, int dim, int data_offset, int op, void* stream) {
  fwd::trt_::EmbeddingBagWithFixedOffset(input, output, batch, len, data, count, dim, data_offset, op,
                                         static_cast<cudaStream_t>(stream));
  return (int)cudaGetLastError();
}

int ref_eb_gather(const int* input, float* output, int batch, int len, const float* data, int count,
                  int dim, int data_offset, void* stream) {
  fwd::trt_::Gather(input, output, batch, len, data, count, dim, data_offset,
                    static_cast<cudaStream_t>(stream));
  return (int)cudaGetLastError();
}

}  // extern "C"
