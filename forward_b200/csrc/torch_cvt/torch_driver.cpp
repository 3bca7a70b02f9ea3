// Test harness for the torch parser slice: TorchScript file -> graph -> description creator
// -> TrtEmbeddingBagDesc, and on into the TensorRT-side layer creator and plugin (through the
// host driver of libfwd_eb_plugin.so).  This is the "parsed model picks the plugin up" chain of
// Forward (Parser::ParseValue, source/fwd_torch/torch_cvt/torch_module_parser.cpp:104-163, then
// TrtNetworkCreator, source/trt_engine/trt_network_crt/trt_network_creator.cpp:54-69) cut down
// to the one node this repository handles.  Not part of the product ABI.
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "torch_desc_manager.h"

struct fwd_eb_host;
extern "C" fwd_eb_host* fwd_eb_host_build_desc(const void* embedding_bag_desc, int idx_rank,
                                               const int* idx_dims, int off_rank, const int* off_dims,
                                               int weights_rank, const int* weights_dims);

struct fwd_eb_parsed {
  fwd::torch_::TorchModule module;
  std::shared_ptr<fwd::TrtEmbeddingBagDesc> desc;
  std::vector<std::string> input_names;
  std::string node_text;
};

extern "C" {

void fwd_eb_torch_free(fwd_eb_parsed* p) { delete p; }

// Returns nullptr and writes the reason to `err` when the file does not load, holds no
// aten::embedding_bag node, or the node cannot be converted faithfully.
fwd_eb_parsed* fwd_eb_torch_parse(const char* path, char* err, size_t err_cap) {
  auto fail = [&](const std::string& why) -> fwd_eb_parsed* {
    if (err && err_cap) std::snprintf(err, err_cap, "%s", why.c_str());
    return nullptr;
  };
  std::unique_ptr<fwd_eb_parsed> p(new fwd_eb_parsed());
  if (!p->module.Load(path)) return fail("load failed: " + p->module.Error());
  fwd::torch_::TorchDescManager manager;
  for (const fwd::torch_::JitNode* node : p->module.Graph()->nodes()) {
    fwd::torch_::ILayerDescCreator* creator = manager.FindDescCreator(node, p->module);
    if (!creator) continue;  // a node of another operator: not ours to convert
    std::vector<const fwd::torch_::JitValue*> inputs;
    std::shared_ptr<fwd::TrtLayerDesc> desc = creator->Create(node, p->module, inputs);
    if (!desc) return fail("the EmbeddingBag description creator rejected the node");
    p->desc = std::dynamic_pointer_cast<fwd::TrtEmbeddingBagDesc>(desc);
    if (!p->desc || p->desc->Name() != "EmbeddingBag") return fail("unexpected description type");
    for (const auto* v : inputs) p->input_names.push_back(v->debugName());
    return p.release();
  }
  return fail("no aten::embedding_bag node in the graph");
}

int fwd_eb_torch_desc_info(const fwd_eb_parsed* p, int* dim, int* count, int* offset, int* op,
                           long long* padding_idx, int* include_last_offset, int* weighted,
                           int* half_table, int* half_output) {
  if (!p || !p->desc) return -1;
  const auto& d = *p->desc;
  *dim = d.dim;
  *count = d.count;
  *offset = d.offset;
  *op = d.op;
  *padding_idx = d.padding_idx;
  *include_last_offset = d.include_last_offset;
  *weighted = d.has_per_sample_weights;
  *half_table = d.data.Type() == nvinfer1::DataType::kHALF;
  *half_output = d.half_output;
  return (int)p->input_names.size();
}

const char* fwd_eb_torch_input_name(const fwd_eb_parsed* p, int i) {
  return (p && i >= 0 && i < (int)p->input_names.size()) ? p->input_names[i].c_str() : "";
}

size_t fwd_eb_torch_desc_weights(const fwd_eb_parsed* p, void* dst, size_t cap) {
  if (!p || !p->desc) return 0;
  const size_t n = (size_t)p->desc->data.Bytes();
  if (dst && cap >= n) std::memcpy(dst, p->desc->data.Data(), n);
  return n;
}

// On into the TensorRT side: the description goes through LayerCreatorManager ->
// TLayerCreator<TrtEmbeddingBagDesc> -> EmbeddingBag_TRT plugin; the handle is a fwd_eb_host of
// the plugin library (run it with fwd_eb_host_run).
fwd_eb_host* fwd_eb_torch_build_engine(const fwd_eb_parsed* p, int idx_rank, const int* idx_dims,
                                       int off_rank, const int* off_dims, int weights_rank,
                                       const int* weights_dims) {
  if (!p || !p->desc) return nullptr;
  return fwd_eb_host_build_desc(p->desc.get(), idx_rank, idx_dims, off_rank, off_dims, weights_rank,
                                weights_dims);
}

}  // extern "C"
