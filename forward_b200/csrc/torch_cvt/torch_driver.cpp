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

// ---- whole graphs: every embedding bag of a module, inputs cast as Forward's engine does ------
//
// Parser (torch_module_parser.h) finds the bags and how the graph's inputs and outputs connect to
// them; this harness then plays the engine: one EmbeddingBag_TRT plugin per bag (through the layer
// creator, as above), int64 inputs cast to int32 on the device the way TorchEngine::ParseInput
// does on its way in (source/fwd_torch/torch_engine/torch_engine.cpp:134-149), the bags enqueued
// on one stream, and each graph output assembled from its bags' pooled rows (aten::cat along
// dim 1 becomes a strided device copy).

#include <cuda_runtime_api.h>

#include "torch_module_parser.h"

extern "C" {
int fwd_eb_host_run(fwd_eb_host* h, const void* d0, const void* d1, const void* d2, void* d_out, void* stream);
void fwd_eb_host_free(fwd_eb_host* h);
int fwd_eb_cast_i64_to_i32(const void* d_src, void* d_dst, long long count, void* stream);
}

struct fwd_eb_tensor_arg {
  const void* data;    // device
  int dtype;           // 0 int32, 1 int64, 2 float32
  int rank;
  long long dims[4];
  int graph_input;     // which graph input (position among the non-self inputs) ...
  int element;         // ... and which element of it when that input is a list (-1: a plain tensor)
};

struct fwd_eb_net {
  fwd::torch_::Parser parser;
  std::vector<fwd_eb_host*> engines;        // one per layer, built on the first run
  std::vector<std::vector<long long>> built_numel;   // the input sizes each engine was built for
  std::vector<void*> layer_out;             // [bags, dim] per layer
  std::vector<std::vector<void*>> cast;     // int32 copies of int64 inputs, per layer and input
  std::string error;
  ~fwd_eb_net() {
    for (auto* e : engines)
      if (e) fwd_eb_host_free(e);
    for (void* p : layer_out) cudaFree(p);
    for (auto& v : cast)
      for (void* p : v) cudaFree(p);
  }
};

extern "C" {

void fwd_eb_torch_net_free(fwd_eb_net* n) { delete n; }

fwd_eb_net* fwd_eb_torch_parse_network(const char* path, char* err, size_t err_cap) {
  std::unique_ptr<fwd_eb_net> n(new fwd_eb_net());
  if (!n->parser.Parse(path)) {
    if (err && err_cap) std::snprintf(err, err_cap, "%s", n->parser.Error().c_str());
    return nullptr;
  }
  const size_t layers = n->parser.GetNetwork().layers.size();
  n->engines.assign(layers, nullptr);
  n->built_numel.resize(layers);
  n->layer_out.assign(layers, nullptr);
  n->cast.resize(layers);
  return n.release();
}

int fwd_eb_torch_net_num_layers(const fwd_eb_net* n) { return n ? (int)n->parser.GetNetwork().layers.size() : -1; }
int fwd_eb_torch_net_num_outputs(const fwd_eb_net* n) { return n ? (int)n->parser.GetNetwork().outputs.size() : -1; }
int fwd_eb_torch_net_num_graph_inputs(const fwd_eb_net* n) { return n ? (int)n->parser.Module().Inputs().size() : -1; }
const char* fwd_eb_torch_net_error(const fwd_eb_net* n) { return n ? n->error.c_str() : ""; }

// dim / rows / op of layer i; returns the number of tensor inputs the layer takes.
int fwd_eb_torch_net_layer_info(const fwd_eb_net* n, int i, int* dim, int* count, int* op) {
  if (!n || i < 0 || i >= (int)n->parser.GetNetwork().layers.size()) return -1;
  const auto& l = n->parser.GetNetwork().layers[i];
  *dim = l.desc->dim;
  *count = l.desc->count;
  *op = l.desc->op;
  return (int)l.inputs.size();
}

// Where input j of layer i comes from (see InputRef).
int fwd_eb_torch_net_layer_input(const fwd_eb_net* n, int i, int j, int* graph_input, int* element, int* from_list) {
  if (!n || i < 0 || i >= (int)n->parser.GetNetwork().layers.size()) return -1;
  const auto& l = n->parser.GetNetwork().layers[i];
  if (j < 0 || j >= (int)l.inputs.size()) return -1;
  *graph_input = l.inputs[j].graph_input;
  *element = l.inputs[j].element;
  *from_list = l.inputs[j].from_list ? 1 : 0;
  return 0;
}

// Layers concatenated into graph output o; returns how many (dst receives up to cap of them).
int fwd_eb_torch_net_output_layers(const fwd_eb_net* n, int o, int* dst, int cap) {
  if (!n || o < 0 || o >= (int)n->parser.GetNetwork().outputs.size()) return -1;
  const auto& v = n->parser.GetNetwork().outputs[o];
  for (int k = 0; k < (int)v.size() && k < cap; ++k) dst[k] = v[k];
  return (int)v.size();
}

// Run the parsed graph.  `args` describe the device tensors the caller feeds (one per plain
// graph input, one per element of a list input).  d_outputs[o] receives graph output o as fp32
// [bags, sum of its layers' dims] (fp16 where the layers emit fp16).  0 on success.
int fwd_eb_torch_net_run(fwd_eb_net* n, const fwd_eb_tensor_arg* args, int n_args, void* const* d_outputs,
                         void* stream) {
  if (!n || !args || !d_outputs) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const auto& net = n->parser.GetNetwork();
  auto fail = [&](const std::string& why) {
    n->error = why;
    return -1;
  };
  std::vector<long long> bags(net.layers.size(), 0);
  for (size_t li = 0; li < net.layers.size(); ++li) {
    const auto& layer = net.layers[li];
    const void* ptr[3] = {nullptr, nullptr, nullptr};
    int rank[3] = {0, 0, 0};
    int dims[3][4] = {};
    std::vector<long long> numel(layer.inputs.size(), 0);
    if (n->cast[li].empty()) n->cast[li].assign(layer.inputs.size(), nullptr);
    for (size_t j = 0; j < layer.inputs.size() && j < 3; ++j) {
      const auto& ref = layer.inputs[j];
      const fwd_eb_tensor_arg* a = nullptr;
      for (int k = 0; k < n_args; ++k) {
        if (args[k].graph_input == ref.graph_input && args[k].element == (ref.from_list ? ref.element : -1)) a = &args[k];
      }
      if (!a || !a->data || a->rank < 1 || a->rank > 4) return fail("a graph input the bags need was not fed");
      const size_t item = a->dtype == 1 ? 8 : 4;
      const char* base = static_cast<const char*>(a->data);
      int r = a->rank;
      long long d[4] = {a->dims[0], a->dims[1], a->dims[2], a->dims[3]};
      if (!ref.from_list && ref.element >= 0) {  // row `element` along dim 0
        if (r < 2 || ref.element >= d[0]) return fail("aten::select index outside the fed tensor");
        long long row = 1;
        for (int q = 1; q < r; ++q) row *= d[q];
        base += (size_t)ref.element * (size_t)row * item;
        for (int q = 1; q < r; ++q) d[q - 1] = d[q];
        --r;
      }
      long long count = 1;
      for (int q = 0; q < r; ++q) count *= d[q];
      numel[j] = count;
      const bool weights = layer.desc->has_per_sample_weights && j + 1 == layer.inputs.size();
      if (weights) {
        if (a->dtype != 2) return fail("per_sample_weights must be float32");
      } else if (a->dtype == 1) {  // int64 -> int32, as TorchEngine::ParseInput does
        if (!n->cast[li][j] && cudaMalloc(&n->cast[li][j], (size_t)(count > 0 ? count : 1) * 4) != cudaSuccess)
          return fail("out of device memory for an int32 copy of an input");
        if (fwd_eb_cast_i64_to_i32(base, n->cast[li][j], count, stream) != 0) return fail("int64 -> int32 cast failed");
        base = static_cast<const char*>(n->cast[li][j]);
      } else if (a->dtype != 0) {
        return fail("indices and offsets must be int32 or int64");
      }
      ptr[j] = base;
      rank[j] = r;
      for (int q = 0; q < r; ++q) dims[j][q] = (int)d[q];
    }
    const bool two_d = rank[0] == 2;
    const int n_struct = (int)layer.inputs.size() - (layer.desc->has_per_sample_weights ? 1 : 0);
    const int w_slot = n_struct;
    bags[li] = two_d ? dims[0][0] : (n_struct > 1 ? dims[1][rank[1] - 1] - (layer.desc->include_last_offset ? 1 : 0) : 0);
    if (!n->engines[li]) {
      n->engines[li] = fwd_eb_host_build_desc(layer.desc.get(), rank[0], dims[0], two_d ? 0 : rank[1],
                                              two_d ? nullptr : dims[1],
                                              layer.desc->has_per_sample_weights ? rank[w_slot] : 0,
                                              layer.desc->has_per_sample_weights ? dims[w_slot] : nullptr);
      if (!n->engines[li]) return fail("the plugin refused a layer of the graph");
      n->built_numel[li] = numel;
      const size_t esize = layer.desc->half_output ? 2 : 4;
      const size_t out_bytes = (size_t)(bags[li] > 0 ? bags[li] : 1) * layer.desc->dim * esize;
      if (cudaMalloc(&n->layer_out[li], out_bytes) != cudaSuccess) return fail("out of device memory");
    } else if (n->built_numel[li] != numel) {
      return fail("input sizes differ from those the engine was built for");
    }
    const void* in1 = two_d ? (layer.desc->has_per_sample_weights ? ptr[w_slot] : nullptr) : ptr[1];
    const void* in2 = two_d ? nullptr : (layer.desc->has_per_sample_weights ? ptr[w_slot] : nullptr);
    if (fwd_eb_host_run(n->engines[li], ptr[0], in1, in2, n->layer_out[li], stream) != 0)
      return fail("enqueue failed");
  }
  for (size_t o = 0; o < net.outputs.size(); ++o) {
    const auto& parts = net.outputs[o];
    long long total = 0;
    for (int li : parts) total += net.layers[li].desc->dim;
    long long col = 0;
    for (int li : parts) {
      const auto& d = *net.layers[li].desc;
      const size_t esize = d.half_output ? 2 : 4;
      if (bags[li] != bags[parts[0]] || d.half_output != net.layers[parts[0]].desc->half_output)
        return fail("bags concatenated into one output differ in batch size or element type");
      if (cudaMemcpy2DAsync(static_cast<char*>(d_outputs[o]) + col * esize, (size_t)total * esize,
                            n->layer_out[li], (size_t)d.dim * esize, (size_t)d.dim * esize,
                            (size_t)bags[li], cudaMemcpyDeviceToDevice, st) != cudaSuccess)
        return fail("assembling an output failed");
      col += d.dim;
    }
  }
  return 0;
}

}  // extern "C"
