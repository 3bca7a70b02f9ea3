// Drives the plugin the way TensorRT does, for the tests: description -> layer creator ->
// network -> "engine" (format negotiation, configure, serialise) -> fresh load through the
// registry -> enqueue.  This is the order Forward's own unit test goes through
// (source/unit_test/unit_test_torch_helper.h:147-208: build, Save, Load, ForwardWithName),
// minus TensorRT itself, which is not installed here.
//
// The extern "C" functions below are a test harness, not part of the product ABI.
#include <cuda_runtime_api.h>

#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "embedding_bag_plugin.h"
#include "trt_creator_manager.h"
#include "trt_shim/mini_trt.h"

#ifndef FWD_EB_TRT_SHIM
#error "host_driver.cpp belongs to the TensorRT stand-in build only"
#endif

using fwd::TrtEmbeddingBagDesc;
using fwd::trt_::EmbeddingBagPlugin;

struct fwd_eb_host {
  std::unique_ptr<mini_trt::Network> network;          // build side (owns the layer's plugin)
  nvinfer1::IPluginV2DynamicExt* engine_plugin{nullptr};  // run side: the engine's own instance
  std::vector<nvinfer1::PluginTensorDesc> in_desc;
  nvinfer1::PluginTensorDesc out_desc{};
  std::string layer_name;
  std::vector<char> blob;
  bool configured{false};
  // every way out of build / load / clone, the failing ones included, releases the engine's
  // plugin the way TensorRT does: terminate, then destroy
  ~fwd_eb_host() {
    if (engine_plugin) {
      engine_plugin->terminate();
      engine_plugin->destroy();
    }
  }
};

namespace {

nvinfer1::Dims MakeDims(int rank, const int* d) {
  nvinfer1::Dims out;
  out.nbDims = rank;
  for (int i = 0; i < rank && i < nvinfer1::Dims::MAX_DIMS; ++i) out.d[i] = d[i];
  return out;
}

// Format negotiation + configurePlugin, as the builder and the runtime both do.
bool Negotiate(fwd_eb_host* h) {
  const int nb_in = (int)h->in_desc.size();
  std::vector<nvinfer1::PluginTensorDesc> all = h->in_desc;
  all.push_back(h->out_desc);
  for (int pos = 0; pos <= nb_in; ++pos) {
    if (!h->engine_plugin->supportsFormatCombination(pos, all.data(), nb_in, 1)) return false;
  }
  std::vector<nvinfer1::DynamicPluginTensorDesc> din(nb_in);
  for (int i = 0; i < nb_in; ++i) din[i] = {h->in_desc[i], h->in_desc[i].dims, h->in_desc[i].dims};
  nvinfer1::DynamicPluginTensorDesc dout{h->out_desc, h->out_desc.dims, h->out_desc.dims};
  h->engine_plugin->configurePlugin(din.data(), nb_in, &dout, 1);
  h->configured = true;
  return true;
}

void FillDescs(fwd_eb_host* h, mini_trt::Layer* layer) {
  h->in_desc.clear();
  for (mini_trt::Tensor* t : layer->inputs) {
    h->in_desc.push_back({t->getDimensions(), t->getType(), nvinfer1::TensorFormat::kLINEAR, 1.0f});
  }
  h->out_desc = {layer->output->getDimensions(), layer->output->getType(),
                 nvinfer1::TensorFormat::kLINEAR, 1.0f};
}

}  // namespace

extern "C" {

void fwd_eb_host_free(fwd_eb_host* h) { delete h; }

fwd_eb_host* fwd_eb_host_build_desc(const void* embedding_bag_desc, int idx_rank, const int* idx_dims,
                                    int off_rank, const int* off_dims, int weights_rank,
                                    const int* weights_dims);

// Build: TrtEmbeddingBagDesc -> LayerCreatorManager -> CreateLayer -> network; then the engine's
// own clone is configured and serialised.  `weights_rank` 0 = no per-sample-weights input.
fwd_eb_host* fwd_eb_host_build(const void* table, int half_table, int count, int dim, int offset,
                               int op, long long padding_idx, int include_last_offset,
                               int half_output, int idx_rank, const int* idx_dims, int off_rank,
                               const int* off_dims, int weights_rank, const int* weights_dims) {
  auto desc = std::make_shared<TrtEmbeddingBagDesc>();
  desc->dim = dim;
  desc->count = count;
  desc->offset = offset;
  desc->op = op;
  desc->padding_idx = padding_idx;
  desc->include_last_offset = include_last_offset != 0;
  desc->has_per_sample_weights = weights_rank > 0;
  desc->half_output = half_output != 0;
  desc->data.SetType(half_table ? nvinfer1::DataType::kHALF : nvinfer1::DataType::kFLOAT);
  desc->data.SetCount((int64_t)dim * count);
  desc->data.SetData(static_cast<const char*>(table), (int64_t)dim * count * (half_table ? 2 : 4));
  return fwd_eb_host_build_desc(desc.get(), idx_rank, idx_dims, off_rank, off_dims, weights_rank,
                                weights_dims);
}

// Build around a table that stays outside the plugin: `key` names a device table registered with
// fwd_eb_plugin_register_weights.
fwd_eb_host* fwd_eb_host_build_external(const char* key, int half_table, int count, int dim, int offset,
                                        int op, long long padding_idx, int include_last_offset,
                                        int half_output, int idx_rank, const int* idx_dims, int off_rank,
                                        const int* off_dims, int weights_rank, const int* weights_dims) {
  if (!key) return nullptr;
  auto desc = std::make_shared<TrtEmbeddingBagDesc>();
  desc->dim = dim;
  desc->count = count;
  desc->offset = offset;
  desc->op = op;
  desc->padding_idx = padding_idx;
  desc->include_last_offset = include_last_offset != 0;
  desc->has_per_sample_weights = weights_rank > 0;
  desc->half_output = half_output != 0;
  desc->data.SetType(half_table ? nvinfer1::DataType::kHALF : nvinfer1::DataType::kFLOAT);
  desc->external_weights = key;
  return fwd_eb_host_build_desc(desc.get(), idx_rank, idx_dims, off_rank, off_dims, weights_rank,
                                weights_dims);
}

// The same from a description some parser produced (`embedding_bag_desc` is a
// fwd::TrtEmbeddingBagDesc*; the torch parser slice enters here).
fwd_eb_host* fwd_eb_host_build_desc(const void* embedding_bag_desc, int idx_rank, const int* idx_dims,
                                    int off_rank, const int* off_dims, int weights_rank,
                                    const int* weights_dims) {
  const auto* desc = static_cast<const TrtEmbeddingBagDesc*>(embedding_bag_desc);
  if (!desc) return nullptr;
  std::unique_ptr<fwd_eb_host> h(new fwd_eb_host());
  h->network.reset(new mini_trt::Network());
  fwd::trt_::ITensorVector inputs;
  inputs.push_back(h->network->addInput("input", nvinfer1::DataType::kINT32, MakeDims(idx_rank, idx_dims)));
  if (off_rank > 0)
    inputs.push_back(h->network->addInput("offsets", nvinfer1::DataType::kINT32, MakeDims(off_rank, off_dims)));
  if (weights_rank > 0)
    inputs.push_back(h->network->addInput("per_sample_weights", nvinfer1::DataType::kFLOAT,
                                          MakeDims(weights_rank, weights_dims)));

  static fwd::trt_::LayerCreatorManager manager;
  fwd::trt_::ILayerCreator* creator = manager.FindCreator(desc->Name());  // "EmbeddingBag"
  if (!creator) return nullptr;
  fwd::trt_::ITensorVector outputs = creator->CreateLayer(h->network.get(), desc, inputs);
  if (outputs.empty()) return nullptr;
  mini_trt::Layer* layer = h->network->LayerAt(h->network->getNbLayers() - 1);
  h->layer_name = layer->getName();
  FillDescs(h.get(), layer);

  // the builder works on its own clone of the network's plugin
  h->engine_plugin = static_cast<nvinfer1::IPluginV2DynamicExt*>(layer->getPlugin().getNbOutputs() == 1
                                                                    ? layer->plugin->clone()
                                                                    : nullptr);
  if (!h->engine_plugin || h->engine_plugin->initialize() != 0) return nullptr;
  if (!Negotiate(h.get())) return nullptr;
  h->blob.resize(h->engine_plugin->getSerializationSize());
  h->engine_plugin->serialize(h->blob.data());
  return h.release();
}

size_t fwd_eb_host_blob(fwd_eb_host* h, void* dst, size_t cap) {
  if (!h) return 0;
  if (dst && cap >= h->blob.size()) std::memcpy(dst, h->blob.data(), h->blob.size());
  return h->blob.size();
}

// Load: registry lookup by name/version -> deserializePlugin -> initialize -> configure, with
// the tensor shapes of `like` (the meta data an engine file carries).
fwd_eb_host* fwd_eb_host_load(const void* blob, size_t len, const fwd_eb_host* like) {
  if (!like) return nullptr;
  nvinfer1::IPluginCreator* creator = getPluginRegistry()->getPluginCreator("EmbeddingBag_TRT", "001");
  if (!creator) return nullptr;
  nvinfer1::IPluginV2* p = creator->deserializePlugin("embedding_bag", blob, len);
  if (!p) return nullptr;
  std::unique_ptr<fwd_eb_host> h(new fwd_eb_host());
  h->engine_plugin = static_cast<nvinfer1::IPluginV2DynamicExt*>(p);
  h->in_desc = like->in_desc;
  h->out_desc = like->out_desc;
  h->layer_name = like->layer_name;
  h->blob.assign(static_cast<const char*>(blob), static_cast<const char*>(blob) + len);
  if (h->engine_plugin->initialize() != 0) return nullptr;
  if (!Negotiate(h.get())) return nullptr;
  return h.release();
}

// A second execution context: TensorRT clones the plugin per context.
fwd_eb_host* fwd_eb_host_clone_context(const fwd_eb_host* src) {
  if (!src || !src->engine_plugin) return nullptr;
  std::unique_ptr<fwd_eb_host> h(new fwd_eb_host());
  h->engine_plugin = src->engine_plugin->clone();
  if (!h->engine_plugin) return nullptr;
  h->in_desc = src->in_desc;
  h->out_desc = src->out_desc;
  h->layer_name = src->layer_name;
  h->blob = src->blob;
  if (!Negotiate(h.get())) return nullptr;
  return h.release();
}

int fwd_eb_host_output_dims(const fwd_eb_host* h, int* dims8, int* dtype) {
  if (!h) return -1;
  for (int i = 0; i < h->out_desc.dims.nbDims; ++i) dims8[i] = h->out_desc.dims.d[i];
  if (dtype) *dtype = (int)h->out_desc.type;
  return h->out_desc.dims.nbDims;
}

const char* fwd_eb_host_layer_name(const fwd_eb_host* h) { return h ? h->layer_name.c_str() : ""; }

int fwd_eb_host_table_uploads(const fwd_eb_host* h) {
  auto* p = h ? dynamic_cast<EmbeddingBagPlugin*>(h->engine_plugin) : nullptr;
  return p && p->Table() ? p->Table()->Uploads() : -1;
}

// 1 when both handles' plugins share one table object (clones do, separate loads do not).
int fwd_eb_host_shares_table(const fwd_eb_host* a, const fwd_eb_host* b) {
  auto* pa = a ? dynamic_cast<EmbeddingBagPlugin*>(a->engine_plugin) : nullptr;
  auto* pb = b ? dynamic_cast<EmbeddingBagPlugin*>(b->engine_plugin) : nullptr;
  return pa && pb && pa->Table() == pb->Table();
}

// supportsFormatCombination with one tensor's type/format overridden.
int fwd_eb_host_format_ok(fwd_eb_host* h, int pos, int type, int format) {
  if (!h) return -1;
  std::vector<nvinfer1::PluginTensorDesc> all = h->in_desc;
  all.push_back(h->out_desc);
  if (pos < 0 || pos >= (int)all.size()) return -1;
  all[pos].type = static_cast<nvinfer1::DataType>(type);
  all[pos].format = static_cast<nvinfer1::TensorFormat>(format);
  return h->engine_plugin->supportsFormatCombination(pos, all.data(), (int)h->in_desc.size(), 1) ? 1 : 0;
}

size_t fwd_eb_host_workspace(fwd_eb_host* h) {
  return h ? h->engine_plugin->getWorkspaceSize(h->in_desc.data(), (int)h->in_desc.size(), &h->out_desc, 1) : 0;
}

// enqueue with device pointers in input order (indices, [offsets], [weights]).
int fwd_eb_host_run(fwd_eb_host* h, const void* d0, const void* d1, const void* d2, void* d_out,
                    void* stream) {
  if (!h || !h->configured) return -100;
  const void* inputs[3] = {d0, d1, d2};
  void* outputs[1] = {d_out};
  return h->engine_plugin->enqueue(h->in_desc.data(), &h->out_desc, inputs, outputs, nullptr,
                                   static_cast<cudaStream_t>(stream));
}

const char* fwd_eb_host_last_log() {
  static thread_local std::string keep;
  keep = mini_trt::LastLoggedError();
  return keep.c_str();
}

int fwd_eb_host_logged_errors() { return mini_trt::LoggedErrors(); }

// Creator-level checks without a network: returns 1 when createPlugin accepted the fields.
int fwd_eb_host_creator_accepts(int n_fields, const char* const* names, const int* types,
                                const void* const* data, const int* lengths) {
  nvinfer1::IPluginCreator* creator = getPluginRegistry()->getPluginCreator("EmbeddingBag_TRT", "001");
  if (!creator) return -1;
  std::vector<nvinfer1::PluginField> f;
  for (int i = 0; i < n_fields; ++i)
    f.emplace_back(names[i], data[i], static_cast<nvinfer1::PluginFieldType>(types[i]), lengths[i]);
  nvinfer1::PluginFieldCollection fc{n_fields, f.data()};
  nvinfer1::IPluginV2* p = creator->createPlugin("probe", &fc);
  if (!p) return 0;
  p->destroy();
  return 1;
}

int fwd_eb_host_creator_field_names(char* dst, size_t cap) {
  nvinfer1::IPluginCreator* creator = getPluginRegistry()->getPluginCreator("EmbeddingBag_TRT", "001");
  if (!creator) return -1;
  const nvinfer1::PluginFieldCollection* fc = creator->getFieldNames();
  std::string s;
  for (int i = 0; i < fc->nbFields; ++i) s += std::string(i ? "," : "") + fc->fields[i].name;
  std::snprintf(dst, cap, "%s", s.c_str());
  return fc->nbFields;
}

}  // extern "C"
