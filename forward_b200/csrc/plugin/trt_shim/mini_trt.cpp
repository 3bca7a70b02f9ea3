// A very small host that plays TensorRT's part for the plugin tests: plugin registry, logger,
// symbolic-dimension builder and a network definition that accepts plugin layers.  Only
// compiled together with the interface stand-in in this directory (never with real TensorRT).
#include "mini_trt.h"

#include <cstdio>
#include <cstring>
#include <mutex>

namespace mini_trt {

// ---- logger --------------------------------------------------------------------------------

class Logger : public nvinfer1::ILogger {
 public:
  void log(Severity severity, const char* msg) noexcept override {
    std::lock_guard<std::mutex> hold(lock_);
    if (severity <= Severity::kERROR) {
      last_error_ = msg ? msg : "";
      ++errors_;
    }
  }
  std::string LastError() {
    std::lock_guard<std::mutex> hold(lock_);
    return last_error_;
  }
  int Errors() {
    std::lock_guard<std::mutex> hold(lock_);
    return errors_;
  }

 private:
  std::mutex lock_;
  std::string last_error_;
  int errors_{0};
};

static Logger& TheLogger() {
  static Logger logger;
  return logger;
}

std::string LastLoggedError() { return TheLogger().LastError(); }
int LoggedErrors() { return TheLogger().Errors(); }

// ---- registry ------------------------------------------------------------------------------

class Registry : public nvinfer1::IPluginRegistry {
 public:
  bool registerCreator(nvinfer1::IPluginCreator& creator, const char* ns) noexcept override {
    std::lock_guard<std::mutex> hold(lock_);
    for (auto& e : entries_) {
      if (!std::strcmp(e.creator->getPluginName(), creator.getPluginName()) &&
          !std::strcmp(e.creator->getPluginVersion(), creator.getPluginVersion()) && e.ns == (ns ? ns : ""))
        return false;  // already there
    }
    creator.setPluginNamespace(ns ? ns : "");
    entries_.push_back({&creator, ns ? ns : ""});
    return true;
  }
  nvinfer1::IPluginCreator* getPluginCreator(const char* name, const char* version,
                                             const char* ns) noexcept override {
    std::lock_guard<std::mutex> hold(lock_);
    for (auto& e : entries_) {
      if (!std::strcmp(e.creator->getPluginName(), name) &&
          !std::strcmp(e.creator->getPluginVersion(), version) && e.ns == (ns ? ns : ""))
        return e.creator;
    }
    return nullptr;
  }

 private:
  struct Entry {
    nvinfer1::IPluginCreator* creator;
    std::string ns;
  };
  std::mutex lock_;
  std::vector<Entry> entries_;
};

static Registry& TheRegistry() {
  static Registry registry;
  return registry;
}

// ---- symbolic dimensions -------------------------------------------------------------------

const nvinfer1::IDimensionExpr* ExprBuilder::constant(int32_t value) noexcept {
  nodes_.emplace_back(new Expr(value));
  return nodes_.back().get();
}

const nvinfer1::IDimensionExpr* ExprBuilder::operation(nvinfer1::DimensionOperation op,
                                                       const nvinfer1::IDimensionExpr& a,
                                                       const nvinfer1::IDimensionExpr& b) noexcept {
  const int32_t x = a.getConstantValue(), y = b.getConstantValue();
  int32_t r = 0;
  switch (op) {
    case nvinfer1::DimensionOperation::kSUM: r = x + y; break;
    case nvinfer1::DimensionOperation::kPROD: r = x * y; break;
    case nvinfer1::DimensionOperation::kMAX: r = x > y ? x : y; break;
    case nvinfer1::DimensionOperation::kMIN: r = x < y ? x : y; break;
    case nvinfer1::DimensionOperation::kSUB: r = x - y; break;
  }
  return constant(r);
}

// ---- network -------------------------------------------------------------------------------

Layer::~Layer() {
  if (plugin) plugin->destroy();
}

nvinfer1::ITensor* Network::addInput(const char* name, nvinfer1::DataType type,
                                     nvinfer1::Dims dims) noexcept {
  tensors_.emplace_back(new Tensor(name ? name : "", type, dims));
  inputs_.push_back(tensors_.back().get());
  return tensors_.back().get();
}

nvinfer1::IPluginV2Layer* Network::addPluginV2(nvinfer1::ITensor* const* inputs, int32_t nbInputs,
                                               nvinfer1::IPluginV2& plugin) noexcept {
  auto* dyn = dynamic_cast<nvinfer1::IPluginV2DynamicExt*>(&plugin);
  if (!dyn || nbInputs < 1) return nullptr;
  std::unique_ptr<Layer> layer(new Layer());
  layer->plugin = dyn->clone();  // TensorRT keeps its own copy; the caller destroys theirs
  if (!layer->plugin) return nullptr;
  ExprBuilder exprs;
  std::vector<nvinfer1::DimsExprs> in(nbInputs);
  std::vector<nvinfer1::DataType> types(nbInputs);
  for (int i = 0; i < nbInputs; ++i) {
    const nvinfer1::Dims d = inputs[i]->getDimensions();
    in[i].nbDims = d.nbDims;
    for (int k = 0; k < d.nbDims; ++k) in[i].d[k] = exprs.constant(d.d[k]);
    types[i] = inputs[i]->getType();
    layer->inputs.push_back(static_cast<Tensor*>(inputs[i]));
  }
  nvinfer1::DimsExprs out = layer->plugin->getOutputDimensions(0, in.data(), nbInputs, exprs);
  if (out.nbDims < 0) return nullptr;
  nvinfer1::Dims od;
  od.nbDims = out.nbDims;
  for (int k = 0; k < out.nbDims; ++k) od.d[k] = out.d[k]->getConstantValue();
  const nvinfer1::DataType ot = layer->plugin->getOutputDataType(0, types.data(), nbInputs);
  tensors_.emplace_back(new Tensor("", ot, od));
  layer->output = tensors_.back().get();
  layers_.push_back(std::move(layer));
  return layers_.back().get();
}

}  // namespace mini_trt

extern "C" nvinfer1::IPluginRegistry* getPluginRegistry() noexcept { return &mini_trt::TheRegistry(); }
extern "C" nvinfer1::ILogger* getLogger() noexcept { return &mini_trt::TheLogger(); }
