// Concrete classes of the small TensorRT stand-in host (see mini_trt.cpp).
#pragma once

#include <memory>
#include <string>
#include <vector>

#include "NvInfer.h"

namespace mini_trt {

std::string LastLoggedError();
int LoggedErrors();

class Expr : public nvinfer1::IDimensionExpr {
 public:
  explicit Expr(int32_t v) : v_(v) {}
  bool isConstant() const noexcept override { return true; }
  int32_t getConstantValue() const noexcept override { return v_; }

 private:
  int32_t v_;
};

class ExprBuilder : public nvinfer1::IExprBuilder {
 public:
  const nvinfer1::IDimensionExpr* constant(int32_t value) noexcept override;
  const nvinfer1::IDimensionExpr* operation(nvinfer1::DimensionOperation op,
                                            const nvinfer1::IDimensionExpr& a,
                                            const nvinfer1::IDimensionExpr& b) noexcept override;

 private:
  std::vector<std::unique_ptr<Expr>> nodes_;
};

class Tensor : public nvinfer1::ITensor {
 public:
  Tensor(std::string name, nvinfer1::DataType type, nvinfer1::Dims dims)
      : name_(std::move(name)), type_(type), dims_(dims) {}
  nvinfer1::Dims getDimensions() const noexcept override { return dims_; }
  nvinfer1::DataType getType() const noexcept override { return type_; }
  const char* getName() const noexcept override { return name_.c_str(); }

 private:
  std::string name_;
  nvinfer1::DataType type_;
  nvinfer1::Dims dims_;
};

class Layer : public nvinfer1::IPluginV2Layer {
 public:
  ~Layer();
  void setName(const char* name) noexcept override { name_ = name ? name : ""; }
  const char* getName() const noexcept override { return name_.c_str(); }
  nvinfer1::ITensor* getOutput(int32_t index) const noexcept override { return index == 0 ? output : nullptr; }
  int32_t getNbOutputs() const noexcept override { return 1; }
  nvinfer1::IPluginV2& getPlugin() noexcept override { return *plugin; }

  nvinfer1::IPluginV2DynamicExt* plugin{nullptr};
  std::vector<Tensor*> inputs;
  Tensor* output{nullptr};

 private:
  std::string name_;
};

class Network : public nvinfer1::INetworkDefinition {
 public:
  nvinfer1::ITensor* addInput(const char* name, nvinfer1::DataType type,
                              nvinfer1::Dims dims) noexcept override;
  nvinfer1::IPluginV2Layer* addPluginV2(nvinfer1::ITensor* const* inputs, int32_t nbInputs,
                                        nvinfer1::IPluginV2& plugin) noexcept override;
  int32_t getNbLayers() const noexcept override { return (int32_t)layers_.size(); }
  void markOutput(nvinfer1::ITensor&) noexcept override {}
  Layer* LayerAt(int i) { return layers_[i].get(); }

 private:
  std::vector<std::unique_ptr<Tensor>> tensors_;
  std::vector<Tensor*> inputs_;
  std::vector<std::unique_ptr<Layer>> layers_;
};

}  // namespace mini_trt
