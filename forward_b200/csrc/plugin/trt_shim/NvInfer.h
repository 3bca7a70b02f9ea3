// Stand-in for the TensorRT headers, used ONLY when real TensorRT is not installed.
//
// It declares, in our own words, the part of the nvinfer1 interface that Forward's
// EmbeddingBag plugin, its creator and its layer creator use (method names and argument
// lists as they appear at the call sites in Forward:
//   source/trt_engine/trt_network_crt/plugins/embedding_bag_plugin/embedding_bag_plugin.h:51-161
//   source/trt_engine/trt_network_crt/plugins/common/plugin.h:34-46
//   source/trt_engine/trt_network_crt/layer_creators/trt_embedding_bag_creator.h:54-75).
// It is self-consistent with the small host in mini_trt.cpp, which plays TensorRT's role in
// the tests, and is NOT binary compatible with libnvinfer: a build against real TensorRT
// must put the real headers first on the include path, and then this directory is unused.
#pragma once

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>

#define FWD_EB_TRT_SHIM 1

namespace nvinfer1 {

enum class DataType : int32_t { kFLOAT = 0, kHALF = 1, kINT8 = 2, kINT32 = 3, kBOOL = 4 };
enum class TensorFormat : int32_t { kLINEAR = 0, kCHW2 = 1, kHWC8 = 2, kCHW4 = 3 };

class Dims {
 public:
  static constexpr int32_t MAX_DIMS = 8;
  int32_t nbDims{0};
  int32_t d[MAX_DIMS]{};
};

struct Weights {
  DataType type;
  const void* values;
  int64_t count;
};

class ILogger {
 public:
  enum class Severity : int32_t { kINTERNAL_ERROR = 0, kERROR = 1, kWARNING = 2, kINFO = 3, kVERBOSE = 4 };
  virtual void log(Severity severity, const char* msg) noexcept = 0;
  virtual ~ILogger() = default;
};

// ---- symbolic dimensions (dynamic shapes) -----------------------------------------------

class IDimensionExpr {
 public:
  virtual bool isConstant() const noexcept = 0;
  virtual int32_t getConstantValue() const noexcept = 0;

 protected:
  virtual ~IDimensionExpr() = default;
};

class DimsExprs {
 public:
  int32_t nbDims{0};
  const IDimensionExpr* d[Dims::MAX_DIMS]{};
};

enum class DimensionOperation : int32_t { kSUM = 0, kPROD = 1, kMAX = 2, kMIN = 3, kSUB = 4 };

class IExprBuilder {
 public:
  virtual const IDimensionExpr* constant(int32_t value) noexcept = 0;
  virtual const IDimensionExpr* operation(DimensionOperation op, const IDimensionExpr& first,
                                          const IDimensionExpr& second) noexcept = 0;

 protected:
  virtual ~IExprBuilder() = default;
};

// ---- plugin interfaces ------------------------------------------------------------------

struct PluginTensorDesc {
  Dims dims;
  DataType type;
  TensorFormat format;
  float scale;
};

struct DynamicPluginTensorDesc {
  PluginTensorDesc desc;
  Dims min;
  Dims max;
};

enum class PluginFieldType : int32_t {
  kFLOAT16 = 0, kFLOAT32 = 1, kFLOAT64 = 2, kINT8 = 3, kINT16 = 4, kINT32 = 5, kCHAR = 6, kDIMS = 7,
  kUNKNOWN = 8
};

class PluginField {
 public:
  const char* name;
  const void* data;
  PluginFieldType type;
  int32_t length;
  PluginField(const char* name_ = nullptr, const void* data_ = nullptr,
              PluginFieldType type_ = PluginFieldType::kUNKNOWN, int32_t length_ = 0)
      : name(name_), data(data_), type(type_), length(length_) {}
};

struct PluginFieldCollection {
  int32_t nbFields;
  const PluginField* fields;
};

class IPluginV2 {
 public:
  virtual int32_t getNbOutputs() const noexcept = 0;
  virtual int32_t initialize() noexcept = 0;
  virtual void terminate() noexcept = 0;
  virtual size_t getSerializationSize() const noexcept = 0;
  virtual void serialize(void* buffer) const noexcept = 0;
  virtual const char* getPluginType() const noexcept = 0;
  virtual const char* getPluginVersion() const noexcept = 0;
  virtual void destroy() noexcept = 0;
  virtual void setPluginNamespace(const char* pluginNamespace) noexcept = 0;
  virtual const char* getPluginNamespace() const noexcept = 0;

 protected:
  virtual ~IPluginV2() noexcept = default;
};

class IPluginV2Ext : public IPluginV2 {
 public:
  virtual DataType getOutputDataType(int32_t index, const DataType* inputTypes,
                                     int32_t nbInputs) const noexcept = 0;
};

class IPluginV2DynamicExt : public IPluginV2Ext {
 public:
  virtual IPluginV2DynamicExt* clone() const noexcept = 0;
  virtual DimsExprs getOutputDimensions(int32_t outputIndex, const DimsExprs* inputs,
                                        int32_t nbInputs, IExprBuilder& exprBuilder) noexcept = 0;
  virtual bool supportsFormatCombination(int32_t pos, const PluginTensorDesc* inOut,
                                         int32_t nbInputs, int32_t nbOutputs) noexcept = 0;
  virtual void configurePlugin(const DynamicPluginTensorDesc* in, int32_t nbInputs,
                               const DynamicPluginTensorDesc* out, int32_t nbOutputs) noexcept = 0;
  virtual size_t getWorkspaceSize(const PluginTensorDesc* inputs, int32_t nbInputs,
                                  const PluginTensorDesc* outputs,
                                  int32_t nbOutputs) const noexcept = 0;
  virtual int32_t enqueue(const PluginTensorDesc* inputDesc, const PluginTensorDesc* outputDesc,
                          const void* const* inputs, void* const* outputs, void* workspace,
                          cudaStream_t stream) noexcept = 0;
};

class IPluginCreator {
 public:
  virtual const char* getPluginName() const noexcept = 0;
  virtual const char* getPluginVersion() const noexcept = 0;
  virtual const PluginFieldCollection* getFieldNames() noexcept = 0;
  virtual IPluginV2* createPlugin(const char* name, const PluginFieldCollection* fc) noexcept = 0;
  virtual IPluginV2* deserializePlugin(const char* name, const void* serialData,
                                       size_t serialLength) noexcept = 0;
  virtual void setPluginNamespace(const char* pluginNamespace) noexcept = 0;
  virtual const char* getPluginNamespace() const noexcept = 0;
  virtual ~IPluginCreator() = default;
};

class IPluginRegistry {
 public:
  virtual bool registerCreator(IPluginCreator& creator, const char* pluginNamespace) noexcept = 0;
  virtual IPluginCreator* getPluginCreator(const char* pluginName, const char* pluginVersion,
                                           const char* pluginNamespace = "") noexcept = 0;

 protected:
  virtual ~IPluginRegistry() = default;
};

// ---- the slice of the network-definition API the layer creator touches --------------------

class ITensor {
 public:
  virtual Dims getDimensions() const noexcept = 0;
  virtual DataType getType() const noexcept = 0;
  virtual const char* getName() const noexcept = 0;

 protected:
  virtual ~ITensor() = default;
};

class ILayer {
 public:
  virtual void setName(const char* name) noexcept = 0;
  virtual const char* getName() const noexcept = 0;
  virtual ITensor* getOutput(int32_t index) const noexcept = 0;
  virtual int32_t getNbOutputs() const noexcept = 0;

 protected:
  virtual ~ILayer() = default;
};

class IPluginV2Layer : public ILayer {
 public:
  virtual IPluginV2& getPlugin() noexcept = 0;
};

class INetworkDefinition {
 public:
  virtual ITensor* addInput(const char* name, DataType type, Dims dimensions) noexcept = 0;
  virtual IPluginV2Layer* addPluginV2(ITensor* const* inputs, int32_t nbInputs,
                                      IPluginV2& plugin) noexcept = 0;
  virtual int32_t getNbLayers() const noexcept = 0;
  virtual void markOutput(ITensor& tensor) noexcept = 0;
  virtual ~INetworkDefinition() = default;
};

template <typename T>
class PluginRegistrar {
 public:
  PluginRegistrar();

 private:
  T instance{};
};

}  // namespace nvinfer1

// Provided by mini_trt.cpp (libnvinfer exports the same two names).
extern "C" nvinfer1::IPluginRegistry* getPluginRegistry() noexcept;
extern "C" nvinfer1::ILogger* getLogger() noexcept;

namespace nvinfer1 {
template <typename T>
PluginRegistrar<T>::PluginRegistrar() {
  getPluginRegistry()->registerCreator(instance, "");
}
}  // namespace nvinfer1

#define REGISTER_TENSORRT_PLUGIN(name) \
  static nvinfer1::PluginRegistrar<name> pluginRegistrar##name {}
