// The slice of Forward's neutral IR that the EmbeddingBag path uses.
//
// Mirrors, with the same names and members:
//   FwdWeights            source/common/fwd_weights.h:133-196   (byte-blob weights holder)
//   TrtLayerDesc/Output   source/common/trt_layer_desc.h:60-80
//   TrtEmbeddingBagDesc   source/common/trt_layer_desc.h:234-241
// and widens them where the reference is lossy for this path: 64-bit byte counts
// (fwd_weights.h:172 takes an int), and the extra EmbeddingBag attributes the torch creator
// used to drop (padding_idx, include_last_offset, per_sample_weights, fp16 tables).
#pragma once

#include <NvInfer.h>

#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "fwd_macros.h"

FWD_NAMESPACE_BEGIN

class FwdWeights {
 public:
  FwdWeights() = default;
  explicit FwdWeights(const std::vector<float>& data) : type_(nvinfer1::DataType::kFLOAT), count_((int64_t)data.size()) {
    const char* p = reinterpret_cast<const char*>(data.data());
    data_.assign(p, p + data.size() * sizeof(float));
  }
  operator nvinfer1::Weights() const { return {type_, data_.data(), count_}; }
  bool Empty() const { return count_ == 0; }
  const void* Data() const { return data_.data(); }
  int64_t Bytes() const { return (int64_t)data_.size(); }
  void SetData(const char* data, int64_t num_bytes) { data_.assign(data, data + num_bytes); }
  nvinfer1::DataType Type() const { return type_; }
  void SetType(const nvinfer1::DataType& type) { type_ = type; }
  int64_t Count() const { return count_; }
  void SetCount(int64_t count) { count_ = count; }

 private:
  nvinfer1::DataType type_{nvinfer1::DataType::kFLOAT};
  int64_t count_{0};
  std::vector<char> data_;
};

struct TrtLayerDesc;

struct TrtLayerOutput {
  std::shared_ptr<TrtLayerDesc> layer_desc;
  int index{0};
};

struct TrtLayerDesc {
  virtual ~TrtLayerDesc() = default;
  virtual const std::string Name() const = 0;
  std::vector<TrtLayerOutput> inputs;
};

#define TRT_LAYER_DESC(LayerDesc)                  \
  static const char* NAME() { return #LayerDesc; } \
  const std::string Name() const override { return NAME(); }

struct TrtEmbeddingBagDesc : TrtLayerDesc {
  TRT_LAYER_DESC(EmbeddingBag);
  FwdWeights data;  // the table; Type() says fp32 or fp16
  int dim{0};
  int count{0};
  int offset{0};    // logical id of row 0 ("data_offset": the row-shard origin)
  int op{0};        // ReduceOperation value == torch mode integer
  // attributes the reference parser ignored (torch_embedding_bag_creator.h:54-61)
  int64_t padding_idx{-1};
  bool include_last_offset{false};
  bool has_per_sample_weights{false};
  bool half_output{false};  // emit kHALF like torch does for fp16 tables (default kFLOAT as the reference)
  // Non-empty: the table stays outside the plan.  It is the name a device table was registered
  // under (fwd_eb_plugin_register_weights); `data` then carries no bytes, only its Type().
  std::string external_weights;
};

FWD_NAMESPACE_END
