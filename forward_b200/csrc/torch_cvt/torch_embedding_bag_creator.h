// aten::embedding_bag -> TrtEmbeddingBagDesc.
//
// Same role as Forward's source/fwd_torch/torch_cvt/torch_desc_creators/
// torch_embedding_bag_creator.h:40-73, which reads inputs 0 (weight), 1 (indices), 2 (offsets)
// and 4 (mode) and silently drops the rest (:54-61).  The schema is
//   aten::embedding_bag(weight, indices, offsets, scale_grad_by_freq, mode, sparse,
//                       per_sample_weights, include_last_offset[, padding_idx])
// and the dropped ones change the result, so they are read here: a per_sample_weights tensor
// becomes a third layer input, include_last_offset and padding_idx go into the description,
// fp16 weights stay fp16.  Anything that cannot be honoured fails the conversion instead of
// producing a wrong engine.
#pragma once

#include <memory>
#include <vector>

#include "fwd_log.h"
#include "i_torch_layer_creator.h"

FWD_TORCH_NAMESPACE_BEGIN

template <>
class TLayerDescCreator<TrtEmbeddingBagDesc> : public ILayerDescCreator {
 public:
  bool Check(const JitNode* node, const TorchModule& module) override {
    (void)module;
    return node->kind() == c10::aten::embedding_bag;
  }

  std::shared_ptr<TrtLayerDesc> Create(const JitNode* node, const TorchModule& module,
                                       std::vector<const JitValue*>& input_values) override {
    LOG(INFO) << "TrtEmbeddingBagDescCreator::Create";
    const auto inputs = node->inputs();
    if (inputs.size() < 5) return nullptr;
    auto layer_desc = std::make_shared<TrtEmbeddingBagDesc>();
    try {
      const at::Tensor weight = module.Get(inputs[0]).toTensor().contiguous().cpu();
      if (weight.dim() != 2) {
        LOG(ERROR) << "embedding_bag: weight must be 2-D";
        return nullptr;
      }
      layer_desc->op = static_cast<int>(module.Get(inputs[4]).toInt());  // 0 sum, 1 mean, 2 max
      layer_desc->count = static_cast<int>(weight.size(0));
      layer_desc->dim = static_cast<int>(weight.size(1));
      layer_desc->offset = 0;
      if (weight.scalar_type() == c10::kHalf) {
        layer_desc->data.SetType(nvinfer1::DataType::kHALF);
        layer_desc->data.SetData(static_cast<const char*>(weight.data_ptr()), weight.numel() * 2);
        layer_desc->half_output = true;  // torch returns fp16 for fp16 weights
      } else {
        const at::Tensor w32 = weight.to(c10::kFloat);
        layer_desc->data.SetType(nvinfer1::DataType::kFLOAT);
        layer_desc->data.SetData(static_cast<const char*>(w32.data_ptr()), w32.numel() * 4);
      }
      layer_desc->data.SetCount(weight.numel());

      input_values.push_back(inputs[1]);  // indices
      input_values.push_back(inputs[2]);  // offsets

      if (inputs.size() > 6) {  // per_sample_weights: None, or a run-time tensor
        const bool none = module.IsConstant(inputs[6]) && module.Get(inputs[6]).isNone();
        if (!none) {
          if (layer_desc->op != 0) {
            LOG(ERROR) << "embedding_bag: per_sample_weights need mode 'sum'";
            return nullptr;
          }
          layer_desc->has_per_sample_weights = true;
          input_values.push_back(inputs[6]);
        }
      }
      if (inputs.size() > 7) layer_desc->include_last_offset = module.Get(inputs[7]).toBool();
      if (inputs.size() > 8) {
        const c10::IValue pad = module.Get(inputs[8]);
        if (!pad.isNone()) {
          int64_t p = pad.toInt();
          if (p < 0) p += layer_desc->count;  // torch counts negative padding_idx from the end
          layer_desc->padding_idx = p;
        }
      }
    } catch (const std::exception& e) {
      LOG(ERROR) << "embedding_bag: " << e.what();
      return nullptr;
    }
    return layer_desc;
  }
};

FWD_TORCH_NAMESPACE_END
