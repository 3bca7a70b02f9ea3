// Ordered list of description creators; the first whose Check() accepts a node wins
// (Forward: source/fwd_torch/torch_cvt/torch_desc_manager.{h,cpp}, registration of the
// EmbeddingBag creator at torch_desc_manager.cpp:93, lookup at :129-142).
#pragma once

#include <memory>
#include <vector>

#include "i_torch_layer_creator.h"

FWD_TORCH_NAMESPACE_BEGIN

class TorchDescManager {
 public:
  TorchDescManager();
  ILayerDescCreator* FindDescCreator(const JitNode* node, const TorchModule& module);

 private:
  template <typename DescT>
  void RegisterCreator();
  std::vector<std::shared_ptr<ILayerDescCreator>> layer_desc_creators_;
};

FWD_TORCH_NAMESPACE_END
