// Ordered list of description creators; the first whose Check() accepts an operation wins
// (Forward: source/fwd_tf/tf_cvt/tf_desc_manager.{h,cpp}; the EmbeddingBag creator is registered
// at tf_desc_manager.cpp:66, ahead of the plain Gather and Reduce creators, so a Sum or GatherV2
// that fits the pattern never reaches those).
#pragma once

#include <memory>
#include <vector>

#include "i_tf_layer_creator.h"

FWD_TF_NAMESPACE_BEGIN

class TfDescManager {
 public:
  TfDescManager();
  ILayerDescCreator* FindDescCreator(const Operation& op);

 private:
  template <typename DescT>
  void RegisterCreator();
  std::vector<std::shared_ptr<ILayerDescCreator>> layer_desc_creators_;
};

FWD_TF_NAMESPACE_END
