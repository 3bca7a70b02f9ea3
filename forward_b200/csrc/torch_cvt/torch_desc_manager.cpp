#include "torch_desc_manager.h"

#include "torch_embedding_bag_creator.h"

FWD_TORCH_NAMESPACE_BEGIN

template <typename DescT>
void TorchDescManager::RegisterCreator() {
  layer_desc_creators_.push_back(std::make_shared<TLayerDescCreator<DescT>>());
}

TorchDescManager::TorchDescManager() { RegisterCreator<TrtEmbeddingBagDesc>(); }

ILayerDescCreator* TorchDescManager::FindDescCreator(const JitNode* node, const TorchModule& module) {
  for (auto& creator : layer_desc_creators_) {
    if (creator->Check(node, module)) return creator.get();
  }
  return nullptr;
}

FWD_TORCH_NAMESPACE_END
