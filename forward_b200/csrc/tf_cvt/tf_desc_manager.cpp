#include "tf_desc_manager.h"

#include "tf_embedding_bag_creator.h"

FWD_TF_NAMESPACE_BEGIN

template <typename DescT>
void TfDescManager::RegisterCreator() {
  layer_desc_creators_.push_back(std::make_shared<TLayerDescCreator<DescT>>());
}

TfDescManager::TfDescManager() { RegisterCreator<TrtEmbeddingBagDesc>(); }

ILayerDescCreator* TfDescManager::FindDescCreator(const Operation& op) {
  for (auto& creator : layer_desc_creators_) {
    if (creator->Check(op)) return creator.get();
  }
  return nullptr;
}

FWD_TF_NAMESPACE_END
