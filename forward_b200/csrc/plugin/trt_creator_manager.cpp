#include "trt_creator_manager.h"

#include "embedding_bag_plugin.h"
#include "trt_embedding_bag_creator.h"

FWD_TRT_NAMESPACE_BEGIN

// Static registration with TensorRT's registry (trt_creator_manager.cpp:85 in Forward).
REGISTER_TENSORRT_PLUGIN(EmbeddingBagPluginCreator);

template <typename DescT>
void LayerCreatorManager::RegisterCreator() {
  layer_creator_map_[DescT::NAME()] = std::make_shared<TLayerCreator<DescT>>();
}

LayerCreatorManager::LayerCreatorManager() { RegisterCreator<TrtEmbeddingBagDesc>(); }

ILayerCreator* LayerCreatorManager::FindCreator(const std::string& layer_name) const {
  auto it = layer_creator_map_.find(layer_name);
  return it == layer_creator_map_.end() ? nullptr : it->second.get();
}

FWD_TRT_NAMESPACE_END
