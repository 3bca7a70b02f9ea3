// Name -> layer-creator map of the TensorRT back-end, as in Forward's
// source/trt_engine/trt_network_crt/trt_creator_manager.{h,cpp} (RegisterCreator<T>() at
// .cpp:119 keyed by T::NAME(), lookup at .cpp:158-166), reduced to the creators this
// repository provides.
#pragma once

#include <map>
#include <memory>
#include <string>

#include "layer_creator_iface.h"

FWD_TRT_NAMESPACE_BEGIN

class LayerCreatorManager {
 public:
  LayerCreatorManager();
  ILayerCreator* FindCreator(const std::string& layer_name) const;

 private:
  template <typename DescT>
  void RegisterCreator();
  std::map<std::string, std::shared_ptr<ILayerCreator>> layer_creator_map_;
};

FWD_TRT_NAMESPACE_END
