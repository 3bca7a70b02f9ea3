// Layer-creator interface of Forward's TensorRT back-end
// (source/trt_engine/trt_network_crt/layer_creators/i_trt_layer_creator.h:35-60), same names.
#pragma once

#include <NvInfer.h>

#include <vector>

#include "fwd_log.h"
#include "trt_layer_desc.h"

FWD_TRT_NAMESPACE_BEGIN

using ITensorVector = std::vector<nvinfer1::ITensor*>;

class ILayerCreator {
 public:
  virtual ~ILayerCreator() = default;
  // Returns the layer's output tensors; empty on failure.
  virtual ITensorVector CreateLayer(nvinfer1::INetworkDefinition* network,
                                    const TrtLayerDesc* layer_desc,
                                    const ITensorVector& input_tensors) = 0;
};

template <typename T>
class TLayerCreator;

FWD_TRT_NAMESPACE_END
