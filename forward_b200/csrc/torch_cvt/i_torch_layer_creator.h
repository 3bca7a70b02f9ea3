// Description-creator interface of Forward's torch parser
// (source/fwd_torch/torch_cvt/torch_desc_creators/i_torch_layer_creator.h:40-70), same names.
#pragma once

#include <memory>
#include <vector>

#include "torch_module.h"
#include "trt_layer_desc.h"

FWD_TORCH_NAMESPACE_BEGIN

class ILayerDescCreator {
 public:
  virtual ~ILayerDescCreator() = default;
  // Does this creator handle `node`?
  virtual bool Check(const JitNode* node, const TorchModule& module) = 0;
  // The node's layer description (nullptr on failure); `node_inputs` receives the graph values
  // that become the layer's tensor inputs, in order.
  virtual std::shared_ptr<TrtLayerDesc> Create(const JitNode* node, const TorchModule& module,
                                               std::vector<const JitValue*>& node_inputs) = 0;
};

template <typename T>
class TLayerDescCreator;

FWD_TORCH_NAMESPACE_END
