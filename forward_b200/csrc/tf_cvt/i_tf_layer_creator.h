// Description-creator interface of Forward's TensorFlow parser
// (source/fwd_tf/tf_cvt/tf_desc_creators/i_tf_layer_creator.h:40-69), same names.
#pragma once

#include <memory>
#include <vector>

#include "tf_graph.h"
#include "trt_layer_desc.h"

FWD_TF_NAMESPACE_BEGIN

class ILayerDescCreator {
 public:
  virtual ~ILayerDescCreator() = default;
  // Does this creator handle `op` (possibly together with the nodes feeding it)?
  virtual bool Check(const Operation& op) = 0;
  // The layer description for `op` (nullptr on failure); `op_inputs` receives the graph outputs
  // that become the layer's tensor inputs, in order.
  virtual std::shared_ptr<TrtLayerDesc> Create(const Operation& op, const Graph& graph,
                                               std::vector<Output>& op_inputs) = 0;
};

template <typename T>
class TLayerDescCreator;

FWD_TF_NAMESPACE_END
