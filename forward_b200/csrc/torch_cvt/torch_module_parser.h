// Walks a TorchScript graph from its outputs back to its inputs and turns every
// aten::embedding_bag node it meets into a layer description: the part of Forward's Parser
// (source/fwd_torch/torch_cvt/torch_module_parser.cpp:40-163: Parse, ParseValue, the map of
// already created descriptions) that this path needs.
//
// What it accepts around the bags is what recommender front ends put there:
//   graph output      one tensor, or a tuple / list of tensors;
//   each of them      the pooled output of an embedding_bag node, or aten::cat of several along
//                     dim 1 (DLRM's "concatenate the sparse features");
//   a bag's inputs    a graph input, aten::select(graph input, 0, k) with constant k (one row of
//                     a stacked offsets tensor, as Forward's DLRM test feeds them,
//                     test_torch_dlrm.h:37-56), or element k of a graph input that is a list.
// Anything else is refused with the node's kind in the message; nothing is converted
// approximately.  Unlike the reference there is no dummy run of the module and therefore no
// rule that all inputs share their first dimension (torch_module_parser.cpp:165-184): indices
// and offsets of an EmbeddingBag never do.
#pragma once

#include <map>
#include <memory>
#include <string>
#include <vector>

#include "torch_desc_manager.h"

FWD_TORCH_NAMESPACE_BEGIN

// Where a layer input comes from: graph input `graph_input` (position among the non-self
// inputs), whole (`element` < 0) or its element / row `element`.
struct InputRef {
  int graph_input{-1};
  int element{-1};
  bool from_list{false};  // element of a list input (else: row `element` along dim 0)
};

struct ParsedLayer {
  std::shared_ptr<TrtEmbeddingBagDesc> desc;
  std::vector<InputRef> inputs;  // indices, offsets[, per_sample_weights]
};

struct ParsedNetwork {
  std::vector<ParsedLayer> layers;
  // one entry per graph output: the layers whose pooled outputs are concatenated along dim 1
  std::vector<std::vector<int>> outputs;
};

class Parser {
 public:
  // false, with the reason in Error(), when the file does not load or the graph holds
  // something this parser does not convert
  bool Parse(const std::string& module_path);
  const ParsedNetwork& GetNetwork() const { return network_; }
  const TorchModule& Module() const { return module_; }
  const std::string& Error() const { return error_; }

 private:
  bool ParseOutput(const JitValue* value, std::vector<int>* layers);
  bool ParseValue(const JitValue* value, int* layer);
  bool ParseInput(const JitValue* value, InputRef* ref);
  bool Fail(const std::string& why) {
    if (error_.empty()) error_ = why;
    return false;
  }

  TorchModule module_;
  TorchDescManager desc_manager_;
  ParsedNetwork network_;
  std::map<const JitNode*, int> created_;  // node -> layer already created for it
  std::string error_;
};

FWD_TORCH_NAMESPACE_END
