// The slice of Forward's TorchModule that layer-description creators rely on: load a
// TorchScript file, inline its forward graph, and answer "what constant does this graph value
// hold?" (TorchModule::Get, source/fwd_torch/torch_cvt/torch_module.cpp:169-179 in Forward).
//
// Forward answers that by running the whole module once on dummy inputs and caching every
// intermediate (EvalAll, torch_module.cpp:88-123).  Creators for EmbeddingBag only ever ask for
// values that are constants of the graph or attributes of the module (weight, mode,
// include_last_offset, padding_idx), so here those are resolved directly from the graph — no
// dummy run, and no need for dummy inputs whose first dimensions agree.
#pragma once

#include <torch/script.h>

#include <memory>
#include <string>
#include <vector>

#include "fwd_macros.h"

FWD_TORCH_NAMESPACE_BEGIN

using JitNode = ::torch::jit::Node;
using JitValue = ::torch::jit::Value;

class TorchModule {
 public:
  // false (with the reason in Error()) when the file cannot be loaded
  bool Load(const std::string& module_path);
  const std::shared_ptr<torch::jit::Graph>& Graph() const { return graph_; }
  // graph inputs other than `self`, in order
  const std::vector<const JitValue*>& Inputs() const { return inputs_; }
  // Constant held by `value`: a prim::Constant, or an attribute reached from `self` through
  // prim::GetAttr.  Throws std::runtime_error for anything computed at run time.
  c10::IValue Get(const JitValue* value) const;
  bool IsConstant(const JitValue* value) const;
  const std::string& Error() const { return error_; }

 private:
  torch::jit::Module module_;
  std::shared_ptr<torch::jit::Graph> graph_;
  std::vector<const JitValue*> inputs_;
  std::string error_;
};

FWD_TORCH_NAMESPACE_END
