#include "torch_module.h"

#include <torch/csrc/jit/ir/constants.h>
#include <torch/csrc/jit/passes/inliner.h>

#include <stdexcept>

FWD_TORCH_NAMESPACE_BEGIN

bool TorchModule::Load(const std::string& module_path) {
  try {
    module_ = torch::jit::load(module_path, c10::kCPU);
    module_.eval();
    graph_ = module_.get_method("forward").graph()->copy();
    torch::jit::Inline(*graph_);
  } catch (const c10::Error& e) {
    error_ = e.what_without_backtrace();
    return false;
  } catch (const std::exception& e) {
    error_ = e.what();
    return false;
  }
  inputs_.clear();
  for (const JitValue* in : graph_->inputs()) {
    if (in->debugNameBase() == "self") continue;
    inputs_.push_back(in);
  }
  return true;
}

bool TorchModule::IsConstant(const JitValue* value) const {
  const JitNode* node = value->node();
  if (node->kind() == c10::prim::Constant) return true;
  if (node->kind() == c10::prim::GetAttr) {
    const JitValue* owner = node->input(0);
    return owner == graph_->inputs()[0] || IsConstant(owner);
  }
  return false;
}

c10::IValue TorchModule::Get(const JitValue* value) const {
  const JitNode* node = value->node();
  if (node->kind() == c10::prim::Constant) {
    auto iv = torch::jit::toIValue(value);
    if (!iv) throw std::runtime_error("constant without a value: " + value->debugName());
    return *iv;
  }
  if (node->kind() == c10::prim::GetAttr) {
    const JitValue* owner = node->input(0);
    const std::string& name = node->s(c10::attr::name);
    if (owner == graph_->inputs()[0]) return module_.attr(name);
    c10::IValue parent = Get(owner);
    if (!parent.isObject()) throw std::runtime_error("attribute of a non-object: " + name);
    return parent.toObject()->getAttr(name);
  }
  throw std::runtime_error("value %" + value->debugName() + " is computed at run time (" +
                           node->kind().toQualString() + ")");
}

FWD_TORCH_NAMESPACE_END
