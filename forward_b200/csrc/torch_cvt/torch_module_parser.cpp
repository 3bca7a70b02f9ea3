#include "torch_module_parser.h"

#include <algorithm>

FWD_TORCH_NAMESPACE_BEGIN

namespace {

int OutputIndex(const JitValue* value) {
  const auto outs = value->node()->outputs();
  return (int)(std::find(outs.begin(), outs.end(), value) - outs.begin());
}

bool ConstInt(const TorchModule& m, const JitValue* v, int64_t* out) {
  if (!m.IsConstant(v)) return false;
  const c10::IValue iv = m.Get(v);
  if (!iv.isInt()) return false;
  *out = iv.toInt();
  return true;
}

}  // namespace

bool Parser::Parse(const std::string& module_path) {
  network_ = ParsedNetwork();
  created_.clear();
  error_.clear();
  if (!module_.Load(module_path)) return Fail("load failed: " + module_.Error());
  const auto outputs = module_.Graph()->outputs();
  if (outputs.empty()) return Fail("the graph has no output");
  for (const JitValue* out : outputs) {
    const JitNode* node = out->node();
    if (node->kind() == c10::prim::TupleConstruct || node->kind() == c10::prim::ListConstruct) {
      for (const JitValue* item : node->inputs()) {
        std::vector<int> layers;
        if (!ParseOutput(item, &layers)) return false;
        network_.outputs.push_back(layers);
      }
    } else {
      std::vector<int> layers;
      if (!ParseOutput(out, &layers)) return false;
      network_.outputs.push_back(layers);
    }
  }
  if (network_.layers.empty()) return Fail("no aten::embedding_bag node in the graph");
  return true;
}

// One output tensor: a bag, or a concatenation of bags along dim 1.
bool Parser::ParseOutput(const JitValue* value, std::vector<int>* layers) {
  const JitNode* node = value->node();
  if (node->kind() == c10::aten::cat) {
    int64_t dim = 0;
    if (!ConstInt(module_, node->input(1), &dim) || (dim != 1 && dim != -1))
      return Fail("aten::cat around embedding bags is converted for dim 1 only");
    const JitNode* list = node->input(0)->node();
    if (list->kind() != c10::prim::ListConstruct) return Fail("aten::cat of something that is not a list of tensors");
    for (const JitValue* item : list->inputs()) {
      if (!ParseOutput(item, layers)) return false;  // nested concatenations flatten
    }
    return true;
  }
  int layer = -1;
  if (!ParseValue(value, &layer)) return false;
  layers->push_back(layer);
  return true;
}

// A value that must be the pooled output of an embedding_bag node.
bool Parser::ParseValue(const JitValue* value, int* layer) {
  const JitNode* node = value->node();
  ILayerDescCreator* creator = desc_manager_.FindDescCreator(node, module_);
  if (creator == nullptr)
    return Fail(std::string("no converter for ") + node->kind().toQualString() +
                " (only embedding bags, their concatenation and input slicing are converted)");
  if (OutputIndex(value) != 0)
    return Fail("only the pooled output of aten::embedding_bag can be used (its offset2bag / bag_size / "
                "max_indices outputs are training-time by-products)");
  auto seen = created_.find(node);  // the same node feeding several outputs: one layer
  if (seen != created_.end()) {
    *layer = seen->second;
    return true;
  }
  std::vector<const JitValue*> input_values;
  std::shared_ptr<TrtLayerDesc> desc = creator->Create(node, module_, input_values);
  if (desc == nullptr || input_values.empty())
    return Fail(std::string("creating the description of ") + node->kind().toQualString() + " failed");
  ParsedLayer parsed;
  parsed.desc = std::dynamic_pointer_cast<TrtEmbeddingBagDesc>(desc);
  if (!parsed.desc) return Fail("unexpected description type " + desc->Name());
  for (const JitValue* in : input_values) {
    InputRef ref;
    if (!ParseInput(in, &ref)) return false;
    parsed.inputs.push_back(ref);
  }
  network_.layers.push_back(parsed);
  *layer = (int)network_.layers.size() - 1;
  created_[node] = *layer;
  return true;
}

// A layer input: a graph input, one row of one, or one element of a list input.
bool Parser::ParseInput(const JitValue* value, InputRef* ref) {
  const auto& inputs = module_.Inputs();
  auto position = [&](const JitValue* v) {
    auto it = std::find(inputs.begin(), inputs.end(), v);
    return it == inputs.end() ? -1 : (int)(it - inputs.begin());
  };
  int at = position(value);
  if (at >= 0) {
    ref->graph_input = at;
    return true;
  }
  const JitNode* node = value->node();
  if (node->kind() == c10::aten::select) {
    int64_t dim = 0, index = 0;
    at = position(node->input(0));
    if (at < 0 || !ConstInt(module_, node->input(1), &dim) || !ConstInt(module_, node->input(2), &index) ||
        dim != 0 || index < 0)
      return Fail("aten::select feeding an embedding bag must take row k (constant, dim 0) of a graph input");
    ref->graph_input = at;
    ref->element = (int)index;
    return true;
  }
  if (node->kind() == c10::prim::ListUnpack || node->kind() == c10::aten::__getitem__) {
    at = position(node->input(0));
    int64_t index = OutputIndex(value);
    if (node->kind() == c10::aten::__getitem__ && !ConstInt(module_, node->input(1), &index)) at = -1;
    if (at < 0 || index < 0) return Fail("a list element feeding an embedding bag must come from a graph input, by a constant index");
    ref->graph_input = at;
    ref->element = (int)index;
    ref->from_list = true;
    return true;
  }
  return Fail(std::string("an embedding bag input computed by ") + node->kind().toQualString() +
              " is not converted (inputs must be graph inputs, rows of them, or list elements)");
}

FWD_TORCH_NAMESPACE_END
