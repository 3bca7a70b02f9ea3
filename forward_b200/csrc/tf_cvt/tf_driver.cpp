// Test harness for the TensorFlow parser slice: frozen GraphDef -> walk back from the requested
// outputs -> description creators -> TrtEmbeddingBagDesc, and on into the TensorRT-side layer
// creator and plugin (through the host driver of libfwd_eb_plugin.so).  This is Forward's
// Parser::Parse / ParseOperation chain (source/fwd_tf/tf_cvt/tf_graph_parser.cpp) cut down to the
// node patterns this repository converts: an operation no creator claims is walked through to its
// inputs, a claimed one becomes a description and the walk stops at its run-time inputs.
// Not part of the product ABI.
#include <cstdio>
#include <cstring>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "tf_desc_manager.h"

struct fwd_eb_host;
extern "C" fwd_eb_host* fwd_eb_host_build_desc(const void* embedding_bag_desc, int idx_rank,
                                               const int* idx_dims, int off_rank, const int* off_dims,
                                               int weights_rank, const int* weights_dims);

namespace {
struct Found {
  std::string node;        // the operation the description replaces (a Sum or a GatherV2)
  std::string input_name;  // its run-time input (the indices)
  std::shared_ptr<fwd::TrtEmbeddingBagDesc> desc;
};
}  // namespace

struct fwd_eb_tf_parsed {
  fwd::tf_::Graph graph;
  std::vector<Found> found;
};

extern "C" {

void fwd_eb_tf_free(fwd_eb_tf_parsed* p) { delete p; }

// Parses the GraphDef at `path` and converts what the outputs named in `outputs` (comma
// separated) depend on.  Returns nullptr and writes the reason to `err` when the file does not
// parse, an output does not exist, or a claimed pattern cannot be converted faithfully.
fwd_eb_tf_parsed* fwd_eb_tf_parse(const char* path, const char* outputs, char* err, size_t err_cap) {
  auto fail = [&](const std::string& why) -> fwd_eb_tf_parsed* {
    if (err && err_cap) std::snprintf(err, err_cap, "%s", why.c_str());
    return nullptr;
  };
  std::unique_ptr<fwd_eb_tf_parsed> p(new fwd_eb_tf_parsed());
  if (!p->graph.Load(path)) return fail("load failed: " + p->graph.Error());
  fwd::tf_::TfDescManager manager;
  std::vector<const fwd::tf_::NodeDef*> stack;
  std::string list = outputs ? outputs : "";
  size_t pos = 0;
  while (pos <= list.size()) {
    size_t comma = list.find(',', pos);
    if (comma == std::string::npos) comma = list.size();
    const std::string name = list.substr(pos, comma - pos);
    pos = comma + 1;
    if (name.empty()) continue;
    const fwd::tf_::NodeDef* node = p->graph.OperationByName(name);
    if (!node) return fail("no operation named " + name);
    stack.push_back(node);
  }
  if (stack.empty()) return fail("no output names given");
  std::set<const fwd::tf_::NodeDef*> seen;
  // depth-first from the outputs, inputs in order, so descriptions come out in a stable order
  std::vector<const fwd::tf_::NodeDef*> order(stack.rbegin(), stack.rend());
  while (!order.empty()) {
    const fwd::tf_::NodeDef* node = order.back();
    order.pop_back();
    if (!seen.insert(node).second) continue;
    fwd::tf_::Operation op(&p->graph, node);
    if (fwd::tf_::ILayerDescCreator* creator = manager.FindDescCreator(op)) {
      std::vector<fwd::tf_::Output> inputs;
      std::shared_ptr<fwd::TrtLayerDesc> desc = creator->Create(op, p->graph, inputs);
      if (!desc) return fail("the EmbeddingBag description creator rejected " + node->name);
      Found f;
      f.node = node->name;
      f.desc = std::dynamic_pointer_cast<fwd::TrtEmbeddingBagDesc>(desc);
      if (!f.desc || inputs.size() != 1) return fail("unexpected description for " + node->name);
      f.input_name = inputs[0].Name();
      p->found.push_back(std::move(f));
      continue;  // the pattern's own nodes are covered by the description
    }
    for (int i = node->inputs.size() > 0 ? (int)node->inputs.size() - 1 : -1; i >= 0; --i) {
      const fwd::tf_::NodeDef* in = p->graph.OperationByName(node->inputs[i].first);
      if (!in) return fail("input " + node->inputs[i].first + " of " + node->name + " is missing");
      order.push_back(in);
    }
  }
  return p.release();
}

int fwd_eb_tf_num_descs(const fwd_eb_tf_parsed* p) { return p ? (int)p->found.size() : -1; }

const char* fwd_eb_tf_desc_node(const fwd_eb_tf_parsed* p, int i) {
  return (p && i >= 0 && i < (int)p->found.size()) ? p->found[i].node.c_str() : "";
}

const char* fwd_eb_tf_desc_input(const fwd_eb_tf_parsed* p, int i) {
  return (p && i >= 0 && i < (int)p->found.size()) ? p->found[i].input_name.c_str() : "";
}

int fwd_eb_tf_desc_info(const fwd_eb_tf_parsed* p, int i, int* dim, int* count, int* offset, int* op,
                        int* half_table) {
  if (!p || i < 0 || i >= (int)p->found.size()) return -1;
  const auto& d = *p->found[i].desc;
  *dim = d.dim;
  *count = d.count;
  *offset = d.offset;
  *op = d.op;
  *half_table = d.data.Type() == nvinfer1::DataType::kHALF;
  return 0;
}

size_t fwd_eb_tf_desc_weights(const fwd_eb_tf_parsed* p, int i, void* dst, size_t cap) {
  if (!p || i < 0 || i >= (int)p->found.size()) return 0;
  const size_t n = (size_t)p->found[i].desc->data.Bytes();
  if (dst && cap >= n) std::memcpy(dst, p->found[i].desc->data.Data(), n);
  return n;
}

// On into the TensorRT side: description -> LayerCreatorManager ->
// TLayerCreator<TrtEmbeddingBagDesc> -> EmbeddingBag_TRT plugin; run the handle with
// fwd_eb_host_run of the plugin library.  The TensorFlow patterns have one input: indices
// [batch, L].
fwd_eb_host* fwd_eb_tf_build_engine(const fwd_eb_tf_parsed* p, int i, int idx_rank, const int* idx_dims) {
  if (!p || i < 0 || i >= (int)p->found.size()) return nullptr;
  return fwd_eb_host_build_desc(p->found[i].desc.get(), idx_rank, idx_dims, 0, nullptr, 0, nullptr);
}

}  // extern "C"
