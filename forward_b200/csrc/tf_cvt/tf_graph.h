// A frozen TensorFlow GraphDef, read straight from its protobuf wire format.
//
// Forward walks TensorFlow graphs through the TensorFlow C API (TF_Graph / TF_Operation,
// wrapped by Operation / Output / Tensor / Graph in source/fwd_tf/tf_cvt/tf_cpp_api.h:67-203 and
// tf_graph.h).  This repository converts one node pattern only and must not depend on
// libtensorflow, so the same four wrappers are provided over a small reader of the GraphDef
// message: GraphDef.node(1) -> NodeDef{name(1), op(2), input(3), device(4), attr(5)},
// AttrValue{s(2), i(3), f(4), b(5), type(6), shape(7), tensor(8)}, TensorProto{dtype(1),
// tensor_shape(2), tensor_content(4), half_val(13), float_val(5), double_val(6), int_val(7),
// int64_val(10), bool_val(11)}.  Field numbers are those of TensorFlow's published .proto files.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#define FWD_TF_NAMESPACE_BEGIN \
  namespace fwd {              \
  namespace tf_ {
#define FWD_TF_NAMESPACE_END \
  }                          \
  }

FWD_TF_NAMESPACE_BEGIN

// tensorflow::DataType values used on this path
enum TfDataType {
  TF_INVALID = 0,
  TF_FLOAT = 1,
  TF_DOUBLE = 2,
  TF_INT32 = 3,
  TF_INT64 = 9,
  TF_BOOL = 10,
  TF_HALF = 19
};

size_t DataTypeSize(int dtype);

// A constant held by the graph (the value attribute of a Const node), densely expanded.
class Tensor {
 public:
  Tensor() = default;
  Tensor(int dtype, std::vector<int64_t> dims, std::vector<char> bytes)
      : dtype_(dtype), dims_(std::move(dims)), bytes_(std::move(bytes)) {}

  bool Valid() const { return dtype_ != TF_INVALID; }
  int Type() const { return dtype_; }
  const std::vector<int64_t>& Dims() const { return dims_; }
  size_t Size() const { return DataTypeSize(dtype_) ? bytes_.size() / DataTypeSize(dtype_) : 0; }
  size_t ByteSize() const { return bytes_.size(); }
  template <typename T>
  const T* Data() const {
    return reinterpret_cast<const T*>(bytes_.data());
  }
  // a scalar / one-element int32 tensor (tf_cpp_api.h:151-156); `ok` reports the checks
  int AsInt(bool* ok) const;
  std::vector<int> AsIntList(bool* ok) const;

 private:
  int dtype_{TF_INVALID};
  std::vector<int64_t> dims_;
  std::vector<char> bytes_;
};

struct AttrValue {
  enum Kind { kNone, kString, kInt, kFloat, kBool, kType, kShape, kTensor, kList } kind{kNone};
  std::string s;
  int64_t i{0};
  float f{0};
  bool b{false};
  int type{0};
  bool unknown_rank{false};
  std::vector<int64_t> shape;
  std::shared_ptr<Tensor> tensor;
};

struct NodeDef {
  std::string name, op, device;
  std::vector<std::pair<std::string, int>> inputs;  // data inputs: producer name, output index
  std::vector<std::string> control_inputs;          // "^name"
  std::map<std::string, AttrValue> attrs;
};

class Output;

class Graph {
 public:
  bool Load(const std::string& path);
  bool Parse(const void* bytes, size_t len);
  const std::string& Error() const { return error_; }

  const NodeDef* OperationByName(const std::string& name) const;
  const std::vector<NodeDef>& Nodes() const { return nodes_; }

 private:
  std::vector<NodeDef> nodes_;
  std::map<std::string, size_t> by_name_;
  std::string error_;
};

// One node of a graph (tf_cpp_api.h:67-124).  A default-constructed Operation is invalid.
class Operation {
 public:
  Operation() = default;
  Operation(const Graph* graph, const NodeDef* node) : graph_(graph), node_(node) {}

  bool Valid() const { return graph_ && node_; }
  std::string OpType() const { return node_ ? node_->op : ""; }
  std::string Name() const { return node_ ? node_->name : ""; }
  int NumInputs() const { return node_ ? (int)node_->inputs.size() : 0; }
  Output Input(int index) const;

  const AttrValue* Attr(const char* name) const;
  bool GetAttrBool(const char* name, bool fallback = false) const;
  int64_t GetAttrInt(const char* name, int64_t fallback = 0) const;
  int GetAttrType(const char* name) const;

  const Graph* GetGraph() const { return graph_; }
  const NodeDef* Node() const { return node_; }

 protected:
  const Graph* graph_{nullptr};
  const NodeDef* node_{nullptr};
};

// One output of a node (tf_cpp_api.h:171-203).
class Output : public Operation {
 public:
  Output() = default;
  Output(const Graph* graph, const NodeDef* node, int index) : Operation(graph, node), index_(index) {}
  int Index() const { return index_; }

  // The constant this output carries: a Const node's value, looked through Identity nodes.
  // Invalid when the output is not a compile-time constant.
  Tensor GetConstantTensor() const;
  // Static shape where the graph states it (Const value, Placeholder shape attribute, looked
  // through Identity); -1 for an unknown extent.  False when the rank is unknown.
  bool GetTensorShape(std::vector<int64_t>* dims) const;

 private:
  int index_{0};
};

FWD_TF_NAMESPACE_END
