// TensorFlow node patterns -> TrtEmbeddingBagDesc.
//
// Same role and the same three patterns as Forward's
// source/fwd_tf/tf_cvt/tf_desc_creators/tf_embedding_bag_creator.h:41-140:
//
//   Sum(Mul([Identity](GatherV2(table, indices, axis 0)), m))            -> op 0   (SUM)
//   Sum(Square(Mul([Identity](GatherV2(table, indices, axis 0)), m)))    -> op 3   (SQUARE_SUM)
//   GatherV2(table, indices, axis 0)                                     -> op 999 (GATHER)
//
// i.e. the first- and second-order terms of a factorisation machine over a fixed number of
// feature ids per sample (indices [batch, L]; the plugin's fixed-length form).  The table is the
// constant feeding GatherV2, or the node "<scope>_weights" when the graph has one (:108-119).
//
// As in the reference, the second Mul operand `m` (a sequence mask or feature values) is NOT
// applied: the conversion is exact only where `m` is one for every looked-up id, which is how
// the reference's fixture builds it (a full-length sequence mask).  A warning is logged.
// Stricter than the reference, to fail instead of converting wrongly: a Sum must reduce axis 1
// without keep_dims (the reference does not look, :80-92), the table must be fp32 or fp16 and of
// rank 1 or 2, and every constant it needs must really be constant.
#pragma once

#include <memory>
#include <string>
#include <vector>

#include "fwd_log.h"
#include "i_tf_layer_creator.h"

FWD_TF_NAMESPACE_BEGIN

template <>
class TLayerDescCreator<TrtEmbeddingBagDesc> : public ILayerDescCreator {
 public:
  bool Check(const Operation& op) override {
    Operation gather;
    int op_type = 0;
    return Match(op, &gather, &op_type);
  }

  std::shared_ptr<TrtLayerDesc> Create(const Operation& op, const Graph& graph,
                                       std::vector<Output>& op_inputs) override {
    LOG(INFO) << "TrtEmbeddingBagDesc::Create";
    Operation gather;
    int op_type = 0;
    if (!Match(op, &gather, &op_type)) return nullptr;

    if (gather.NumInputs() != 3) return nullptr;
    const Output table = gather.Input(0);
    const Output indices = gather.Input(1);
    bool ok = false;
    const Tensor axis = gather.Input(2).GetConstantTensor();
    if (!axis.Valid() || axis.AsInt(&ok) != 0 || !ok) {
      LOG(ERROR) << "EmbeddingBag pattern at " << gather.Name() << ": gather axis must be the constant 0";
      return nullptr;
    }
    if (gather.GetAttrInt("batch_dims", 0) != 0) {
      LOG(ERROR) << "EmbeddingBag pattern at " << gather.Name() << ": batch_dims must be 0";
      return nullptr;
    }

    // a weights node generated from a file takes precedence (reference :108-119)
    std::string scope = table.Name();
    scope = scope.substr(0, scope.find_last_of('/')) + "_weights";
    Tensor weights;
    if (const NodeDef* from_file = graph.OperationByName(scope))
      weights = Output(&graph, from_file, 0).GetConstantTensor();
    else
      weights = table.GetConstantTensor();
    if (!weights.Valid() || weights.Size() == 0) {
      LOG(ERROR) << "EmbeddingBag pattern at " << gather.Name() << ": the table is not a constant";
      return nullptr;
    }
    const std::vector<int64_t>& dims = weights.Dims();
    if (dims.empty() || dims.size() > 2) {
      LOG(ERROR) << "EmbeddingBag pattern at " << gather.Name() << ": table of rank " << dims.size();
      return nullptr;
    }
    if (dims[0] > 0x7fffffffLL || (dims.size() == 2 && dims[1] > 0x7fffffffLL)) return nullptr;

    if (op.OpType() == "Sum") {
      // gathered tensor: [batch, L] + table dims[1:]; the pooled axis is L
      const int gathered_rank = 2 + (int)dims.size() - 1;
      bool axes_ok = false;
      const Tensor axes = op.Input(1).GetConstantTensor();
      const std::vector<int> list = axes.Valid() ? axes.AsIntList(&axes_ok) : std::vector<int>();
      const int axis1 = list.size() == 1 ? (list[0] < 0 ? list[0] + gathered_rank : list[0]) : -1;
      if (!axes_ok || axis1 != 1) {
        LOG(ERROR) << "EmbeddingBag pattern at " << op.Name() << ": Sum must reduce axis 1 only";
        return nullptr;
      }
      if (op.GetAttrBool("keep_dims", false)) {
        LOG(ERROR) << "EmbeddingBag pattern at " << op.Name() << ": keep_dims is not supported";
        return nullptr;
      }
      LOG(WARNING) << "EmbeddingBag pattern at " << op.Name()
                   << ": the second Mul operand is assumed to be all ones";
    }

    auto layer_desc = std::make_shared<TrtEmbeddingBagDesc>();
    if (weights.Type() == TF_FLOAT) {
      layer_desc->data.SetType(nvinfer1::DataType::kFLOAT);
    } else if (weights.Type() == TF_HALF) {
      layer_desc->data.SetType(nvinfer1::DataType::kHALF);
    } else {
      LOG(ERROR) << "EmbeddingBag pattern at " << gather.Name() << ": table dtype " << weights.Type();
      return nullptr;
    }
    layer_desc->data.SetData(weights.Data<char>(), (int64_t)weights.ByteSize());
    layer_desc->data.SetCount((int64_t)weights.Size());
    layer_desc->count = (int)dims[0];
    layer_desc->dim = dims.size() == 1 ? 1 : (int)dims[1];
    layer_desc->offset = 0;
    layer_desc->op = op_type;

    op_inputs.push_back(indices);
    return layer_desc;
  }

 private:
  // The three shapes a lookup takes in a frozen graph, as a table: the operator types met on the
  // way from the pattern's top node down to its GatherV2 (optional steps in brackets), and the
  // pooling mode each stands for.
  //   GatherV2                                          -> GATHER (999)
  //   Sum > Mul > [Identity] > GatherV2                 -> SUM (0)
  //   Sum > Square > Mul > [Identity] > GatherV2        -> SQUARE_SUM (3)
  struct Step {
    const char* type;
    bool optional;
  };
  static bool Descend(Operation at, const Step* steps, int n_steps, Operation* gather) {
    for (int i = 0; i < n_steps; ++i) {
      if (!at.Valid()) return false;
      if (at.OpType() == steps[i].type) {
        if (i + 1 == n_steps) {
          *gather = at;
          return true;
        }
        at = at.Input(0);
      } else if (!steps[i].optional) {
        return false;
      }
    }
    return false;
  }
  static bool Match(const Operation& op, Operation* gather, int* op_type) {
    static const Step kGather[] = {{"GatherV2", false}};
    static const Step kSum[] = {{"Sum", false}, {"Mul", false}, {"Identity", true}, {"GatherV2", false}};
    static const Step kSquareSum[] = {{"Sum", false}, {"Square", false}, {"Mul", false}, {"Identity", true},
                                      {"GatherV2", false}};
    static const struct {
      const Step* steps;
      int count;
      int mode;
    } kPatterns[] = {{kGather, 1, 999}, {kSum, 4, 0}, {kSquareSum, 5, 3}};
    for (const auto& pattern : kPatterns) {
      if (Descend(op, pattern.steps, pattern.count, gather)) {
        *op_type = pattern.mode;
        return true;
      }
    }
    return false;
  }
};

FWD_TF_NAMESPACE_END
