// TrtEmbeddingBagDesc -> EmbeddingBag_TRT plugin layer.
//
// Same job and same flow as Forward's
// source/trt_engine/trt_network_crt/layer_creators/trt_embedding_bag_creator.h:41-86:
// look the creator up in TensorRT's registry by name and version, hand it the desc as plugin
// fields, add the plugin to the network, name the layer.  Differences: the table is passed
// with its real element type (the reference always says FLOAT32, :63-65, which misreads fp16
// weights), the extra attributes travel as optional fields, and a third input (per-sample
// weights) is accepted.
#pragma once

#include <string>
#include <vector>

#include "embedding_bag_plugin.h"
#include "layer_creator_iface.h"

FWD_TRT_NAMESPACE_BEGIN

template <>
class TLayerCreator<TrtEmbeddingBagDesc> : public ILayerCreator {
 public:
  ITensorVector CreateLayer(nvinfer1::INetworkDefinition* network, const TrtLayerDesc* layer_desc,
                            const ITensorVector& input_tensors) override {
    LOG(INFO) << "TrtEmbeddingBagDesc::CreateLayer";
    const auto desc = dynamic_cast<const TrtEmbeddingBagDesc*>(layer_desc);
    T_CHECK(desc);
    // indices [+ offsets] [+ per-sample weights]
    T_CHECK_LE(input_tensors.size(), desc->has_per_sample_weights ? 3u : 2u);
    T_CHECK(!input_tensors.empty());

    nvinfer1::IPluginCreator* creator = getPluginRegistry()->getPluginCreator(
        EMBEDDING_BAG_PLUGIN_NAME, EMBEDDING_BAG_PLUGIN_VERSION);
    T_CHECK(creator);

    const bool half = desc->data.Type() == nvinfer1::DataType::kHALF;
    const int padding = static_cast<int>(desc->padding_idx);
    const int last = desc->include_last_offset ? 1 : 0;
    const int weighted = desc->has_per_sample_weights ? 1 : 0;
    const int half_out = desc->half_output ? 1 : 0;
    std::vector<nvinfer1::PluginField> fields;
    fields.emplace_back("dim", &desc->dim, nvinfer1::PluginFieldType::kINT32, 1);
    fields.emplace_back("count", &desc->count, nvinfer1::PluginFieldType::kINT32, 1);
    fields.emplace_back("offset", &desc->offset, nvinfer1::PluginFieldType::kINT32, 1);
    fields.emplace_back("op", &desc->op, nvinfer1::PluginFieldType::kINT32, 1);
    const int half_table = half ? 1 : 0;
    if (desc->external_weights.empty()) {
      fields.emplace_back("data", desc->data.Data(),
                          half ? nvinfer1::PluginFieldType::kFLOAT16 : nvinfer1::PluginFieldType::kFLOAT32,
                          desc->dim * desc->count);
    } else {
      // the table was registered on the device under a name: only the name goes into the plugin
      fields.emplace_back("external_weights", desc->external_weights.c_str(),
                          nvinfer1::PluginFieldType::kCHAR, static_cast<int>(desc->external_weights.size()));
      if (half_table) fields.emplace_back("half_table", &half_table, nvinfer1::PluginFieldType::kINT32, 1);
    }
    if (padding >= 0) fields.emplace_back("padding_idx", &padding, nvinfer1::PluginFieldType::kINT32, 1);
    if (last) fields.emplace_back("include_last_offset", &last, nvinfer1::PluginFieldType::kINT32, 1);
    if (weighted) fields.emplace_back("per_sample_weights", &weighted, nvinfer1::PluginFieldType::kINT32, 1);
    if (half_out) fields.emplace_back("half_output", &half_out, nvinfer1::PluginFieldType::kINT32, 1);

    const nvinfer1::PluginFieldCollection collection{static_cast<int>(fields.size()), fields.data()};
    nvinfer1::IPluginV2* plugin = creator->createPlugin("embedding_bag", &collection);
    if (plugin == nullptr) {
      LOG(ERROR) << "Create Network: the EmbeddingBag_TRT creator rejected the layer description.";
      return {};
    }
    // the network keeps its own clone; ours is released as the reference's InferUniquePtr does
    nvinfer1::IPluginV2Layer* layer = network->addPluginV2(
        input_tensors.data(), static_cast<int>(input_tensors.size()), *plugin);
    plugin->destroy();
    if (layer == nullptr) {
      LOG(ERROR) << "Create Network: Fail to create [embedding_bag] layer.";
      return {};
    }
    layer->setName((std::to_string(network->getNbLayers()) + std::string(" [Embedding Bag]")).c_str());
    return {layer->getOutput(0)};
  }
};

FWD_TRT_NAMESPACE_END
