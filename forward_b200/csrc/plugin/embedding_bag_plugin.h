// EmbeddingBag_TRT plugin, version 001, on the sm_100a kernels behind the C ABI.
//
// Same class names, plugin name / version, creator fields and virtual overrides as
// Forward's source/trt_engine/trt_network_crt/plugins/embedding_bag_plugin/
// embedding_bag_plugin.h:36-161, so TensorRT (and Forward's layer creator) find and drive it
// unchanged.  What differs behind that surface:
//   * the table is held once: the plugin and all of its clones share one host copy and one
//     device copy per GPU (the reference keeps a host vector per clone and uploads once per
//     clone, embedding_bag_plugin.cpp:37-42,116-127,212-214);
//   * fp16 tables, padding_idx, include_last_offset and per_sample_weights (a third input)
//     are honoured; they travel as optional creator fields and as a trailer after the
//     reference's blob layout, so a blob written by the reference still loads;
//   * a table can stay outside the plugin: the host registers a device table under a name
//     (fwd_eb_plugin_register_weights) and the creator field `external_weights` / blob layout
//     "002" carry only that name plus 64-bit sizes, so a plan stays small and a table is never
//     copied through the host (the reference embeds the table in the plan and holds it in a
//     host vector, embedding_bag_plugin.cpp:37-51,191-202; common/fwd_weights.h:172 counts its
//     bytes in an int);
//   * nothing aborts: enqueue / initialize return non-zero and log through getLogger().
#pragma once

#include <NvInferPlugin.h>

#include <cstdint>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "fwd_macros.h"

namespace nvinfer1 {
namespace plugin {
// Forward's plugins derive their creators from this (plugins/common/plugin.h:34-46).
class BaseCreator : public IPluginCreator {
 public:
  void setPluginNamespace(const char* libNamespace) noexcept override { mNamespace = libNamespace; }
  const char* getPluginNamespace() const noexcept override { return mNamespace.c_str(); }

 protected:
  std::string mNamespace;
};
}  // namespace plugin
}  // namespace nvinfer1

FWD_TRT_NAMESPACE_BEGIN

constexpr const char* EMBEDDING_BAG_PLUGIN_NAME{"EmbeddingBag_TRT"};
constexpr const char* EMBEDDING_BAG_PLUGIN_VERSION{"001"};

enum class ReduceOperation { GATHER = 999, SUM = 0, MEAN = 1, MAX = 2, SQUARE_SUM = 3 };

// The three launchers of the reference header (embedding_bag_plugin.h:40-49), kept for
// source compatibility; they forward to the C ABI.
void Gather(const int* input, float* output, int batch_size, int offset, const float* data,
            int count, int dim, int data_offset, const cudaStream_t& stream);
void EmbeddingBagWithFixedOffset(const int* input, float* output, int batch_size, int offset,
                                 const float* data, int count, int dim, int data_offset,
                                 int op_type, const cudaStream_t& stream);
void EmbeddingBag(const int* input, const int* input_2, float* output, int input_size,
                  int block_size, const float* data, int count, int dim, int data_offset,
                  int op_type, const cudaStream_t& stream);

// A table shared by a plugin and its clones: host bytes plus device copies made on demand, or a
// caller-owned device table that was registered under a name (no host bytes, nothing to free).
class EmbeddingTable {
 public:
  EmbeddingTable(const void* host_bytes, size_t num_bytes, bool half);
  // external: `device_table` lives on GPU `device` and stays the caller's
  EmbeddingTable(const void* device_table, int device, bool half, const std::string& key);
  ~EmbeddingTable();
  EmbeddingTable(const EmbeddingTable&) = delete;
  EmbeddingTable& operator=(const EmbeddingTable&) = delete;

  // Device copy on the current GPU; uploaded on the first call for that GPU.  nullptr on failure.
  const void* Device() noexcept;
  const std::vector<char>& Host() const { return host_; }
  bool Half() const { return half_; }
  int Uploads() const { return uploads_; }
  bool External() const { return external_; }
  const std::string& Key() const { return key_; }

 private:
  std::vector<char> host_;
  bool half_;
  bool external_{false};
  std::string key_;
  std::mutex lock_;
  std::vector<std::pair<int, void*>> device_;  // (ordinal, pointer)
  int uploads_{0};
};

struct EmbeddingBagOptions {
  bool half_table{false};
  bool half_output{false};
  bool include_last_offset{false};
  bool has_per_sample_weights{false};
  int64_t padding_idx{-1};
};

class EmbeddingBagPlugin final : public nvinfer1::IPluginV2DynamicExt {
 public:
  // ---- construction -------------------------------------------------------------------------
  EmbeddingBagPlugin() = delete;
  // reference constructor: fp32 table, reference semantics
  EmbeddingBagPlugin(const float* data, int dim, int count, int offset, ReduceOperation op);
  // extended constructor: `data` holds dim*count elements of the table's element type
  EmbeddingBagPlugin(const void* data, int dim, int count, int offset, ReduceOperation op,
                     const EmbeddingBagOptions& options);
  // external table: rows [offset, offset + count) of the logical table, registered under `key`
  EmbeddingBagPlugin(const std::string& key, int dim, int64_t count, int64_t offset, ReduceOperation op,
                     const EmbeddingBagOptions& options);
  // from an engine blob (layout "001" with or without trailer, or "002")
  EmbeddingBagPlugin(void const* blob, size_t blob_bytes);
  ~EmbeddingBagPlugin() noexcept override;

  // ---- identity, copies, blob ------------------------------------------------------------------
  const char* getPluginType() const noexcept override;
  const char* getPluginVersion() const noexcept override;
  const char* getPluginNamespace() const noexcept override;
  void setPluginNamespace(const char* ns) noexcept override;
  nvinfer1::IPluginV2DynamicExt* clone() const noexcept override;
  void destroy() noexcept override;
  size_t getSerializationSize() const noexcept override;
  void serialize(void* dst) const noexcept override;

  // ---- shape and format negotiation ------------------------------------------------------------
  int getNbOutputs() const noexcept override;
  nvinfer1::DataType getOutputDataType(int index, const nvinfer1::DataType* in_types,
                                       int nb_inputs) const noexcept override;
  nvinfer1::DimsExprs getOutputDimensions(int out_index, const nvinfer1::DimsExprs* in_dims,
                                          int nb_inputs,
                                          nvinfer1::IExprBuilder& exprs) noexcept override;
  bool supportsFormatCombination(int pos, const nvinfer1::PluginTensorDesc* in_out, int nb_inputs,
                                 int nb_outputs) noexcept override;
  size_t getWorkspaceSize(const nvinfer1::PluginTensorDesc* in, int nb_inputs,
                          const nvinfer1::PluginTensorDesc* out, int nb_outputs) const noexcept override;

  // ---- life cycle and execution ----------------------------------------------------------------
  void configurePlugin(const nvinfer1::DynamicPluginTensorDesc* in, int nb_inputs,
                       const nvinfer1::DynamicPluginTensorDesc* out, int nb_outputs) noexcept override;
  int initialize() noexcept override;
  void terminate() noexcept override;
  int enqueue(const nvinfer1::PluginTensorDesc* in_desc, const nvinfer1::PluginTensorDesc* out_desc,
              const void* const* inputs, void* const* outputs, void* workspace,
              cudaStream_t stream) noexcept override;

  // ---- for tests: did construction / deserialisation succeed, and how the table is shared -------
  bool Valid() const { return valid_; }
  const std::shared_ptr<EmbeddingTable>& Table() const { return table_; }
  const EmbeddingBagOptions& Options() const { return opt_; }

 private:
  EmbeddingBagPlugin(const EmbeddingBagPlugin& other);  // clone: shares the table

  std::shared_ptr<EmbeddingTable> table_;
  const void* d_data_{nullptr};  // cached Device() of the GPU configured on
  EmbeddingBagOptions opt_;
  ReduceOperation op_{ReduceOperation::SUM};
  int dim_{0};
  int64_t count_{0};        // rows held (the reference's int `count_`)
  int64_t data_offset_{0};  // logical id of row 0 (the reference's int `data_offset_`)
  bool valid_{true};
  std::string namespace_;
};

class EmbeddingBagPluginCreator : public nvinfer1::plugin::BaseCreator {
 public:
  EmbeddingBagPluginCreator();
  ~EmbeddingBagPluginCreator() override = default;
  const char* getPluginName() const noexcept override;
  const char* getPluginVersion() const noexcept override;
  const nvinfer1::PluginFieldCollection* getFieldNames() noexcept override;
  nvinfer1::IPluginV2DynamicExt* createPlugin(const char* name,
                                              const nvinfer1::PluginFieldCollection* fc) noexcept override;
  nvinfer1::IPluginV2DynamicExt* deserializePlugin(const char* name, const void* serialData,
                                                   size_t serialLength) noexcept override;

 private:
  nvinfer1::PluginFieldCollection mFC;
  std::vector<nvinfer1::PluginField> mPluginAttributes;
};

FWD_TRT_NAMESPACE_END

extern "C" {
// Tables that stay outside the plugin.  Register a device table (row-major [num_rows, dim], fp32
// or fp16, on GPU `device`, owned by the caller, alive as long as any plugin uses it) under a
// name before createPlugin / deserializePlugin meets that name in the `external_weights` field or
// in a "002" blob.  0 on success; a name can be registered again with identical geometry (the
// pointer is replaced).  Unregister when no plugin uses the name any more.
int fwd_eb_plugin_register_weights(const char* key, const void* d_table, int device, long long num_rows,
                                   int dim, int half);
int fwd_eb_plugin_unregister_weights(const char* key);
}
