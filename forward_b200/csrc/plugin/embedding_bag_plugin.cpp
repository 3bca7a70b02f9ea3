// Implementation of the EmbeddingBag_TRT plugin on top of the C ABI (include/fwd_eb.h).
// Behaviour at the TensorRT boundary follows Forward's
// source/trt_engine/trt_network_crt/plugins/embedding_bag_plugin/embedding_bag_plugin.cpp
// (line references below are to that file) unless a comment says otherwise.
#include "embedding_bag_plugin.h"

#include <cuda_runtime_api.h>

#include <cstdio>
#include <cstring>
#include <map>

#include "blob_io.h"
#include "fwd_eb.h"

FWD_TRT_NAMESPACE_BEGIN

namespace {

constexpr uint32_t kTrailerMagic = 0x32424546u;  // "FEB2"
enum : uint32_t { kHalfTable = 1, kHalfOutput = 2, kIncludeLast = 4, kWeighted = 8 };

void LogError(const char* what) {
  if (auto* logger = getLogger()) logger->log(nvinfer1::ILogger::Severity::kERROR, what);
}

int LogStatus(int rc, const char* where) {
  if (rc != 0) {
    char msg[640];
    std::snprintf(msg, sizeof(msg), "EmbeddingBag_TRT %s failed (%d): %s", where, rc,
                  fwd_eb_last_error_string());
    LogError(msg);
  }
  return rc;
}

nvinfer1::DimsExprs Invalid() {
  nvinfer1::DimsExprs bad;
  bad.nbDims = -1;
  return bad;
}

uint32_t PackFlags(const EmbeddingBagOptions& o) {
  return (o.half_table ? kHalfTable : 0u) | (o.half_output ? kHalfOutput : 0u) |
         (o.include_last_offset ? kIncludeLast : 0u) | (o.has_per_sample_weights ? kWeighted : 0u);
}

size_t TableBytes(int dim, int64_t count, bool half) {
  return (size_t)dim * (size_t)count * (half ? 2u : 4u);
}

// Bytes of the float vector in the blob: fp16 tables ride in it padded to whole floats.
size_t BlobFloatCount(int dim, int64_t count, bool half) {
  return (TableBytes(dim, count, half) + 3) / 4;
}

// Blob layout "002" (tables that stay outside the plugin).  It opens with an int that no "001"
// blob can open with (there it is `dim`, positive):
//   int32 -2 | char[4] "002" | int32 dim | int64 count | int64 data_offset | int32 op |
//   uint32 flags | int64 padding_idx | uint32 key length | key bytes
constexpr int kLayout002 = -2;

// ---- registered external tables -----------------------------------------------------------
struct ExternalTable {
  const void* ptr;
  int device;
  long long rows;
  int dim;
  bool half;
};
std::mutex g_registry_lock;
std::map<std::string, ExternalTable>& Registry() {
  static std::map<std::string, ExternalTable> r;
  return r;
}
bool FindExternal(const std::string& key, ExternalTable* out) {
  std::lock_guard<std::mutex> hold(g_registry_lock);
  auto it = Registry().find(key);
  if (it == Registry().end()) return false;
  *out = it->second;
  return true;
}

// ---- one user of the library's built-in split scratch at a time, per GPU ---------------------
// fwd_eb_forward_static_scratch keeps its partial sums in ONE array per GPU.  TensorRT may run
// several execution contexts (each with its own clone of this plugin) or auxiliary streams at
// once, so calls are chained through an event per GPU: a call waits for the previous user's
// kernels, and leaves its own mark behind.  The lock covers wait + launch + record, so two host
// threads cannot both wait for the same predecessor.
std::mutex g_scratch_lock;
cudaEvent_t g_scratch_event[64] = {};

cudaEvent_t ScratchEvent(int dev) {  // call with g_scratch_lock held
  if (dev < 0 || dev >= 64) return nullptr;
  if (!g_scratch_event[dev] &&
      cudaEventCreateWithFlags(&g_scratch_event[dev], cudaEventDisableTiming) != cudaSuccess) {
    cudaGetLastError();
    g_scratch_event[dev] = nullptr;
  }
  return g_scratch_event[dev];
}

int OrderedStaticScratch(fwd_eb_params* p, cudaStream_t stream) {
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  int dev = -1;
  if (cudaStreamIsCapturing(stream, &capturing) != cudaSuccess || cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    capturing = cudaStreamCaptureStatusActive;  // cannot tell: take the path that needs no ordering
  }
  if (capturing == cudaStreamCaptureStatusNone) {
    std::lock_guard<std::mutex> hold(g_scratch_lock);
    cudaEvent_t ev = ScratchEvent(dev);
    if (ev && cudaStreamWaitEvent(stream, ev, 0) == cudaSuccess) {
      const int rc = fwd_eb_forward_static_scratch(p, stream);
      cudaEventRecord(ev, stream);
      return rc;
    }
    cudaGetLastError();
  }
  // A stream that is being captured cannot wait for work outside its graph, and the array's
  // address must not be looked up for the first time inside a capture: one CTA per bag needs
  // no scratch at all.
  p->strategy = FWD_EB_STRATEGY_CTA;
  return fwd_eb_forward(p, stream);
}

}  // namespace

// ---- launchers with the reference's signatures ---------------------------------------------

void Gather(const int* input, float* output, int batch_size, int offset, const float* data,
            int count, int dim, int data_offset, const cudaStream_t& stream) {
  LogStatus(fwd_eb_gather_f32(input, output, batch_size, offset, data, count, dim, data_offset, stream),
            "Gather");
}

void EmbeddingBagWithFixedOffset(const int* input, float* output, int batch_size, int offset,
                                 const float* data, int count, int dim, int data_offset,
                                 int op_type, const cudaStream_t& stream) {
  LogStatus(fwd_eb_bag_fixed_f32(input, output, batch_size, offset, data, count, dim, data_offset,
                                 op_type, stream),
            "EmbeddingBagWithFixedOffset");
}

void EmbeddingBag(const int* input, const int* input_2, float* output, int input_size,
                  int block_size, const float* data, int count, int dim, int data_offset,
                  int op_type, const cudaStream_t& stream) {
  LogStatus(fwd_eb_bag_f32(input, input_2, output, input_size, block_size, data, count, dim,
                           data_offset, op_type, stream),
            "EmbeddingBag");
}

// ---- shared table ----------------------------------------------------------------------------

EmbeddingTable::EmbeddingTable(const void* host_bytes, size_t num_bytes, bool half) : half_(half) {
  const char* p = static_cast<const char*>(host_bytes);
  host_.assign(p, p + num_bytes);
}

EmbeddingTable::EmbeddingTable(const void* device_table, int device, bool half, const std::string& key)
    : half_(half), external_(true), key_(key) {
  device_.emplace_back(device, const_cast<void*>(device_table));
}

EmbeddingTable::~EmbeddingTable() {
  if (external_) return;  // the caller's memory
  int prev = -1;
  cudaGetDevice(&prev);
  for (auto& entry : device_) {
    if (cudaSetDevice(entry.first) == cudaSuccess) cudaFree(entry.second);
  }
  if (prev >= 0) cudaSetDevice(prev);
}

const void* EmbeddingTable::Device() noexcept {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  std::lock_guard<std::mutex> hold(lock_);
  for (auto& entry : device_) {
    if (entry.first == dev) return entry.second;
  }
  if (external_) return nullptr;  // registered for another GPU
  void* d = nullptr;
  const size_t bytes = host_.empty() ? 16 : host_.size();
  if (cudaMalloc(&d, bytes) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  if (!host_.empty() &&
      cudaMemcpy(d, host_.data(), host_.size(), cudaMemcpyHostToDevice) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(d);
    return nullptr;
  }
  device_.emplace_back(dev, d);
  ++uploads_;
  return d;
}

// ---- plugin -----------------------------------------------------------------------------------

EmbeddingBagPlugin::EmbeddingBagPlugin(const float* data, int dim, int count, int offset,
                                       ReduceOperation op)
    : EmbeddingBagPlugin(static_cast<const void*>(data), dim, count, offset, op,
                         EmbeddingBagOptions{}) {}

EmbeddingBagPlugin::EmbeddingBagPlugin(const void* data, int dim, int count, int offset,
                                       ReduceOperation op, const EmbeddingBagOptions& options)
    : opt_(options), op_(op), dim_(dim), count_(count), data_offset_(offset) {
  valid_ = dim > 0 && count >= 0 && (data != nullptr || count == 0);
  if (valid_) {
    table_ = std::make_shared<EmbeddingTable>(data, TableBytes(dim, count, opt_.half_table),
                                              opt_.half_table);
  } else {
    LogError("EmbeddingBag_TRT: bad constructor arguments");
  }
}

EmbeddingBagPlugin::EmbeddingBagPlugin(const std::string& key, int dim, int64_t count, int64_t offset,
                                       ReduceOperation op, const EmbeddingBagOptions& options)
    : opt_(options), op_(op), dim_(dim), count_(count), data_offset_(offset) {
  ExternalTable ext;
  valid_ = dim > 0 && count >= 0 && FindExternal(key, &ext) && ext.dim == dim && ext.rows >= count &&
           ext.half == opt_.half_table;
  if (valid_) {
    table_ = std::make_shared<EmbeddingTable>(ext.ptr, ext.device, ext.half, key);
  } else {
    LogError("EmbeddingBag_TRT: external weights are not registered under that name, or their "
             "geometry (dim, rows, element type) does not match the layer");
  }
}

EmbeddingBagPlugin::EmbeddingBagPlugin(void const* serialData, size_t serialLength) {
  blob::Reader in(serialData, serialLength);
  int first = 0;
  {
    blob::Reader peek = in;
    peek.value(&first);
  }
  if (first == kLayout002) {
    char tag[4] = {0, 0, 0, 0};
    int op = 0;
    uint32_t flags = 0, keylen = 0;
    int64_t pad = -1;
    in.value(&first);
    in.value(&tag);
    in.value(&dim_);
    in.value(&count_);
    in.value(&data_offset_);
    in.value(&op);
    in.value(&flags);
    in.value(&pad);
    in.value(&keylen);
    std::string key;
    std::vector<char> raw;
    bool ok = in.ok() && std::memcmp(tag, "002", 4) == 0 && keylen <= 4096 && keylen <= in.left();
    if (ok) {
      const char* base = static_cast<const char*>(serialData) + (serialLength - in.left());
      key.assign(base, base + keylen);
    }
    op_ = static_cast<ReduceOperation>(op);
    opt_.half_table = flags & kHalfTable;
    opt_.half_output = flags & kHalfOutput;
    opt_.include_last_offset = flags & kIncludeLast;
    opt_.has_per_sample_weights = flags & kWeighted;
    opt_.padding_idx = pad;
    ExternalTable ext;
    valid_ = ok && dim_ > 0 && count_ >= 0 && FindExternal(key, &ext) && ext.dim == dim_ &&
             ext.rows >= count_ && ext.half == opt_.half_table;
    if (valid_) {
      table_ = std::make_shared<EmbeddingTable>(ext.ptr, ext.device, ext.half, key);
    } else {
      LogError("EmbeddingBag_TRT: \"002\" blob is damaged, or the weights it names are not registered "
               "(fwd_eb_plugin_register_weights) with the geometry it records");
    }
    return;
  }
  // reference order (.cpp:44-51): dim, count, data_offset, op, vector<float>
  std::vector<char> payload;
  int op = 0, count32 = 0, offset32 = 0;
  in.value(&dim_);
  in.value(&count32);
  in.value(&offset32);
  in.value(&op);
  count_ = count32;
  data_offset_ = offset32;
  in.counted(&payload, sizeof(float));
  op_ = static_cast<ReduceOperation>(op);
  uint32_t magic = 0, flags = 0;
  if (in.ok() && in.left() >= 16) {
    blob::Reader tail = in;
    int64_t pad = -1;
    if (tail.value(&magic) && magic == kTrailerMagic && tail.value(&flags) && tail.value(&pad)) {
      opt_.half_table = flags & kHalfTable;
      opt_.half_output = flags & kHalfOutput;
      opt_.include_last_offset = flags & kIncludeLast;
      opt_.has_per_sample_weights = flags & kWeighted;
      opt_.padding_idx = pad;
    }
  }
  valid_ = in.ok() && dim_ > 0 && count_ >= 0 &&
           payload.size() >= TableBytes(dim_, count_, opt_.half_table);
  if (valid_) {
    table_ = std::make_shared<EmbeddingTable>(payload.data(),
                                              TableBytes(dim_, count_, opt_.half_table),
                                              opt_.half_table);
  } else {
    LogError("EmbeddingBag_TRT: truncated or inconsistent serialized plugin");
  }
}

EmbeddingBagPlugin::EmbeddingBagPlugin(const EmbeddingBagPlugin& o)
    : table_(o.table_), d_data_(nullptr), opt_(o.opt_), op_(o.op_), dim_(o.dim_), count_(o.count_),
      data_offset_(o.data_offset_), valid_(o.valid_), namespace_(o.namespace_) {}

EmbeddingBagPlugin::~EmbeddingBagPlugin() noexcept { terminate(); }

int EmbeddingBagPlugin::getNbOutputs() const noexcept { return 1; }

nvinfer1::DimsExprs EmbeddingBagPlugin::getOutputDimensions(
    int outputIndex, const nvinfer1::DimsExprs* inputs, int nbInputs,
    nvinfer1::IExprBuilder& exprBuilder) noexcept {
  if (outputIndex != 0 || !inputs || nbInputs < 1) return Invalid();
  const bool two_d = inputs[0].nbDims == 2;
  const int structural = nbInputs - (opt_.has_per_sample_weights ? 1 : 0);
  // one structural input: 2-D [batch, L] indices (.cpp:59-80)
  if (structural == 1) {
    if (!two_d) {
      LogError("EmbeddingBag_TRT: a single input must be a 2-D index matrix");
      return Invalid();
    }
    nvinfer1::DimsExprs output = inputs[0];
    if (op_ != ReduceOperation::GATHER) {
      output.d[1] = exprBuilder.constant(dim_);
    } else if (dim_ > 1) {  // gather keeps [batch, L] and appends dim (not for dim == 1, .cpp:73-76)
      output.nbDims += 1;
      output.d[2] = exprBuilder.constant(dim_);
    }
    return output;
  }
  if (structural != 2) return Invalid();
  // indices + offsets: offsets are 1-D, or [1, B] as DLRM slices them (.cpp:82-85)
  const nvinfer1::DimsExprs& off = inputs[1];
  const bool row_vector = off.nbDims == 2 && off.d[0]->isConstant() && off.d[0]->getConstantValue() == 1;
  if (!(off.nbDims == 1 || row_vector)) {
    LogError("EmbeddingBag_TRT: offsets must be 1-D or [1, B]");
    return Invalid();
  }
  if (op_ == ReduceOperation::GATHER) {
    LogError("EmbeddingBag_TRT: GATHER takes no offsets");  // .cpp:89-92
    return Invalid();
  }
  nvinfer1::DimsExprs output;
  output.nbDims = 2;
  const nvinfer1::IDimensionExpr* bags = off.nbDims == 1 ? off.d[0] : off.d[1];
  if (opt_.include_last_offset) {
    bags = exprBuilder.operation(nvinfer1::DimensionOperation::kSUB, *bags, *exprBuilder.constant(1));
  }
  output.d[0] = bags;
  output.d[1] = exprBuilder.constant(dim_);
  return output;
}

bool EmbeddingBagPlugin::supportsFormatCombination(int pos, const nvinfer1::PluginTensorDesc* inOut,
                                                   int nbInputs, int nbOutputs) noexcept {
  const int max_inputs = opt_.has_per_sample_weights ? 3 : 2;
  if (!inOut || nbInputs < 1 || nbInputs > max_inputs || nbOutputs != 1 || pos < 0 ||
      pos >= nbInputs + nbOutputs)
    return false;
  const nvinfer1::PluginTensorDesc& d = inOut[pos];
  if (d.format != nvinfer1::TensorFormat::kLINEAR) return false;
  if (pos >= nbInputs) {  // the output: fp32 as the reference (.cpp:109-112), fp16 on request
    return d.type == (opt_.half_output ? nvinfer1::DataType::kHALF : nvinfer1::DataType::kFLOAT);
  }
  if (opt_.has_per_sample_weights && pos == nbInputs - 1) return d.type == nvinfer1::DataType::kFLOAT;
  return d.type == nvinfer1::DataType::kINT32;  // indices and offsets (.cpp:105-108)
}

void EmbeddingBagPlugin::configurePlugin(const nvinfer1::DynamicPluginTensorDesc*, int,
                                         const nvinfer1::DynamicPluginTensorDesc*, int) noexcept {
  // The reference uploads its own copy here (.cpp:116-127); this plugin asks the shared table,
  // which uploads at most once per GPU however many clones exist.
  if (!valid_ || d_data_) return;
  d_data_ = table_->Device();
  if (!d_data_) LogError("EmbeddingBag_TRT: could not place the table on the device");
  // Calls with a few very long bags go through the library's built-in scratch array.  Its device
  // address is looked up on first use, which must not happen inside a stream capture: do it
  // here, where TensorRT is still setting up, together with the event that orders its users.
  if (fwd_eb_static_scratch_prepare() == 0) {
    int dev = -1;
    if (cudaGetDevice(&dev) == cudaSuccess) {
      std::lock_guard<std::mutex> hold(g_scratch_lock);
      ScratchEvent(dev);
    }
  }
  cudaGetLastError();
}

size_t EmbeddingBagPlugin::getWorkspaceSize(const nvinfer1::PluginTensorDesc*, int,
                                            const nvinfer1::PluginTensorDesc*, int) const noexcept {
  return 0;  // as the reference (.cpp:129-133); long bags use fwd_eb_forward_static_scratch
}

int EmbeddingBagPlugin::initialize() noexcept { return valid_ ? 0 : 1; }

void EmbeddingBagPlugin::terminate() noexcept { d_data_ = nullptr; }

int EmbeddingBagPlugin::enqueue(const nvinfer1::PluginTensorDesc* inputDesc,
                                const nvinfer1::PluginTensorDesc* outputDesc,
                                const void* const* inputs, void* const* outputs, void* workspace,
                                cudaStream_t stream) noexcept {
  (void)workspace;
  if (!valid_ || !inputDesc || !outputDesc || !inputs || !outputs) return 1;
  if (inputDesc[0].type != nvinfer1::DataType::kINT32) {
    LogError("Unsupported input data type");  // .cpp:182-185
    return -1;
  }
  const void* table = d_data_ ? d_data_ : table_->Device();
  if (!table && count_ > 0) {
    LogError("EmbeddingBag_TRT: table is not on the device");
    return 1;
  }
  fwd_eb_params p;
  std::memset(&p, 0, sizeof(p));
  p.table = table;
  p.table_dtype = opt_.half_table ? FWD_EB_F16 : FWD_EB_F32;
  p.dim = dim_;
  p.num_rows = count_;
  p.row_lo = data_offset_;
  p.indices = inputs[0];
  p.index_dtype = FWD_EB_I32;
  p.mode = static_cast<int>(op_);
  p.padding_idx = opt_.padding_idx;
  p.include_last_offset = opt_.include_last_offset;
  p.out = outputs[0];
  p.out_dtype = outputDesc[0].type == nvinfer1::DataType::kHALF ? FWD_EB_F16 : FWD_EB_F32;

  const nvinfer1::Dims& idims = inputDesc[0].dims;
  int next_input = 1;
  if (idims.nbDims > 1) {
    // 2-D indices: every bag has d[1] entries (.cpp:152-171)
    const int64_t batch = idims.d[0], len = idims.d[1];
    p.num_indices = batch * len;
    if (op_ != ReduceOperation::GATHER) {
      p.fixed_len = (int32_t)len;
      p.num_bags = batch;
      if (len == 0) return 1;
    }
  } else {
    // 1-D indices + offsets; the number of bags is the number of offsets (.cpp:173-181)
    p.num_indices = idims.d[0];
    const nvinfer1::Dims& odims = inputDesc[1].dims;
    const int64_t n_off = odims.nbDims == 1 ? odims.d[0] : odims.d[1];
    p.offsets = inputs[1];
    p.num_bags = n_off - (opt_.include_last_offset ? 1 : 0);
    next_input = 2;
  }
  if (opt_.has_per_sample_weights) p.per_sample_weights = static_cast<const float*>(inputs[next_input]);

  int rc;
  if (op_ != ReduceOperation::GATHER && fwd_eb_workspace_size(&p) > 0 &&
      fwd_eb_workspace_size(&p) <= FWD_EB_STATIC_SCRATCH_BYTES) {
    // few, very long bags: TensorRT gave no workspace (getWorkspaceSize is 0), so split through
    // the library's built-in scratch, one user at a time per GPU
    rc = OrderedStaticScratch(&p, stream);
  } else {
    rc = fwd_eb_forward(&p, stream);
  }
  return LogStatus(rc, "enqueue") == 0 ? 0 : 1;
}

size_t EmbeddingBagPlugin::getSerializationSize() const noexcept {
  if (table_ && table_->External())
    return sizeof(int) + 4 + sizeof(int) + 2 * sizeof(int64_t) + sizeof(int) + sizeof(uint32_t) +
           sizeof(int64_t) + sizeof(uint32_t) + table_->Key().size();
  return 4 * sizeof(int) + sizeof(size_t) +
         BlobFloatCount(dim_, count_, opt_.half_table) * sizeof(float) + 2 * sizeof(uint32_t) +
         sizeof(int64_t);
}

void EmbeddingBagPlugin::serialize(void* buffer) const noexcept {
  // reference layout first (.cpp:196-202) so its reader and ours agree on the common part
  blob::Writer out(buffer);
  if (table_ && table_->External()) {  // layout "002": the table's name instead of its bytes
    const char tag[4] = {'0', '0', '2', 0};
    out.value(kLayout002);
    out.value(tag);
    out.value(dim_);
    out.value(count_);
    out.value(data_offset_);
    out.value(static_cast<int>(op_));
    out.value(PackFlags(opt_));
    out.value(opt_.padding_idx);
    out.value(static_cast<uint32_t>(table_->Key().size()));
    out.bytes(table_->Key().data(), table_->Key().size());
    return;
  }
  out.value(dim_);
  out.value(static_cast<int>(count_));        // an embedded table never exceeds the int the creator took
  out.value(static_cast<int>(data_offset_));
  out.value(static_cast<int>(op_));
  const size_t floats = BlobFloatCount(dim_, count_, opt_.half_table);
  const size_t bytes = table_ ? table_->Host().size() : 0;
  out.value<size_t>(floats);
  out.bytes(table_ ? table_->Host().data() : nullptr, bytes);
  const char zeros[4] = {0, 0, 0, 0};
  out.bytes(zeros, floats * sizeof(float) - bytes);
  out.value(kTrailerMagic);
  out.value(PackFlags(opt_));
  out.value(opt_.padding_idx);
}

const char* EmbeddingBagPlugin::getPluginType() const noexcept { return EMBEDDING_BAG_PLUGIN_NAME; }
const char* EmbeddingBagPlugin::getPluginVersion() const noexcept { return EMBEDDING_BAG_PLUGIN_VERSION; }
void EmbeddingBagPlugin::destroy() noexcept { delete this; }

nvinfer1::IPluginV2DynamicExt* EmbeddingBagPlugin::clone() const noexcept {
  return new (std::nothrow) EmbeddingBagPlugin(*this);
}

void EmbeddingBagPlugin::setPluginNamespace(const char* pluginNamespace) noexcept {
  namespace_ = pluginNamespace ? pluginNamespace : "";
}
const char* EmbeddingBagPlugin::getPluginNamespace() const noexcept { return namespace_.c_str(); }

nvinfer1::DataType EmbeddingBagPlugin::getOutputDataType(int index, const nvinfer1::DataType* inputTypes,
                                                         int nbInputs) const noexcept {
  (void)index;
  (void)inputTypes;
  (void)nbInputs;
  return opt_.half_output ? nvinfer1::DataType::kHALF : nvinfer1::DataType::kFLOAT;
}

// ---- creator ----------------------------------------------------------------------------------

EmbeddingBagPluginCreator::EmbeddingBagPluginCreator() {
  using nvinfer1::PluginField;
  using nvinfer1::PluginFieldType;
  // the reference's five (.cpp:229-243) ...
  mPluginAttributes.emplace_back(PluginField("dim", nullptr, PluginFieldType::kINT32, 1));
  mPluginAttributes.emplace_back(PluginField("count", nullptr, PluginFieldType::kINT32, 1));
  mPluginAttributes.emplace_back(PluginField("offset", nullptr, PluginFieldType::kINT32, 1));
  mPluginAttributes.emplace_back(PluginField("op", nullptr, PluginFieldType::kINT32, 1));
  mPluginAttributes.emplace_back(PluginField("data", nullptr, PluginFieldType::kFLOAT32, 1));
  // ... and the optional ones
  mPluginAttributes.emplace_back(PluginField("padding_idx", nullptr, PluginFieldType::kINT32, 1));
  mPluginAttributes.emplace_back(PluginField("include_last_offset", nullptr, PluginFieldType::kINT32, 1));
  mPluginAttributes.emplace_back(PluginField("per_sample_weights", nullptr, PluginFieldType::kINT32, 1));
  mPluginAttributes.emplace_back(PluginField("half_output", nullptr, PluginFieldType::kINT32, 1));
  mPluginAttributes.emplace_back(PluginField("external_weights", nullptr, PluginFieldType::kCHAR, 1));
  mPluginAttributes.emplace_back(PluginField("half_table", nullptr, PluginFieldType::kINT32, 1));
  mFC.nbFields = (int)mPluginAttributes.size();
  mFC.fields = mPluginAttributes.data();
}

const char* EmbeddingBagPluginCreator::getPluginName() const noexcept { return EMBEDDING_BAG_PLUGIN_NAME; }
const char* EmbeddingBagPluginCreator::getPluginVersion() const noexcept { return EMBEDDING_BAG_PLUGIN_VERSION; }
const nvinfer1::PluginFieldCollection* EmbeddingBagPluginCreator::getFieldNames() noexcept { return &mFC; }

nvinfer1::IPluginV2DynamicExt* EmbeddingBagPluginCreator::createPlugin(
    const char* name, const nvinfer1::PluginFieldCollection* fc) noexcept {
  (void)name;
  if (!fc || (fc->nbFields > 0 && !fc->fields)) return nullptr;
  int dim = 0, count = 0, offset = 0, op = 0;
  const void* data = nullptr;
  bool have[5] = {false, false, false, false, false};
  EmbeddingBagOptions opt;
  std::string external_key;
  bool half_table_field = false;
  auto int_field = [](const nvinfer1::PluginField& f, int* out) {
    if (f.type != nvinfer1::PluginFieldType::kINT32 || !f.data) return false;
    *out = *static_cast<const int*>(f.data);
    return true;
  };
  for (int i = 0; i < fc->nbFields; ++i) {
    const nvinfer1::PluginField& f = fc->fields[i];
    if (!f.name) return nullptr;
    int v = 0;
    if (!std::strcmp(f.name, "dim")) {
      if (!(have[0] = int_field(f, &dim))) return nullptr;
    } else if (!std::strcmp(f.name, "count")) {
      if (!(have[1] = int_field(f, &count))) return nullptr;
    } else if (!std::strcmp(f.name, "offset")) {
      if (!(have[2] = int_field(f, &offset))) return nullptr;
    } else if (!std::strcmp(f.name, "op")) {
      if (!(have[3] = int_field(f, &op))) return nullptr;
    } else if (!std::strcmp(f.name, "data")) {
      // fp32 as the reference passes it (.cpp:283-285), or fp16 for half tables
      if (f.type == nvinfer1::PluginFieldType::kFLOAT16) {
        opt.half_table = true;
      } else if (f.type != nvinfer1::PluginFieldType::kFLOAT32) {
        LogError("EmbeddingBag_TRT: field 'data' must be FLOAT32 or FLOAT16");
        return nullptr;
      }
      data = f.data;
      have[4] = true;
    } else if (!std::strcmp(f.name, "padding_idx")) {
      if (!int_field(f, &v)) return nullptr;
      opt.padding_idx = v;
    } else if (!std::strcmp(f.name, "include_last_offset")) {
      if (!int_field(f, &v)) return nullptr;
      opt.include_last_offset = v != 0;
    } else if (!std::strcmp(f.name, "per_sample_weights")) {
      if (!int_field(f, &v)) return nullptr;
      opt.has_per_sample_weights = v != 0;
    } else if (!std::strcmp(f.name, "half_output")) {
      if (!int_field(f, &v)) return nullptr;
      opt.half_output = v != 0;
    } else if (!std::strcmp(f.name, "external_weights")) {
      // the name a device table was registered under: the plugin holds no copy of the table
      if (f.type != nvinfer1::PluginFieldType::kCHAR || !f.data || f.length <= 0 || f.length > 4096) {
        LogError("EmbeddingBag_TRT: field 'external_weights' must be a CHAR string");
        return nullptr;
      }
      external_key.assign(static_cast<const char*>(f.data), (size_t)f.length);
      while (!external_key.empty() && external_key.back() == '\0') external_key.pop_back();
    } else if (!std::strcmp(f.name, "half_table")) {
      if (!int_field(f, &v)) return nullptr;
      half_table_field = v != 0;
    } else {
      LogError("EmbeddingBag_TRT: unknown creator field");  // the reference asserts (.cpp:286-288)
      return nullptr;
    }
  }
  if (!external_key.empty()) {
    have[4] = true;  // no table bytes travel with an external table
    opt.half_table = half_table_field;
  }
  for (bool h : have) {
    if (!h) {
      LogError("EmbeddingBag_TRT: fields dim, count, offset, op and data are required");
      return nullptr;
    }
  }
  switch (op) {
    case 0: case 1: case 2: case 3: case 999:
      break;
    default:
      LogError("EmbeddingBag_TRT: unknown op");
      return nullptr;
  }
  if (opt.has_per_sample_weights && op != 0) {
    LogError("EmbeddingBag_TRT: per_sample_weights need op 0 (sum)");
    return nullptr;
  }
  auto* obj = external_key.empty()
                  ? new (std::nothrow) EmbeddingBagPlugin(data, dim, count, offset,
                                                          static_cast<ReduceOperation>(op), opt)
                  : new (std::nothrow) EmbeddingBagPlugin(external_key, dim, count, offset,
                                                          static_cast<ReduceOperation>(op), opt);
  if (!obj) return nullptr;
  if (!obj->Valid()) {
    obj->destroy();
    return nullptr;
  }
  obj->setPluginNamespace(mNamespace.c_str());
  return obj;
}

nvinfer1::IPluginV2DynamicExt* EmbeddingBagPluginCreator::deserializePlugin(
    const char* name, const void* serialData, size_t serialLength) noexcept {
  (void)name;
  if (!serialData) return nullptr;
  auto* obj = new (std::nothrow) EmbeddingBagPlugin(serialData, serialLength);
  if (!obj) return nullptr;
  if (!obj->Valid()) {
    obj->destroy();
    return nullptr;
  }
  obj->setPluginNamespace(mNamespace.c_str());
  return obj;
}

FWD_TRT_NAMESPACE_END

extern "C" int fwd_eb_plugin_register_weights(const char* key, const void* d_table, int device,
                                              long long num_rows, int dim, int half) {
  using namespace fwd::trt_;
  if (!key || !*key || !d_table || device < 0 || num_rows < 0 || dim <= 0) return -1;
  std::lock_guard<std::mutex> hold(g_registry_lock);
  auto it = Registry().find(key);
  if (it != Registry().end() &&
      (it->second.rows != num_rows || it->second.dim != dim || it->second.half != (half != 0)))
    return -2;  // the name is taken by a table of another shape
  Registry()[key] = ExternalTable{d_table, device, num_rows, dim, half != 0};
  return 0;
}

extern "C" int fwd_eb_plugin_unregister_weights(const char* key) {
  using namespace fwd::trt_;
  if (!key) return -1;
  std::lock_guard<std::mutex> hold(g_registry_lock);
  return Registry().erase(key) ? 0 : -1;
}
