// Host-buffer sessions (include/fwd_eb_session.h): table residency, pinned
// staging slots and a small in-flight pipeline around fwd_eb_forward.
//
// Stands where the reference has TrtForwardEngine::Execute + BufferManager
// (source/trt_engine/trt_engine/trt_fwd_engine.cpp:105-154,
// trt_buffer_manager.h:78-98) and the plugin's table upload
// (embedding_bag_plugin.cpp:116-127).
#include <cstring>
#include <new>
#include <vector>

#include "eb_internal.h"
#include "fwd_eb_session.h"

using fwd_eb::cuda_fail;
using fwd_eb::fail;

namespace {

struct Slot {
  cudaStream_t stream = nullptr;
  cudaEvent_t done = nullptr;
  // pinned host staging
  void* h_idx = nullptr;
  void* h_off = nullptr;
  float* h_w = nullptr;
  void* h_out = nullptr;
  // device buffers
  void* d_idx = nullptr;
  void* d_off = nullptr;
  float* d_w = nullptr;
  void* d_out = nullptr;
  void* d_ws = nullptr;
  size_t ws_bytes = 0;
  bool busy = false;
  int64_t out_rows = 0;
};

struct DeviceGuard {
  int prev = -1;
  bool ok = false;
  explicit DeviceGuard(int want) {
    if (cudaGetDevice(&prev) != cudaSuccess) return;
    if (prev != want && cudaSetDevice(want) != cudaSuccess) return;
    ok = true;
    if (prev == want) prev = -1;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

}  // namespace

struct fwd_eb_session {
  fwd_eb_session_config cfg;
  int device = 0;
  void* d_table = nullptr;
  bool owns_table = false;
  size_t isize = 4, tsize = 4, osize = 4;
  std::vector<Slot> slots;

  int64_t offsets_per_call(int64_t bags) const {
    if (cfg.fixed_len > 0 || cfg.mode == FWD_EB_MODE_GATHER) return 0;
    return bags + (cfg.include_last_offset ? 1 : 0);
  }
  int64_t out_rows(int64_t n, int64_t bags) const {
    return cfg.mode == FWD_EB_MODE_GATHER ? n : bags;
  }
};

static void release(fwd_eb_session* s) {
  if (!s) return;
  DeviceGuard g(s->device);
  for (Slot& sl : s->slots) {
    if (sl.stream) cudaStreamSynchronize(sl.stream);
    if (sl.h_idx) cudaFreeHost(sl.h_idx);
    if (sl.h_off) cudaFreeHost(sl.h_off);
    if (sl.h_w) cudaFreeHost(sl.h_w);
    if (sl.h_out) cudaFreeHost(sl.h_out);
    if (sl.d_idx) cudaFree(sl.d_idx);
    if (sl.d_off) cudaFree(sl.d_off);
    if (sl.d_w) cudaFree(sl.d_w);
    if (sl.d_out) cudaFree(sl.d_out);
    if (sl.d_ws) cudaFree(sl.d_ws);
    if (sl.done) cudaEventDestroy(sl.done);
    if (sl.stream) cudaStreamDestroy(sl.stream);
  }
  if (s->owns_table && s->d_table) cudaFree(s->d_table);
  delete s;
}

#define SESSION_CUDA(call, what)                   \
  do {                                             \
    cudaError_t e_ = (call);                       \
    if (e_ != cudaSuccess) {                       \
      int rc_ = cuda_fail(e_, what);               \
      release(s);                                  \
      return rc_;                                  \
    }                                              \
  } while (0)

extern "C" {

int fwd_eb_session_create(const fwd_eb_session_config* cfg, fwd_eb_session** out) {
  if (!cfg || !out) return fail(FWD_EB_EINVAL, "session config or out pointer is null");
  *out = nullptr;
  if (cfg->dim <= 0 || cfg->num_rows < 0 || cfg->max_indices < 0 || cfg->max_bags < 0)
    return fail(FWD_EB_EINVAL, "bad session sizes");
  if (cfg->depth < 1 || cfg->depth > 16) return fail(FWD_EB_EINVAL, "depth must be 1..16");
  if ((cfg->table_dtype != FWD_EB_F32 && cfg->table_dtype != FWD_EB_F16) ||
      (cfg->out_dtype != FWD_EB_F32 && cfg->out_dtype != FWD_EB_F16) ||
      (cfg->index_dtype != FWD_EB_I32 && cfg->index_dtype != FWD_EB_I64))
    return fail(FWD_EB_EINVAL, "unknown dtype in session config");
  if (cfg->weighted && cfg->mode != FWD_EB_MODE_SUM)
    return fail(FWD_EB_EINVAL, "per_sample_weights need mode SUM");
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
    cudaGetLastError();
    return fail(FWD_EB_ENOGPU, "no CUDA device is available; this library has no CPU path");
  }
  int dev = cfg->device;
  if (dev < 0 && cudaGetDevice(&dev) != cudaSuccess) return fail(FWD_EB_ENOGPU, "cudaGetDevice failed");
  if (dev >= ndev) return fail(FWD_EB_EINVAL, "device %d does not exist", dev);

  fwd_eb_session* s = new (std::nothrow) fwd_eb_session();
  if (!s) return fail(FWD_EB_EINVAL, "out of host memory");
  s->cfg = *cfg;
  s->device = dev;
  s->isize = cfg->index_dtype == FWD_EB_I64 ? 8 : 4;
  s->tsize = cfg->table_dtype == FWD_EB_F16 ? 2 : 4;
  s->osize = cfg->out_dtype == FWD_EB_F16 ? 2 : 4;
  DeviceGuard g(dev);
  if (!g.ok) {
    delete s;
    return fail(FWD_EB_ENOGPU, "cannot select device %d", dev);
  }
  if (!cfg->external_table && cfg->num_rows > 0) {
    SESSION_CUDA(cudaMalloc(&s->d_table, (size_t)cfg->num_rows * cfg->dim * s->tsize),
                 "table allocation");
    s->owns_table = true;
  }
  const size_t n_idx = (size_t)(cfg->max_indices > 0 ? cfg->max_indices : 1);
  const size_t n_off = (size_t)s->offsets_per_call(cfg->max_bags) + 1;
  const size_t n_out =
      (size_t)(s->out_rows(cfg->max_indices, cfg->max_bags) > 0 ? s->out_rows(cfg->max_indices, cfg->max_bags) : 1) *
      cfg->dim;
  s->slots.resize(cfg->depth);
  for (Slot& sl : s->slots) {
    SESSION_CUDA(cudaStreamCreateWithFlags(&sl.stream, cudaStreamNonBlocking), "stream");
    SESSION_CUDA(cudaEventCreateWithFlags(&sl.done, cudaEventDisableTiming), "event");
    SESSION_CUDA(cudaMallocHost(&sl.h_idx, n_idx * s->isize), "pinned indices");
    SESSION_CUDA(cudaMallocHost(&sl.h_off, n_off * s->isize), "pinned offsets");
    SESSION_CUDA(cudaMallocHost(&sl.h_out, n_out * s->osize), "pinned output");
    SESSION_CUDA(cudaMalloc(&sl.d_idx, n_idx * s->isize), "device indices");
    SESSION_CUDA(cudaMalloc(&sl.d_off, n_off * s->isize), "device offsets");
    SESSION_CUDA(cudaMalloc(&sl.d_out, n_out * s->osize), "device output");
    if (cfg->weighted) {
      SESSION_CUDA(cudaMallocHost(reinterpret_cast<void**>(&sl.h_w), n_idx * sizeof(float)),
                   "pinned weights");
      SESSION_CUDA(cudaMalloc(reinterpret_cast<void**>(&sl.d_w), n_idx * sizeof(float)),
                   "device weights");
    }
  }
  *out = s;
  fwd_eb::clear_error();
  return 0;
}

void fwd_eb_session_destroy(fwd_eb_session* s) { release(s); }

int fwd_eb_session_load_table(fwd_eb_session* s, const void* h_rows, int64_t first_row,
                              int64_t rows) {
  if (!s || !h_rows) return fail(FWD_EB_EINVAL, "null argument");
  if (!s->d_table) return fail(FWD_EB_EINVAL, "session has no table storage");
  if (first_row < 0 || rows < 0 || first_row + rows > s->cfg.num_rows)
    return fail(FWD_EB_EINVAL, "rows [%lld, %lld) outside the table", (long long)first_row,
                (long long)(first_row + rows));
  DeviceGuard g(s->device);
  const size_t row_bytes = (size_t)s->cfg.dim * s->tsize;
  cudaError_t e = cudaMemcpy(static_cast<char*>(s->d_table) + (size_t)first_row * row_bytes, h_rows,
                             (size_t)rows * row_bytes, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return cuda_fail(e, "table upload");
  return 0;
}

void* fwd_eb_session_device_table(fwd_eb_session* s) { return s ? s->d_table : nullptr; }

int fwd_eb_session_adopt_table(fwd_eb_session* s, void* d_table) {
  if (!s || !d_table) return fail(FWD_EB_EINVAL, "null argument");
  if (s->owns_table) return fail(FWD_EB_EINVAL, "session already owns a table");
  s->d_table = d_table;
  return 0;
}

int fwd_eb_session_slot(fwd_eb_session* s, int32_t slot, void** h_indices, void** h_offsets,
                        float** h_weights, void** h_out) {
  if (!s || slot < 0 || slot >= (int32_t)s->slots.size())
    return fail(FWD_EB_EINVAL, "bad session or slot");
  Slot& sl = s->slots[slot];
  if (h_indices) *h_indices = sl.h_idx;
  if (h_offsets) *h_offsets = sl.h_off;
  if (h_weights) *h_weights = sl.h_w;
  if (h_out) *h_out = sl.h_out;
  return 0;
}

int fwd_eb_session_copy_bytes(fwd_eb_session* s, int64_t num_indices, int64_t num_bags,
                              int64_t* h2d, int64_t* d2h) {
  if (!s) return fail(FWD_EB_EINVAL, "null session");
  if (h2d)
    *h2d = num_indices * (int64_t)s->isize + s->offsets_per_call(num_bags) * (int64_t)s->isize +
           (s->cfg.weighted ? num_indices * 4 : 0);
  if (d2h) *d2h = s->out_rows(num_indices, num_bags) * s->cfg.dim * (int64_t)s->osize;
  return 0;
}

int fwd_eb_session_submit(fwd_eb_session* s, int32_t slot, int64_t num_indices, int64_t num_bags) {
  if (!s || slot < 0 || slot >= (int32_t)s->slots.size())
    return fail(FWD_EB_EINVAL, "bad session or slot");
  if (num_indices < 0 || num_bags < 0 || num_indices > s->cfg.max_indices ||
      num_bags > s->cfg.max_bags)
    return fail(FWD_EB_ETOOBIG, "call of %lld indices / %lld bags exceeds the session capacity",
                (long long)num_indices, (long long)num_bags);
  if (!s->d_table && s->cfg.num_rows > 0) return fail(FWD_EB_EINVAL, "no table loaded");
  Slot& sl = s->slots[slot];
  if (sl.busy) return fail(FWD_EB_EINVAL, "slot %d is still in flight: wait for it first", slot);
  DeviceGuard g(s->device);
  cudaError_t e;
  if (num_indices > 0) {
    e = cudaMemcpyAsync(sl.d_idx, sl.h_idx, (size_t)num_indices * s->isize, cudaMemcpyHostToDevice,
                        sl.stream);
    if (e != cudaSuccess) return cuda_fail(e, "indices H2D");
    if (s->cfg.weighted) {
      e = cudaMemcpyAsync(sl.d_w, sl.h_w, (size_t)num_indices * 4, cudaMemcpyHostToDevice, sl.stream);
      if (e != cudaSuccess) return cuda_fail(e, "weights H2D");
    }
  }
  const int64_t n_off = s->offsets_per_call(num_bags);
  if (n_off > 0) {
    e = cudaMemcpyAsync(sl.d_off, sl.h_off, (size_t)n_off * s->isize, cudaMemcpyHostToDevice,
                        sl.stream);
    if (e != cudaSuccess) return cuda_fail(e, "offsets H2D");
  }

  fwd_eb_params p;
  memset(&p, 0, sizeof(p));
  p.table = s->d_table;
  p.table_dtype = s->cfg.table_dtype;
  p.dim = s->cfg.dim;
  p.num_rows = s->cfg.num_rows;
  p.row_lo = s->cfg.row_lo;
  p.indices = sl.d_idx;
  p.offsets = n_off > 0 ? sl.d_off : nullptr;
  p.index_dtype = s->cfg.index_dtype;
  p.fixed_len = s->cfg.fixed_len;
  p.num_indices = num_indices;
  p.num_bags = s->cfg.mode == FWD_EB_MODE_GATHER ? 0 : num_bags;
  p.per_sample_weights = s->cfg.weighted ? sl.d_w : nullptr;
  p.mode = s->cfg.mode;
  p.include_last_offset = s->cfg.include_last_offset;
  p.padding_idx = s->cfg.padding_idx;
  p.out = sl.d_out;
  p.out_dtype = s->cfg.out_dtype;
  p.flags = s->cfg.flags;
  // scratch for split bags: grown on demand (rare: few, very long bags)
  const size_t need = fwd_eb_workspace_size(&p);
  if (need > sl.ws_bytes) {
    cudaStreamSynchronize(sl.stream);
    if (sl.d_ws) cudaFree(sl.d_ws);
    sl.d_ws = nullptr;
    sl.ws_bytes = 0;
    e = cudaMalloc(&sl.d_ws, need);
    if (e != cudaSuccess) return cuda_fail(e, "workspace allocation");
    sl.ws_bytes = need;
  }
  if (need > 0) {
    p.workspace = sl.d_ws;
    p.workspace_bytes = sl.ws_bytes;
  }
  int rc = fwd_eb_forward(&p, sl.stream);
  if (rc != 0) return rc;

  sl.out_rows = s->out_rows(num_indices, num_bags);
  if (sl.out_rows > 0) {
    e = cudaMemcpyAsync(sl.h_out, sl.d_out, (size_t)sl.out_rows * s->cfg.dim * s->osize,
                        cudaMemcpyDeviceToHost, sl.stream);
    if (e != cudaSuccess) return cuda_fail(e, "output D2H");
  }
  e = cudaEventRecord(sl.done, sl.stream);
  if (e != cudaSuccess) return cuda_fail(e, "event record");
  sl.busy = true;
  return 0;
}

int fwd_eb_session_wait(fwd_eb_session* s, int32_t slot) {
  if (!s || slot < 0 || slot >= (int32_t)s->slots.size())
    return fail(FWD_EB_EINVAL, "bad session or slot");
  Slot& sl = s->slots[slot];
  if (!sl.busy) return 0;
  cudaError_t e = cudaEventSynchronize(sl.done);
  sl.busy = false;
  if (e != cudaSuccess) return cuda_fail(e, "waiting for a slot");
  return 0;
}

int fwd_eb_session_run(fwd_eb_session* s, const void* h_indices, int64_t num_indices,
                       const void* h_offsets, int64_t num_bags, const float* h_weights,
                       void* h_out) {
  if (!s) return fail(FWD_EB_EINVAL, "null session");
  if (num_indices < 0 || num_bags < 0 || num_indices > s->cfg.max_indices ||
      num_bags > s->cfg.max_bags)
    return fail(FWD_EB_ETOOBIG, "call exceeds the session capacity");
  int rc = fwd_eb_session_wait(s, 0);
  if (rc) return rc;
  Slot& sl = s->slots[0];
  const int64_t n_off = s->offsets_per_call(num_bags);
  if (num_indices > 0) {
    if (!h_indices) return fail(FWD_EB_EINVAL, "indices is null");
    memcpy(sl.h_idx, h_indices, (size_t)num_indices * s->isize);
    if (s->cfg.weighted) {
      if (!h_weights) return fail(FWD_EB_EINVAL, "weights are null");
      memcpy(sl.h_w, h_weights, (size_t)num_indices * 4);
    }
  }
  if (n_off > 0) {
    if (!h_offsets) return fail(FWD_EB_EINVAL, "offsets is null");
    memcpy(sl.h_off, h_offsets, (size_t)n_off * s->isize);
  }
  rc = fwd_eb_session_submit(s, 0, num_indices, num_bags);
  if (rc) return rc;
  rc = fwd_eb_session_wait(s, 0);
  if (rc) return rc;
  const int64_t rows = s->out_rows(num_indices, num_bags);
  if (rows > 0) {
    if (!h_out) return fail(FWD_EB_EINVAL, "out is null");
    memcpy(h_out, sl.h_out, (size_t)rows * s->cfg.dim * s->osize);
  }
  return 0;
}

}  // extern "C"
