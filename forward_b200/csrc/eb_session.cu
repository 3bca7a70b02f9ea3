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
  // One pinned input block and its device twin, laid out [offsets | indices | weights]
  // (each area 256-byte aligned), so that a call's inputs go up in ONE copy: on a B200 a second,
  // small host-to-device copy per call costs about 30 us of copy-engine time when copies in both
  // directions are in flight, far more than its bytes.
  char* h_in = nullptr;
  char* d_in = nullptr;
  void* h_out = nullptr;  // pinned
  void* d_out = nullptr;
  void* d_ws = nullptr;
  size_t ws_bytes = 0;
  bool busy = false;
  int64_t out_rows = 0;
};

struct Span {
  size_t begin, end;
};

// Areas closer than this are sent as one copy, unused bytes between them included.
constexpr size_t kMergeGapBytes = 1u << 20;

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
  size_t off_at = 0, idx_at = 0, w_at = 0, in_bytes = 0;  // areas of a slot's input block

  void* h_idx(const Slot& sl) const { return sl.h_in + idx_at; }
  void* h_off(const Slot& sl) const { return sl.h_in + off_at; }
  float* h_w(const Slot& sl) const {
    return cfg.weighted ? reinterpret_cast<float*>(sl.h_in + w_at) : nullptr;
  }
  void* d_idx(const Slot& sl) const { return sl.d_in + idx_at; }
  void* d_off(const Slot& sl) const { return sl.d_in + off_at; }
  float* d_w(const Slot& sl) const {
    return cfg.weighted ? reinterpret_cast<float*>(sl.d_in + w_at) : nullptr;
  }

  // The host-to-device copies of one call: the used part of each area, neighbours merged
  // across small gaps.  Returns the number of spans written to `out` (at most 3).
  int input_spans(int64_t num_indices, int64_t num_bags, Span* out) const {
    Span used[3];
    int n = 0;
    const int64_t n_off = offsets_per_call(num_bags);
    if (n_off > 0) used[n++] = {off_at, off_at + (size_t)n_off * isize};
    if (num_indices > 0) {
      used[n++] = {idx_at, idx_at + (size_t)num_indices * isize};
      if (cfg.weighted) used[n++] = {w_at, w_at + (size_t)num_indices * 4};
    }
    int m = 0;
    for (int i = 0; i < n; ++i) {
      if (m > 0 && used[i].begin - out[m - 1].end <= kMergeGapBytes)
        out[m - 1].end = used[i].end;
      else
        out[m++] = used[i];
    }
    return m;
  }

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
    if (sl.h_in) cudaFreeHost(sl.h_in);
    if (sl.h_out) cudaFreeHost(sl.h_out);
    if (sl.d_in) cudaFree(sl.d_in);
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
  auto up256 = [](size_t v) { return (v + 255) & ~(size_t)255; };
  s->off_at = 0;
  s->idx_at = up256(n_off * s->isize);
  s->w_at = s->idx_at + up256(n_idx * s->isize);
  s->in_bytes = s->w_at + (cfg->weighted ? up256(n_idx * sizeof(float)) : 0);
  s->slots.resize(cfg->depth);
  for (Slot& sl : s->slots) {
    SESSION_CUDA(cudaStreamCreateWithFlags(&sl.stream, cudaStreamNonBlocking), "stream");
    SESSION_CUDA(cudaEventCreateWithFlags(&sl.done, cudaEventDisableTiming), "event");
    SESSION_CUDA(cudaMallocHost(reinterpret_cast<void**>(&sl.h_in), s->in_bytes), "pinned inputs");
    SESSION_CUDA(cudaMallocHost(&sl.h_out, n_out * s->osize), "pinned output");
    SESSION_CUDA(cudaMalloc(reinterpret_cast<void**>(&sl.d_in), s->in_bytes), "device inputs");
    SESSION_CUDA(cudaMalloc(&sl.d_out, n_out * s->osize), "device output");
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
  if (h_indices) *h_indices = s->h_idx(sl);
  if (h_offsets) *h_offsets = s->h_off(sl);
  if (h_weights) *h_weights = s->h_w(sl);
  if (h_out) *h_out = sl.h_out;
  return 0;
}

int fwd_eb_session_copy_bytes(fwd_eb_session* s, int64_t num_indices, int64_t num_bags,
                              int64_t* h2d, int64_t* d2h) {
  if (!s) return fail(FWD_EB_EINVAL, "null session");
  if (h2d) {  // what submit really sends, bytes between merged areas included
    Span spans[3];
    const int n = s->input_spans(num_indices, num_bags, spans);
    *h2d = 0;
    for (int i = 0; i < n; ++i) *h2d += (int64_t)(spans[i].end - spans[i].begin);
  }
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
  Span spans[3];
  const int n_spans = s->input_spans(num_indices, num_bags, spans);
  for (int i = 0; i < n_spans; ++i) {
    e = cudaMemcpyAsync(sl.d_in + spans[i].begin, sl.h_in + spans[i].begin,
                        spans[i].end - spans[i].begin, cudaMemcpyHostToDevice, sl.stream);
    if (e != cudaSuccess) return cuda_fail(e, "inputs H2D");
  }
  const int64_t n_off = s->offsets_per_call(num_bags);

  fwd_eb_params p;
  memset(&p, 0, sizeof(p));
  p.table = s->d_table;
  p.table_dtype = s->cfg.table_dtype;
  p.dim = s->cfg.dim;
  p.num_rows = s->cfg.num_rows;
  p.row_lo = s->cfg.row_lo;
  p.indices = s->d_idx(sl);
  p.offsets = n_off > 0 ? s->d_off(sl) : nullptr;
  p.index_dtype = s->cfg.index_dtype;
  p.fixed_len = s->cfg.fixed_len;
  p.num_indices = num_indices;
  p.num_bags = s->cfg.mode == FWD_EB_MODE_GATHER ? 0 : num_bags;
  p.per_sample_weights = s->d_w(sl);
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
    memcpy(s->h_idx(sl), h_indices, (size_t)num_indices * s->isize);
    if (s->cfg.weighted) {
      if (!h_weights) return fail(FWD_EB_EINVAL, "weights are null");
      memcpy(s->h_w(sl), h_weights, (size_t)num_indices * 4);
    }
  }
  if (n_off > 0) {
    if (!h_offsets) return fail(FWD_EB_EINVAL, "offsets is null");
    memcpy(s->h_off(sl), h_offsets, (size_t)n_off * s->isize);
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
