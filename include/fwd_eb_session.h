/*
 * fwd_eb_session.h — host-buffer front of the EmbeddingBag path (C ABI).
 *
 * A session owns what the reference spreads over its plugin and engine:
 *   - the device copy of the table, uploaded once
 *     (EmbeddingBagPlugin::configurePlugin, source/trt_engine/trt_network_crt/
 *      plugins/embedding_bag_plugin/embedding_bag_plugin.cpp:116-127);
 *   - per-call staging of host inputs to the device and of the result back
 *     (TrtForwardEngine::Execute, source/trt_engine/trt_engine/
 *      trt_fwd_engine.cpp:105-154, and BufferManager::PrepareInputBuffer,
 *      source/trt_engine/trt_engine/trt_buffer_manager.h:78-98);
 *   - the stream the kernels run on (trt_fwd_engine.cpp:315-346).
 *
 * Unlike the reference's Execute — copy in, synchronise, enqueue, synchronise,
 * copy out, one call at a time — a session keeps `depth` calls in flight on
 * separate streams so the PCIe copies of one call hide behind the kernel and
 * copies of its neighbours.  Host buffers are pinned slots the caller fills in
 * place (no extra memcpy); a convenience call takes any host pointers.
 *
 * Every function returns 0 on success, a negative FWD_EB_E* code or a positive
 * cudaError_t; text via fwd_eb_last_error_string().  A session is bound to the
 * CUDA device it was created on and may be used from one thread at a time.
 */
#ifndef FWD_EB_SESSION_H_
#define FWD_EB_SESSION_H_

#include "fwd_eb.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct fwd_eb_session fwd_eb_session;

typedef struct fwd_eb_session_config {
  int32_t table_dtype;   /* FWD_EB_F32 / FWD_EB_F16 */
  int32_t dim;
  int64_t num_rows;      /* rows held by this session's device */
  int64_t row_lo;        /* logical id of local row 0 (row shard origin) */
  int32_t mode;          /* FWD_EB_MODE_* */
  int32_t out_dtype;
  int32_t index_dtype;   /* FWD_EB_I32 / FWD_EB_I64 */
  int32_t include_last_offset;
  int64_t padding_idx;   /* < 0 = none */
  int32_t fixed_len;     /* > 0: 2-D indices, no offsets */
  int32_t weighted;      /* calls carry per_sample_weights */
  int64_t max_indices;   /* capacity of one call */
  int64_t max_bags;
  int32_t depth;         /* calls in flight, 1..16 */
  int32_t device;        /* CUDA ordinal, -1 = current device */
  uint32_t flags;        /* FWD_EB_FLAG_* */
  int32_t external_table;/* 1: no table allocation; fwd_eb_session_adopt_table supplies it */
} fwd_eb_session_config;

int fwd_eb_session_create(const fwd_eb_session_config* cfg, fwd_eb_session** out);
void fwd_eb_session_destroy(fwd_eb_session* s);

/* Copy `rows` host rows into the device table starting at local row
 * `first_row` (blocking, like the reference's configurePlugin upload). */
int fwd_eb_session_load_table(fwd_eb_session* s, const void* h_rows, int64_t first_row,
                              int64_t rows);

/* Device address of the table (to fill it in place, e.g. fwd_eb_fill_table). */
void* fwd_eb_session_device_table(fwd_eb_session* s);

/* Use caller-owned device memory as the table (external_table sessions). */
int fwd_eb_session_adopt_table(fwd_eb_session* s, void* d_table);

/* Pinned host buffers of slot `slot` (0 <= slot < depth): write indices /
 * offsets / weights there, read the result from *h_out after wait. Any of the
 * out-pointers may be NULL. */
int fwd_eb_session_slot(fwd_eb_session* s, int32_t slot, void** h_indices, void** h_offsets,
                        float** h_weights, void** h_out);

/* Queue one call on slot `slot`: host-to-device copy of its inputs, the
 * pooling kernel, device-to-host copy of the result.  Returns at once.
 * A slot's offsets, indices and weights live in one pinned block so that they
 * normally go up as a single copy (areas less than 1 MiB apart are merged,
 * the unused bytes between them included). */
int fwd_eb_session_submit(fwd_eb_session* s, int32_t slot, int64_t num_indices, int64_t num_bags);

/* Block until slot `slot`'s result is in its h_out. */
int fwd_eb_session_wait(fwd_eb_session* s, int32_t slot);

/* One blocking call with arbitrary host pointers (staged through slot 0). */
int fwd_eb_session_run(fwd_eb_session* s, const void* h_indices, int64_t num_indices,
                       const void* h_offsets, int64_t num_bags, const float* h_weights,
                       void* h_out);

/* Bytes moved per submit for the sizes given: host-to-device (bytes between
 * merged areas included) and device-to-host. */
int fwd_eb_session_copy_bytes(fwd_eb_session* s, int64_t num_indices, int64_t num_bags,
                              int64_t* h2d, int64_t* d2h);

#ifdef __cplusplus
}
#endif
#endif /* FWD_EB_SESSION_H_ */
