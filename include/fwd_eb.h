/*
 * fwd_eb.h — C ABI of the B200 (sm_100a) EmbeddingBag gather-and-pool kernels.
 *
 * This is the boundary a host binds to: plain pointers and sizes, no C++ or
 * torch types.  The TensorRT plugin (EmbeddingBag_TRT), the host session and
 * the Python ctypes binding all call these entry points and nothing else.
 *
 * Reference interfaces replaced (paths inside the Tencent/Forward tree):
 *   source/trt_engine/trt_network_crt/plugins/embedding_bag_plugin/
 *     embedding_bag_plugin.h:40-49   free launchers Gather /
 *                                    EmbeddingBagWithFixedOffset / EmbeddingBag
 *     embedding_bag_plugin.cu:66-206 the three kernels and their launch code
 *     embedding_bag_plugin.h:39      enum ReduceOperation (mode codes below)
 *
 * Conventions
 *   - every pointer named `d_*` or documented "device" is device memory of the
 *     current CUDA device; `stream` is a cudaStream_t passed as void*;
 *   - launchers never allocate, never synchronise and launch only on `stream`;
 *   - return value 0 = success, negative = FWD_EB_E* (bad arguments, checked on
 *     the host before any launch), positive = a cudaError_t from the launch;
 *   - nothing aborts the process; fwd_eb_last_error_string() describes the
 *     last failure of the calling thread.
 */
#ifndef FWD_EB_H_
#define FWD_EB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FWD_EB_ABI_VERSION 1

/* Pooling modes: the values of the reference enum ReduceOperation
 * (embedding_bag_plugin.h:39), which are also torch's `mode` integers for
 * sum / mean / max. */
enum {
  FWD_EB_MODE_SUM = 0,
  FWD_EB_MODE_MEAN = 1,
  FWD_EB_MODE_MAX = 2,
  FWD_EB_MODE_SQUARE_SUM = 3,
  FWD_EB_MODE_GATHER = 999
};

enum { FWD_EB_F32 = 0, FWD_EB_F16 = 1 };  /* table / output element type   */
/* Output type for MODE_MAX only (and wire type of a sharded max): per column the pair
 * {fp32 value, int32 position inside the bag of the index that supplied it}, 8 bytes;
 * {0, FWD_EB_NO_POS} where no row of the bag lies inside the table window.  What a row shard
 * must send for the owner to apply torch's first-of-equals rule across shards. */
enum { FWD_EB_F32_POS = 2 };
#define FWD_EB_NO_POS 0x7fffffff
enum { FWD_EB_I32 = 0, FWD_EB_I64 = 1 };  /* indices / offsets element type */

/* Pooling strategies (fwd_eb_params.strategy). AUTO picks by shape. */
enum {
  FWD_EB_STRATEGY_AUTO = 0,
  FWD_EB_STRATEGY_GROUP = 1, /* a sub-warp lane group (16 B per lane) per bag    */
  FWD_EB_STRATEGY_CTA = 2,   /* one CTA per bag, lane groups split the bag       */
  FWD_EB_STRATEGY_SPLIT = 3, /* several CTAs per bag + partials in `workspace`   */
  /* a lane group streams a run of consecutive bags: indices one block ahead in a
   * shared-memory ring, a rolling queue of row loads that bag boundaries do not
   * interrupt.  Rows of 128..512 bytes on the 16-byte vector path, int32 indices,
   * fewer than 2^31 of them; a call outside those limits returns
   * FWD_EB_EUNSUPPORTED when STREAM is asked for by name. */
  FWD_EB_STRATEGY_STREAM = 4,
  /* a lane group per bag with the least per-bag work: blocks of one index per lane, no
   * survivor ring, passes of 4 to 7 row loads.  Same shapes as STREAM; what AUTO runs on them
   * (unless the call is a row window above row 0 whose indices were not compacted). */
  FWD_EB_STRATEGY_LITE = 5
};

/* Flags (fwd_eb_params.flags). */
enum {
  /* mean divides by the raw bag length, as embedding_bag_plugin.cu:112 does;
   * default (flag clear) divides by the number of non-padding indices, as
   * torch does.  Identical when padding_idx < 0. */
  FWD_EB_FLAG_MEAN_RAW_LENGTH = 1,
  /* GATHER leaves rows whose index falls outside the table window untouched,
   * as embedding_bag_plugin.cu:177-179 does; default writes zeros there. */
  FWD_EB_FLAG_GATHER_KEEP_SKIPPED = 2,
  /* fp16 mean rounds the fp32 sum once after the division; default mimics
   * torch CPU (round the sum to fp16, divide, round again). */
  FWD_EB_FLAG_MEAN_SINGLE_ROUNDING = 4,
  /* `offsets` holds a {start, end} pair per bag ([num_bags][2], the indices' type)
   * instead of one start per bag: bags need not be back to back in `indices`.
   * This is what fwd_eb_compact_window writes.  fixed_len must be 0;
   * include_last_offset is ignored. */
  FWD_EB_FLAG_OFFSET_PAIRS = 8,
  /* with OFFSET_PAIRS: inside every aligned run of 16 bags (bags 16k .. 16k+15) each
   * bag starts where the previous one ends, as fwd_eb_compact_window lays them
   * out; lets the STREAM strategy walk several bags as one index stream. */
  FWD_EB_FLAG_PAIRS_RUN16 = 16
};

/* Error codes. */
enum {
  FWD_EB_OK = 0,
  FWD_EB_EINVAL = -1,      /* null pointer / negative size / unknown enum      */
  FWD_EB_EUNSUPPORTED = -2,/* legal but not implemented combination            */
  FWD_EB_EALIGN = -3,      /* pointer or stride not aligned as required        */
  FWD_EB_EWORKSPACE = -4,  /* strategy needs more workspace than was given     */
  FWD_EB_ENOGPU = -5,      /* no usable CUDA device                            */
  FWD_EB_ETOOBIG = -6      /* size beyond a documented fixed limit             */
};

/*
 * One gather-and-pool call.  Zero-initialise, then fill.
 *
 * Bags: with `fixed_len` > 0 the indices form a [num_bags, fixed_len] matrix
 * (reference EmbeddingBagCudaWithFixedOffset, embedding_bag_plugin.cu:120-168)
 * and `offsets` is ignored; otherwise bag b covers
 * indices[offsets[b] .. offsets[b+1]) and the last bag ends at `num_indices`
 * (embedding_bag_plugin.cu:80-86) unless `include_last_offset` is set, in which
 * case `offsets` holds num_bags+1 entries.
 *
 * Table window: the device table holds rows [row_lo, row_lo + num_rows) of the
 * logical table; an index outside the window is skipped silently
 * (reference `data_offset` / `count`, embedding_bag_plugin.cu:94).  This is
 * the row-shard filter.
 */
typedef struct fwd_eb_params {
  const void* table;        /* device, row-major [num_rows, dim], 16 B aligned for the fast path */
  int32_t table_dtype;      /* FWD_EB_F32 / FWD_EB_F16 */
  int32_t dim;              /* columns per row (> 0) */
  int64_t num_rows;         /* rows held on this device */
  int64_t row_lo;           /* logical id of local row 0 */
  int64_t table_stride;     /* elements between rows; 0 = dim */

  const void* indices;      /* device, [num_indices] */
  const void* offsets;      /* device, [num_bags] (+1 with include_last_offset); NULL iff fixed_len > 0 */
  int32_t index_dtype;      /* FWD_EB_I32 / FWD_EB_I64, for indices and offsets */
  int32_t fixed_len;        /* > 0: every bag has this many indices */
  int64_t num_indices;
  int64_t num_bags;

  const float* per_sample_weights; /* device fp32 [num_indices] or NULL; SUM only */
  int32_t mode;             /* FWD_EB_MODE_* */
  int32_t include_last_offset;
  int64_t padding_idx;      /* logical index to skip; < 0 = none */

  void* out;                /* device, [num_bags, dim] (GATHER: [num_indices, dim]) */
  int32_t out_dtype;        /* FWD_EB_F32 / FWD_EB_F16 (MODE_MAX also FWD_EB_F32_POS) */
  int32_t strategy;         /* FWD_EB_STRATEGY_* */
  int64_t out_stride;       /* elements between output rows; 0 = dim */

  void* workspace;          /* device scratch for FWD_EB_STRATEGY_SPLIT, or NULL */
  size_t workspace_bytes;
  uint32_t flags;           /* FWD_EB_FLAG_* */
  int32_t reserved;
} fwd_eb_params;

/* ABI version of the loaded library (FWD_EB_ABI_VERSION). */
int fwd_eb_version(void);

/* sizeof(fwd_eb_params) as the library was compiled: lets a foreign-language
 * binding check its own mirror of the struct. */
size_t fwd_eb_params_size(void);

/* Text for the calling thread's last non-zero return value ("" if none). */
const char* fwd_eb_last_error_string(void);

/* General entry point: validates `p`, picks a strategy, launches on `stream`.
 * Replaces the dispatch in EmbeddingBagPlugin::enqueue
 * (embedding_bag_plugin.cpp:146-189) plus the launchers it calls. */
int fwd_eb_forward(const fwd_eb_params* p, void* stream);

/* Several independent calls at once (the tables of one model; the reference enqueues one
 * plugin per table, one after the other, embedding_bag_plugin.cpp:146-189).  The result is that of
 * fwd_eb_forward on each in turn on `stream`; the launches are spread over `stream` and
 * FWD_EB_MANY_STREAMS auxiliary streams the library keeps per GPU (created on first use), forked
 * from `stream` and joined back into it, because a table's grid is often only a wave or two and
 * its ramp and tail are time another table's grid can use (26 tables of 65536 x 20 lookups on a
 * B200: 1218 us one after the other, 1139 us spread).  The calls must be independent: no call's
 * output may be another call's input or output.  Every call is validated before the first
 * launch; calls of different host threads on one GPU are serialised on the host.  The auxiliary
 * streams live until the process ends (like the static scratch they do not survive a
 * cudaDeviceReset()). */
#define FWD_EB_MANY_STREAMS 2
int fwd_eb_forward_many(const fwd_eb_params* const* params, int32_t count, void* stream);

/* Scratch bytes fwd_eb_forward needs for `p` (0 unless the SPLIT strategy is
 * requested or AUTO would choose it when scratch is offered).  The reference
 * plugin reports 0 (embedding_bag_plugin.cpp:129-133). */
size_t fwd_eb_workspace_size(const fwd_eb_params* p);

/*
 * Split-bag pooling for callers that may not allocate device memory.  It has no
 * counterpart in the reference (whose plugin asks TensorRT for no workspace,
 * embedding_bag_plugin.cpp:129-133, and so can never split a long bag).
 *
 * Who needs it: a plugin or serving loop that was given its buffers up front
 * and must not call cudaMalloc afterwards — for example a TensorRT plugin that
 * reported getWorkspaceSize() == 0 and therefore receives no workspace in
 * enqueue(), or a host whose memory pool is frozen once serving starts.
 *
 * Same arguments and results as fwd_eb_forward with
 * strategy = FWD_EB_STRATEGY_SPLIT, except that `workspace`, `workspace_bytes`
 * and `strategy` in `p` are ignored: the partial sums of the split bags go to
 * an array of FWD_EB_STATIC_SCRATCH_BYTES built into the library's device
 * image (every GPU that loads the library holds that much until the process
 * exits).  The call allocates nothing and frees nothing.
 *
 *   - A call whose split needs more than FWD_EB_STATIC_SCRATCH_BYTES
 *     (fwd_eb_workspace_size with strategy SPLIT tells) returns
 *     FWD_EB_ETOOBIG before anything is launched.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current) and caches it; make that
 *     first call before starting any stream capture.
 *   - All calls on a device share the one array and it keeps the previous
 *     call's contents.  Nothing has to be cleared between calls — every slot a
 *     call reads it has written first — but two calls that overlap on the GPU
 *     (different streams, no dependency) would overwrite each other's
 *     partials: keep calls to this entry point ordered on one stream, or
 *     serialise them with events.
 *   - The cached address belongs to the device's current primary context.  A host
 *     that calls cudaDeviceReset() invalidates it (and every other device pointer
 *     it holds); this entry point must not be used across such a reset.
 */
#define FWD_EB_STATIC_SCRATCH_BYTES (8u << 20)
int fwd_eb_forward_static_scratch(const fwd_eb_params* p, void* stream);

/* Do fwd_eb_forward_static_scratch's one-time set-up for the current device now (look up and
 * cache the array's device address), so that the first real call can come at any time — inside
 * a stream capture, for instance.  Launches nothing and allocates nothing; 0 on success.  No
 * counterpart in the reference. */
int fwd_eb_static_scratch_prepare(void);

/*
 * Window compaction: run the table-window / padding filter of `p` once, as a
 * streaming pass, instead of inside the pooling loop.  The reference tests every
 * index of every bag against `data_offset` / `count` in its bag loop
 * (embedding_bag_plugin.cu:94); for a rank that holds one of G row windows of a
 * sharded table that is G times more index traffic and G times more loop
 * iterations than rows it will gather.
 *
 * Reads p->indices / offsets / fixed_len / include_last_offset / num_bags /
 * num_indices / row_lo / num_rows / padding_idx / per_sample_weights (other fields
 * are ignored) and writes
 *   d_kept    int32 [num_indices]  the surviving indices as LOCAL row numbers
 *             (index - row_lo), in bag order; the survivors of bags 16k..16k+15 are
 *             back to back starting at the position where bag 16k starts in
 *             p->indices (entries past a run's survivors are left untouched);
 *   d_kept_weights fp32 [num_indices], the survivors' weights (NULL unless
 *             p->per_sample_weights is set);
 *   d_bounds  int32 [num_bags][2]  {start, end} of every bag's survivors in d_kept;
 *   d_counts  int32 [num_bags] or NULL: non-padding entries of the WHOLE bag, inside
 *             the window or not (the divisor of a sharded mean).
 * Pool the result with indices = d_kept, index_dtype = FWD_EB_I32, offsets =
 * d_bounds, flags |= FWD_EB_FLAG_OFFSET_PAIRS | FWD_EB_FLAG_PAIRS_RUN16, row_lo = 0,
 * padding_idx = -1 and per_sample_weights = d_kept_weights: every index then passes
 * the filter and the pooling kernels take their dense path.  num_indices must be
 * below 2^31.  Launches one kernel on `stream`; allocates nothing.
 */
int fwd_eb_compact_window(const fwd_eb_params* p, int32_t* d_kept, float* d_kept_weights,
                          int32_t* d_bounds, int32_t* d_counts, void* stream);

/* Which strategy AUTO resolves to for `p` (a FWD_EB_STRATEGY_* value, or a
 * negative error).  `p->workspace_bytes` decides whether SPLIT is on offer. */
int fwd_eb_pick_strategy(const fwd_eb_params* p);

/* Number of kernels launched by this library in the calling process so far. */
uint64_t fwd_eb_launch_count(void);

/*
 * Source-compatible forms of the reference's three launchers
 * (embedding_bag_plugin.h:40-49): fp32 table, int32 indices, fp32 output,
 * 32-bit sizes.  `op_type` is a FWD_EB_MODE_* value.
 */
/* Gather(input, output, batch_size, offset, data, count, dim, data_offset, stream)
 * — embedding_bag_plugin.cu:182-188.  Rows are addressed relative to
 * data_offset (the reference kernel forgot to subtract it, .cu:178). */
int fwd_eb_gather_f32(const int* d_input, float* d_output, int batch_size, int offset,
                      const float* d_data, int count, int dim, int data_offset, void* stream);

/* EmbeddingBagWithFixedOffset(...) — embedding_bag_plugin.cu:190-196. */
int fwd_eb_bag_fixed_f32(const int* d_input, float* d_output, int batch_size, int offset,
                         const float* d_data, int count, int dim, int data_offset, int op_type,
                         void* stream);

/* EmbeddingBag(input, input_2, output, input_size, block_size, ...) —
 * embedding_bag_plugin.cu:198-206; block_size is the number of bags. */
int fwd_eb_bag_f32(const int* d_input, const int* d_offsets, float* d_output, int input_size,
                   int block_size, const float* d_data, int count, int dim, int data_offset,
                   int op_type, void* stream);

/* ---- helpers for tables too large to stage through the host ---------------- */

/*
 * Fill rows [row_lo, row_lo+num_rows) of a logical table in place on the
 * device with the counter-based generator  value(seed,row,col) = scale * z,
 * z = the centred sum of eight 16-bit uniforms drawn from a 64-bit mix of
 * (seed,row,col), scaled to unit variance (an Irwin-Hall bell: integer
 * arithmetic and one multiplication, so host and device give the same bits).
 * A host twin lives in the test oracle so a CPU check can regenerate only the
 * rows a sampled bag touches.
 */
int fwd_eb_fill_table(void* d_table, int32_t table_dtype, int64_t num_rows, int32_t dim,
                      int64_t row_lo, uint64_t seed, float scale, void* stream);

/* d_dst[i] = (int32) d_src[i] for `count` int64 values: the cast Forward's engine applies to
 * int64 index tensors on their way in (TorchEngine::ParseInput,
 * source/fwd_torch/torch_engine/torch_engine.cpp:134-149).  Values outside the int32 range map
 * to -1, which no table window contains, instead of wrapping. */
int fwd_eb_cast_i64_to_i32(const void* d_src, void* d_dst, int64_t count, void* stream);

/* out[i] = sum over r < num_parts of parts[r][i] (fp32 or fp16 wire, fp32 math,
 * added in r order), optionally cast to `out_dtype`.  Used after a row-shard
 * exchange where each peer's partial lands in its own slot. */
int fwd_eb_combine_partials(const void* d_parts, int32_t part_dtype, int32_t num_parts,
                            int64_t part_stride_elems, int64_t count, void* d_out,
                            int32_t out_dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FWD_EB_H_ */
