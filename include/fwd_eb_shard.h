/*
 * fwd_eb_shard.h — row-sharded EmbeddingBag: pool the rows this GPU owns and hand
 * the partial bags to their owners over NVLink, in the same kernel (C ABI).
 *
 * The reference has no multi-GPU code; its only hook is the plugin's row window
 * (`data_offset_` / `count_`, "reserved for a possible multi-machine search",
 * source/trt_engine/trt_network_crt/plugins/embedding_bag_plugin/
 * embedding_bag_plugin.h:121-124, honoured at embedding_bag_plugin.cu:94).  This
 * header extends that seam: G ranks each hold a row window of one logical table,
 * every rank scans the whole batch, and bag b's pooled value is the sum of the G
 * partial bags.
 *
 * Exchange layout.  Bags are owned in contiguous runs of `bags_per_rank`: rank o
 * owns bags [o*bags_per_rank, (o+1)*bags_per_rank).  Each rank exposes a receive
 * buffer of FWD_EB_SHARD_BUFFERS x G x bags_per_rank x dim elements (parts used in turn, call
 * number modulo FWD_EB_SHARD_BUFFERS, one slot per source rank) and G flag words, all mapped into every
 * peer (CUDA IPC below, or any other peer mapping).  fwd_eb_shard_push pools, and
 * writes bag b's partial row straight into slot [part][rank] of b's owner with
 * plain peer stores.  fwd_eb_shard_combine, queued behind it on the same stream,
 * first publishes `epoch` in every peer's flag word (the pooling grid has
 * completed by then, so its peer stores have been performed), then waits
 * (bounded) until all G flags have reached `epoch` and folds the G slots in rank
 * order — a fixed order, so results do not depend on timing.  No multicast
 * loads, no library kernels on peer memory.
 *
 * Every wait is bounded: after `max_spins` polls the waiting kernel writes
 * FWD_EB_SHARD_TIMEOUT to `status` and returns without touching the output.
 */
#ifndef FWD_EB_SHARD_H_
#define FWD_EB_SHARD_H_

#include "fwd_eb.h"

#ifdef __cplusplus
extern "C" {
#endif

#define FWD_EB_MAX_PEERS 16
/* Parts of a receive buffer, used in turn (call number modulo FWD_EB_SHARD_BUFFERS), and how
 * often and how far the pipeline makes a rank look back.  Only on every k-th call does the main
 * stream wait, and then for this rank's fold of call e-d (which implies it has seen every rank's
 * flag e-d); the calls in between are queued without a wait on another stream.  Waiting on every
 * call for call e-2 cost 4 us of a 29 us step on two B200s.
 *   - Flag raised by the kernel behind the pooling grid, after this rank has folded the call
 *     before (the default): seeing flag f of rank A proves A has folded f-1; a rank B writing
 *     call g has seen flags >= g-(k-1)-d, so the part it overwrites must be older than that:
 *     k + d parts.  Default k = 6, d = 2 (fwd_eb_pipeline_set_lookback changes them).
 *   - Flag raised by the pooling grid itself (x->tickets set): a flag no longer proves a fold;
 *     seeing flag f of A only proves A had folded f-(k-1)-d, hence 2(k-1) + 2d parts.
 *     k = 3, d = 2.
 * The caller may issue consecutive steps on different streams (independent batches: one step's
 * grid then runs beside the tail of the step before).  The look-back is kept per caller stream
 * (up to FWD_EB_PIPELINE_MAIN_STREAMS of them; a stream beyond that waits on every call): a
 * step waits, on its own stream, unless that stream is already behind this rank's fold of some
 * call >= e-(k-1)-d, which is all the argument above uses.  Flags, waits and folds stay in call
 * order on the pipeline's side stream whatever stream a step came in on.  A pipeline is driven
 * by one host thread, and a caller stream it has seen must stay alive (its handle must not be
 * reused for another stream) while the pipeline is in use.
 * The CPU model of these rules (tests/test_exchange_protocol.py) finds no overwrite of an
 * unfolded part with them and does find one with fewer parts. */
#define FWD_EB_PIPELINE_WAIT_EVERY 6
#define FWD_EB_PIPELINE_WAIT_DEPTH 2
#define FWD_EB_PIPELINE_WAIT_EVERY_TICKETS 3
#define FWD_EB_SHARD_BUFFERS 16
#define FWD_EB_PIPELINE_MAIN_STREAMS 4    /* distinct caller streams a pipeline keeps look-back state for */
#define FWD_EB_PIPELINE_LOCAL_STREAMS 2   /* auxiliary streams for a hybrid step's replicated tables */
#define FWD_EB_SHARD_TIMEOUT 1
#define FWD_EB_IPC_HANDLE_BYTES 64

/* Receive-buffer layouts (fwd_eb_shard_exchange.layout). */
enum {
  /* Row shards of one table: [parts][G source ranks][bags_per_rank][dim];
   * the owner folds the G slots with fwd_eb_shard_combine. */
  FWD_EB_LAYOUT_ROW_SHARD = 0,
  /* Whole tables placed on different ranks: [parts][bags_per_rank][num_tables][dim];
   * the rank holding table t pools the whole batch and writes column block
   * `table_index` of every owner's buffer.  Nothing is folded: after
   * fwd_eb_shard_wait that part of the buffer IS the result (the all-to-all of pooled
   * outputs, done by the pooling kernels' own stores). */
  FWD_EB_LAYOUT_TABLE_WISE = 1
};

typedef struct fwd_eb_shard_exchange {
  int32_t world;              /* G, 1..FWD_EB_MAX_PEERS */
  int32_t rank;
  int64_t bags_per_rank;      /* owner of bag b is b / bags_per_rank */
  int32_t wire_dtype;         /* FWD_EB_F32, or FWD_EB_F16 to halve the NVLink bytes; a sharded
                                 MAX uses FWD_EB_F32_POS ({value, position}, 8 bytes a column) */
  uint32_t epoch;             /* call number, starting at 1; epoch % FWD_EB_SHARD_BUFFERS picks the part */
  void* peer_slots[FWD_EB_MAX_PEERS];      /* rank r's receive buffer as mapped here */
  uint32_t* peer_flags[FWD_EB_MAX_PEERS];  /* rank r's G flag words as mapped here */
  int32_t* status;            /* one device word of this rank; 0 = fine */
  int64_t max_spins;          /* bound of the flag wait; 0 = default (about a second) */
  int32_t layout;             /* FWD_EB_LAYOUT_* */
  int32_t num_tables;         /* TABLE_WISE: tables in the whole model */
  int32_t table_index;        /* TABLE_WISE: which of them this call pools */
  /* 1: fwd_eb_shard_push raises this rank's flag itself when its grid completes (the last CTA
   * to finish, found with a ticket counter, publishes `epoch` after a system-scope fence), and
   * the wait / fold that follows only waits.  0: the flag is raised by the kernel that follows
   * the push on the stream (fwd_eb_shard_combine / _wait / _signal).  The pipeline sets it. */
  int32_t raise_from_push;
  /* this rank's own device memory: FWD_EB_SHARD_BUFFERS words, zero-initialised once; needed
   * when raise_from_push is used (NULL otherwise) */
  uint32_t* tickets;
  /* Shipping instead of pushing.  NULL: the pooling kernel stores its rows into the peers'
   * buffers itself.  Otherwise local scratch of fwd_eb_shard_stage_bytes() bytes: the pooling
   * kernel writes every row into it ([parts][world][bags_per_rank][stage_tables][dim], wire
   * type) and fwd_eb_shard_ship, a small copy kernel on the side stream, sends each owner its
   * rows with 16-byte peer stores.  A pooling warp cannot exit before its stores have been
   * acknowledged; with seven of eight rows going over NVLink that wait costs a quarter of the
   * pooling step, while local stores cost nothing and the copy runs beside the next step. */
  void* stage;
  int32_t stage_tables;       /* TABLE_WISE: tables this rank pools in a step (1 for row shards) */
  int32_t stage_slot;         /* TABLE_WISE: which of them this call pools, 0..stage_tables-1 */
} fwd_eb_shard_exchange;

/* Bytes of one rank's receive buffer: row-shard layout for `world` sources, or, with
 * num_tables > 0, table-wise layout. */
size_t fwd_eb_shard_slots_bytes(int32_t world, int64_t bags_per_rank, int32_t dim,
                                int32_t wire_dtype);
size_t fwd_eb_shard_tablewise_bytes(int64_t bags_per_rank, int32_t num_tables, int32_t dim,
                                    int32_t wire_dtype);

/* Bytes of the staging scratch (fwd_eb_shard_exchange.stage); stage_tables = 1 for row shards. */
size_t fwd_eb_shard_stage_bytes(int32_t world, int64_t bags_per_rank, int32_t stage_tables,
                                int32_t dim, int32_t wire_dtype);

/* Send what this call's fwd_eb_shard_push(es) left in x->stage to the owners' buffers: one copy
 * kernel on `stream` (which must be ordered behind the pushes), plain 16-byte stores, owners
 * interleaved.  `num_bags` is the batch size; table_ids[j] (TABLE_WISE, stage_tables entries) is
 * the table whose rows sit in staged slot j.  The flag is raised by the kernel that follows
 * (fwd_eb_shard_combine / _wait).  No multicast, no library kernel on peer memory. */
int fwd_eb_shard_ship(const fwd_eb_shard_exchange* x, int32_t dim, int64_t num_bags,
                      const int32_t* table_ids, void* stream);

/* Pool the local row window of `p` (modes SUM or MEAN, optional weights) and push
 * each bag's partial row to its owner; `p->out` is ignored.  MEAN partials are
 * already divided by the bag's full count, so the owner only adds. */
int fwd_eb_shard_push(const fwd_eb_params* p, const fwd_eb_shard_exchange* x, void* stream);

/* Raise this rank's flag everywhere, wait for all peers' flags, then
 * out[b, :] = sum over r of slot[r][b, :] for the `num_bags` bags this rank owns.
 * Must follow this call's fwd_eb_shard_push on the same stream. */
int fwd_eb_shard_combine(const fwd_eb_shard_exchange* x, int32_t dim, int64_t num_bags,
                         void* d_out, int32_t out_dtype, void* stream);

/* fwd_eb_shard_combine followed by out[b, :] /= max(1, d_counts[b]): for a sharded MEAN whose
 * partials are plain sums (d_counts: int32, one entry per bag this rank owns; NULL = no division,
 * i.e. fwd_eb_shard_combine). */
int fwd_eb_shard_combine_div(const fwd_eb_shard_exchange* x, int32_t dim, int64_t num_bags,
                             const int32_t* d_counts, void* d_out, int32_t out_dtype, void* stream);

/* ROW_SHARD, the copy-engine alternative to fwd_eb_shard_push: `d_stage` holds the partial
 * bags of ALL `num_bags` bags, [num_bags, dim] in the wire dtype, as fwd_eb_forward with this
 * rank's row window (and FWD_EB_FLAG_MEAN_SINGLE_ROUNDING for MEAN) wrote them; each owner's
 * block of rows is sent to slot [part][rank] of that owner with one cudaMemcpyAsync on
 * `stream` (peers first, this rank's own block last).  fwd_eb_shard_combine then follows on
 * the same stream exactly as after a push. */
int fwd_eb_shard_send_staged(const fwd_eb_shard_exchange* x, int32_t dim, int64_t num_bags,
                             const void* d_stage, void* stream);

/* TABLE_WISE: after the last fwd_eb_shard_push of this call on the same stream: raise
 * this rank's flag, wait (bounded) until every rank has raised `epoch`; on success
 * *d_result (if not NULL) receives the address of this call's buffer part, laid out
 * [num_bags owned][num_tables][dim]. */
int fwd_eb_shard_wait(const fwd_eb_shard_exchange* x, int32_t dim, void** d_result, void* stream);

/* Publish `epoch` to every peer without pooling or waiting (tests; a rank that leaves a
 * call early). */
int fwd_eb_shard_signal(const fwd_eb_shard_exchange* x, void* stream);

/* ---- one call = one step: the stream / event choreography in native code ---------
 *
 * A pipeline owns a high-priority side stream and the events that order a step:
 *   main stream   [wait: exchange of step e-2 done]  pooling + push of step e
 *   side stream   [wait: push of step e issued]      flag exchange (+ fold) of step e
 * so the pooling of step e overlaps the flag exchange and fold of step e-1 (see
 * FWD_EB_SHARD_BUFFERS for why that is safe), and a step costs the host one call.  With
 * x->tickets set, the fused-push steps let the pooling grid raise the flag itself (its last
 * CTA, found with a ticket counter): the main stream then carries nothing but pooling grids and
 * the side stream's kernel only waits.  Measured slower on B200 (the per-CTA fence that must
 * precede the ticket: 33.3 against 25.3 us per table-wise step on two GPUs), so the Python layer
 * leaves tickets unset; the path is kept and tested.
 * It keeps the call number itself (x->epoch is overwritten).  Results complete on the side
 * stream: queue consumers there (fwd_eb_pipeline_side_stream) or call
 * fwd_eb_pipeline_sync_result on the stream that will read them; consume a result before
 * the next step is issued. */
typedef struct fwd_eb_pipeline fwd_eb_pipeline;

int fwd_eb_pipeline_create(fwd_eb_pipeline** out);
void fwd_eb_pipeline_destroy(fwd_eb_pipeline* pl);
void* fwd_eb_pipeline_side_stream(fwd_eb_pipeline* pl);
/* Look back on every `every`-th step, for the fold of step e - `depth` (see FWD_EB_SHARD_BUFFERS;
 * every >= 1, depth >= 2, every + depth <= FWD_EB_SHARD_BUFFERS).  Every rank must use the same
 * values; set them before the first step. */
int fwd_eb_pipeline_set_lookback(fwd_eb_pipeline* pl, int32_t every, int32_t depth);

/* Row shards: push `p` on `main_stream`, fold on the side stream into
 * d_out[epoch % FWD_EB_SHARD_BUFFERS] (caller buffers of [bags_per_rank, dim]); *which receives that
 * number. */
int fwd_eb_pipeline_step_rowshard(fwd_eb_pipeline* pl, const fwd_eb_params* p,
                                  fwd_eb_shard_exchange* x, int64_t num_bags_owned,
                                  void* const d_out[FWD_EB_SHARD_BUFFERS], int32_t out_dtype,
                                  void* main_stream, int32_t* which);

/* Row shards, exchange by the copy engines instead of by the pooling kernel's own stores: the
 * plain pooling kernel writes every bag's partial into d_stage[epoch % FWD_EB_SHARD_BUFFERS] (local buffers of
 * [world * bags_per_rank, dim] in the wire dtype) on `main_stream`; the side stream then sends
 * each owner its block with one cudaMemcpyAsync over NVLink, raises the flags, waits (bounded)
 * and folds as above.  All of the exchange runs beside the next step's pooling and takes no SM
 * time from it; a result is complete a copy later than with the fused push.
 * This is also how MODE_MAX is sharded (x->wire_dtype = FWD_EB_F32_POS): each rank's partial is
 * the {value, position} pair of fwd_eb_forward's FWD_EB_F32_POS output, and the fold keeps the
 * greater value, the earlier position among equal values, and a NaN only where it was the
 * bag's first entry — bit for bit what torch's max gives on the unsharded table. */
int fwd_eb_pipeline_step_rowshard_staged(fwd_eb_pipeline* pl, const fwd_eb_params* p,
                                         fwd_eb_shard_exchange* x, int64_t num_bags_owned,
                                         void* const d_stage[FWD_EB_SHARD_BUFFERS],
                                         void* const d_out[FWD_EB_SHARD_BUFFERS], int32_t out_dtype,
                                         void* main_stream, int32_t* which);

/* Row shards with the window filter taken out of the pooling loop (the fastest row-shard step).
 * The reference tests every index against its row window inside the bag loop
 * (embedding_bag_plugin.cu:94); with G windows that loop reads G times more indices than it
 * gathers rows.  Here, on `main_stream`: (1) fwd_eb_compact_window streams over the batch once
 * and keeps this rank's indices as dense sub-bags; (2) the pooling kernel walks those and pushes
 * each partial row into slot [rank] of the bag's owner; then, on the side stream, (3) flags,
 * bounded wait and fold as in fwd_eb_pipeline_step_rowshard.  Partials of a MEAN are plain sums
 * and the owner divides by the bag's full count after the fold.  `p->out` is ignored.
 * Scratch is the caller's (nothing is allocated): */
typedef struct fwd_eb_compact_scratch {
  int32_t* kept;          /* [max num_indices] */
  float* kept_weights;    /* [max num_indices], or NULL when no per_sample_weights are used */
  int32_t* bounds;        /* [max num_bags][2], 8-byte aligned */
  int32_t* counts;        /* MEAN only: [FWD_EB_SHARD_BUFFERS][world * bags_per_rank], one part per step in flight */
} fwd_eb_compact_scratch;
int fwd_eb_pipeline_step_rowshard_compact(fwd_eb_pipeline* pl, const fwd_eb_params* p,
                                          fwd_eb_shard_exchange* x, int64_t num_bags_owned,
                                          const fwd_eb_compact_scratch* scratch,
                                          void* const d_out[FWD_EB_SHARD_BUFFERS], int32_t out_dtype,
                                          void* main_stream, int32_t* which);

/* Table-wise: push the `count` local tables (x->table_index is set from table_index[i]),
 * then the flag exchange on the side stream; *d_result receives this step's buffer part. */
int fwd_eb_pipeline_step_tablewise(fwd_eb_pipeline* pl, const fwd_eb_params* const* params,
                                   const int32_t* table_index, int32_t count,
                                   fwd_eb_shard_exchange* x, int32_t dim, void* main_stream,
                                   void** d_result);

/* Table-wise with replicated tables.  A table small enough to live on every rank needs no
 * exchange: each rank pools only the bags it owns and stores the rows into its own buffer.
 * fwd_eb_shard_pool_local does that for one table: `p` describes this rank's bags only (bag 0 of
 * `p` is the first bag this rank owns, num_bags <= bags_per_rank), the rows land in column block
 * x->table_index of this rank's buffer part of call x->epoch, written by the single-GPU kernels
 * with local stores; `p->out` is ignored.  The hybrid step queues the pushes of the `count`
 * tables this rank holds alone, then the `local_count` replicated tables, then the flag exchange
 * as fwd_eb_pipeline_step_tablewise does.  Needs x->tickets == NULL when local_count > 0. */
int fwd_eb_shard_pool_local(const fwd_eb_params* p, const fwd_eb_shard_exchange* x, void* stream);
/* A table-wise step's launches (one per table, pushes and replicated tables alike) are
 * independent, so the step spreads them over `main_stream` and up to
 * FWD_EB_PIPELINE_LOCAL_STREAMS streams of the pipeline's own, forked from `main_stream` and
 * joined before the flag exchange; 0 queues everything on `main_stream`.  (With x->tickets the
 * pushes stay on `main_stream`: the last push grid raises the flag.) */
int fwd_eb_pipeline_set_local_streams(fwd_eb_pipeline* pl, int32_t streams);
int fwd_eb_pipeline_step_tablewise_hybrid(fwd_eb_pipeline* pl, const fwd_eb_params* const* params,
                                          const int32_t* table_index, int32_t count,
                                          const fwd_eb_params* const* local_params,
                                          const int32_t* local_table_index, int32_t local_count,
                                          fwd_eb_shard_exchange* x, int32_t dim, void* main_stream,
                                          void** d_result);

/* Make `stream` wait for the last step's result. */
int fwd_eb_pipeline_sync_result(fwd_eb_pipeline* pl, void* stream);
/* Block the host until everything the pipeline queued has run. */
int fwd_eb_pipeline_drain(fwd_eb_pipeline* pl);

/* ---- peer mapping through CUDA IPC (one process per GPU on one node) ---------- */

/* cudaMalloc + zero-fill `bytes` and produce the 64-byte handle peers open. */
int fwd_eb_ipc_alloc(size_t bytes, void** d_ptr, unsigned char handle[FWD_EB_IPC_HANDLE_BYTES]);
/* Map a peer's allocation into this process (peer access enabled lazily). */
int fwd_eb_ipc_open(const unsigned char handle[FWD_EB_IPC_HANDLE_BYTES], void** d_peer_ptr);
int fwd_eb_ipc_close(void* d_peer_ptr);
int fwd_eb_ipc_free(void* d_ptr);

#ifdef __cplusplus
}
#endif
#endif /* FWD_EB_SHARD_H_ */
