// Row-sharded pooling fused with its exchange (include/fwd_eb_shard.h).
//
// The pooling loop is the one every strategy shares (pool_range); what changes is the
// epilogue: instead of a local output row, the lane group stores its partial row into the
// owner rank's receive slot through a peer-mapped pointer, so the NVLink transfer of early
// bags overlaps the HBM gathers of later ones and the partial never makes a round trip
// through local memory.  The kernel that follows on the same stream (the fold, or the bare wait
// of the table-wise layout) starts by raising this rank's flag on every peer — by then the
// pooling grid has completed, so all of its peer stores have been performed — and then waits,
// with a bound, for the peers' flags.
#include <climits>
#include <cstdlib>
#include <cstring>
#include <new>

#include "eb_internal.h"
#include "eb_kernels.cuh"
#include "eb_lite.cuh"
#include "eb_stream.cuh"
#include "fwd_eb_shard.h"

namespace fwd_eb {


__device__ __forceinline__ void store_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Raise this rank's flag on every peer (one thread).  Callers run it at the start of a kernel
// that follows the pooling grid on the same stream.
__device__ __forceinline__ void raise_flags(uint32_t* const* peer_flags, int world, int rank,
                                            uint32_t epoch) {
  __threadfence_system();
  for (int r = 0; r < world; ++r) store_release_sys(peer_flags[r] + rank, epoch);
}

struct FlagSet {
  uint32_t* peer_flags[FWD_EB_MAX_PEERS];
};

template <typename TW, int VE, int CPL, int OP, int U, int IPL>
__global__ void __launch_bounds__(kCtaThreads, FWD_EB_MIN_CTAS)
eb_pool_push_kernel(const PoolArgs a, const PushArgs x) {
  const int lanes_log2 = a.lanes_log2;
  const long long seq = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> lanes_log2;
  const int chunk0 = blockIdx.y * (CPL << lanes_log2);
  const bool live = seq < a.num_bags;
  // The grid starts with the bags of the next rank and ends with this rank's own, so the
  // stores that cross NVLink are issued first and the grid's tail stores locally.
  long long bag = seq + x.first_bag;
  if (bag >= a.num_bags) bag -= a.num_bags;
  // programmatic dependent launch, as in eb_pool_group_kernel
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  long long start = 0, end = 0;
  if (live) bag_bounds(a, bag, start, end);

  Accum<CPL, VE> s;
  clear(s);
  pool_range<TW, VE, CPL, OP, U, IPL>(a, start, end, chunk0, s);

  const bool tf16 = sizeof(TW) == 2;
#pragma unroll
  for (int c = 0; c < CPL; ++c)
#pragma unroll
    for (int e = 0; e < VE; ++e) s.v[c][e] = finish(a, s.v[c][e], s.counted, end - start, tf16);
  // bag / bags_per_rank: 32-bit when it fits (a 64-bit division is some hundred instructions)
  long long owner = 0;
  if (live)
    owner = x.small ? (long long)((unsigned)bag / (unsigned)x.bags_per_rank) : bag / x.bags_per_rank;
  if (owner >= x.world) owner = x.world - 1;
  const long long local_bag = bag - owner * x.bags_per_rank;
  // this rank's slot (row shards) or this table's column block (table-wise) at the owner
  char* base = x.peer_slots[owner] + x.col_offset * (a.out_f16 ? 2 : 4);
  store_row<VE, CPL, true>(a, base, x.row_base + local_bag, chunk0, s.v, live);
  push_grid_done(x);
}

// Fold of a sharded MAX: slot r holds, per column of each bag, {value, position of the index
// that supplied it} or {0, kNoPos} when rank r had no row of the bag.  The greater value wins;
// among equal values (+0.0 / -0.0) the earlier position; a NaN partial exists only when the
// NaN was the bag's first non-padding entry, and then it is the result (the sequential rule of
// eb_pool_maxpos_kernel).  A bag without any row gives 0.
template <typename TO>
__global__ void __launch_bounds__(kCtaThreads)
eb_shard_combine_max_kernel(const int2* slots, int world, long long slot_stride, long long count,
                            TO* out, const int* status) {
  if (*static_cast<const volatile int*>(status) != 0) return;
  for (long long i = (long long)blockIdx.x * kCtaThreads + threadIdx.x; i < count;
       i += (long long)gridDim.x * kCtaThreads) {
    float best = 0.0f;
    int best_pos = kNoPos;
    for (int r = 0; r < world; ++r) {
      const int2 pr = slots[r * slot_stride + i];
      const float v = __int_as_float(pr.x);
      const int pos = pr.y;
      if (pos == kNoPos) continue;
      bool take;
      if (best_pos == kNoPos) take = true;
      else if (best != best) take = false;          // a NaN that was the bag's first entry stays
      else if (v != v) take = true;
      else take = v > best || (v == best && pos < best_pos);
      if (take) {
        best = v;
        best_pos = pos;
      }
    }
    if (sizeof(TO) == 2) out[i] = (TO)__float2half_rn(best);
    else out[i] = (TO)best;
  }
}

__global__ void eb_shard_signal_kernel(const FlagSet f, int world, int rank, uint32_t epoch) {
  if (threadIdx.x == 0 && blockIdx.x == 0) raise_flags(f.peer_flags, world, rank, epoch);
}

// Bounded wait for all flags; nothing else (table-wise layout needs no folding).
__global__ void eb_shard_wait_kernel(const FlagSet f, int rank, int world, uint32_t epoch,
                                     int* status, long long max_spins, int raise) {
  if (raise && threadIdx.x == 0) raise_flags(f.peer_flags, world, rank, epoch);
  const uint32_t* flags = f.peer_flags[rank];
  if (threadIdx.x < world) {
    long long spins = 0;
    while ((int)(load_acquire_sys(flags + threadIdx.x) - epoch) < 0) {
      if (++spins >= max_spins) {
        atomicExch(status, FWD_EB_SHARD_TIMEOUT);
        break;
      }
      __nanosleep(64);
    }
  }
}

// Fold the G slots in rank order.  Threads fold 16-byte packets (4 floats or 8 halves per
// slot) when the geometry allows.
template <typename TP, typename TO, bool VEC>
__global__ void __launch_bounds__(kCtaThreads)
eb_shard_combine_kernel(const TP* slots, int world, long long slot_stride, long long count, TO* out,
                        const int* status, const int* counts, int dim) {
  // The flag exchange ran in eb_shard_wait_kernel just before this grid (one warp, so no
  // spinning CTA ever sits on an SM beside the next call's pooling); a wait that gave up has
  // left its mark in the status word and the output is then left alone.
  if (*static_cast<const volatile int*>(status) != 0) return;
  constexpr int PK = VEC ? 16 / (int)sizeof(TP) : 1;  // elements per packet
  const long long packets = count / PK;
  for (long long i = (long long)blockIdx.x * kCtaThreads + threadIdx.x; i < packets;
       i += (long long)gridDim.x * kCtaThreads) {
    float acc[PK];
#pragma unroll
    for (int e = 0; e < PK; ++e) acc[e] = 0.0f;
    for (int r = 0; r < world; ++r) {
      const TP* src = slots + r * slot_stride + i * PK;
      float v[PK];
      if (VEC && sizeof(TP) == 2) {
        uint4 raw = *reinterpret_cast<const uint4*>(src);
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 t = __half22float2(h[e]);
          v[(2 * e) % PK] = t.x;
          v[(2 * e + 1) % PK] = t.y;
        }
      } else if (VEC) {
        float4 raw = *reinterpret_cast<const float4*>(src);
        v[0] = raw.x; v[1 % PK] = raw.y; v[2 % PK] = raw.z; v[3 % PK] = raw.w;
      } else if (sizeof(TP) == 2) {
        v[0] = __half2float(*reinterpret_cast<const __half*>(src));
      } else {
        v[0] = *reinterpret_cast<const float*>(src);
      }
#pragma unroll
      for (int e = 0; e < PK; ++e) acc[e] = __fadd_rn(acc[e], v[e]);
    }
    if (counts) {  // sharded mean whose partials are plain sums: divide by the bag's count
      const int c = counts[(i * PK) / dim];  // a packet never straddles two bags (dim % PK == 0)
      const float d = (float)(c < 1 ? 1 : c);
#pragma unroll
      for (int e = 0; e < PK; ++e) acc[e] = __fdiv_rn(acc[e], d);
    }
    TO* dst = out + i * PK;
    if (VEC && sizeof(TO) == 4) {
#pragma unroll
      for (int e = 0; e < PK; e += 4) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + e) =
            make_float4(acc[e], acc[(e + 1) % PK], acc[(e + 2) % PK], acc[(e + 3) % PK]);
      }
    } else if (VEC) {
      __half2 pk2[PK / 2 > 0 ? PK / 2 : 1];
#pragma unroll
      for (int e = 0; e < PK / 2; ++e) pk2[e] = __floats2half2_rn(acc[2 * e], acc[(2 * e + 1) % PK]);
      if (PK == 8) {
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(pk2);
      } else {
        *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(pk2);
      }
    } else if (sizeof(TO) == 2) {
      reinterpret_cast<__half*>(dst)[0] = __float2half_rn(acc[0]);
    } else {
      reinterpret_cast<float*>(dst)[0] = acc[0];
    }
  }
}

// Ship staged rows to their owners (fwd_eb_shard_ship).  One thread moves 16 bytes at a time;
// segment = one bag's row of one staged table.  Segments are walked bag-major with the owner
// next, so consecutive warps talk to different peers, and every rank starts with its right-hand
// neighbour.
constexpr int kShipMaxTables = 32;
struct ShipArgs {
  const char* stage;             // this call's part: [world][per][S][seg_bytes]
  char* peer[FWD_EB_MAX_PEERS];  // this call's part of every owner's buffer
  long long per;                 // bags per rank
  long long num_bags;
  long long dst_row_stride;      // bytes between destination rows
  long long dst_row_base;        // first destination row (row shards: rank * per)
  int col_bytes[kShipMaxTables]; // destination column offset of staged slot j
  int world, rank, S, seg_bytes;
};

__global__ void __launch_bounds__(256) eb_shard_ship_kernel(const ShipArgs a) {
  const int vps = a.seg_bytes >> 4;  // 16-byte vectors per segment
  const long long total = a.per * a.world * a.S * vps;
  const long long step = (long long)gridDim.x * blockDim.x;
  constexpr int UNR = 4;
  for (long long v0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; v0 < total; v0 += step * UNR) {
    uint4 val[UNR];
    char* dst[UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const long long v = v0 + u * step;
      dst[u] = nullptr;
      if (v < total) {
        const long long seg = v / vps;
        const int c = (int)(v - seg * vps);
        const int j = (int)(seg % a.S);
        const long long t = seg / a.S;
        const int o = (int)((t % a.world + a.rank + 1) % a.world);
        const long long bag = t / a.world;
        if (o * a.per + bag < a.num_bags) {
          val[u] = *reinterpret_cast<const uint4*>(a.stage + ((o * a.per + bag) * a.S + j) * a.seg_bytes + c * 16);
          dst[u] = a.peer[o] + (a.dst_row_base + bag) * a.dst_row_stride + a.col_bytes[j] + c * 16;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u)
      if (dst[u]) *reinterpret_cast<uint4*>(dst[u]) = val[u];
  }
}

static size_t wire_bytes(int wire_dtype) {
  return wire_dtype == FWD_EB_F16 ? 2u : (wire_dtype == FWD_EB_F32_POS ? 8u : 4u);
}

static int check_exchange(const fwd_eb_shard_exchange* x) {
  if (!x) return fail(FWD_EB_EINVAL, "exchange description is null");
  if (x->world < 1 || x->world > FWD_EB_MAX_PEERS)
    return fail(FWD_EB_EINVAL, "world must be 1..%d (got %d)", FWD_EB_MAX_PEERS, x->world);
  if (x->rank < 0 || x->rank >= x->world) return fail(FWD_EB_EINVAL, "rank %d outside the world", x->rank);
  if (x->bags_per_rank <= 0) return fail(FWD_EB_EINVAL, "bags_per_rank must be positive");
  if (x->wire_dtype != FWD_EB_F32 && x->wire_dtype != FWD_EB_F16 && x->wire_dtype != FWD_EB_F32_POS)
    return fail(FWD_EB_EINVAL, "unknown wire_dtype %d", x->wire_dtype);
  if (x->wire_dtype == FWD_EB_F32_POS && x->layout != FWD_EB_LAYOUT_ROW_SHARD)
    return fail(FWD_EB_EINVAL, "the value + position wire type is for row shards");
  if (x->epoch == 0) return fail(FWD_EB_EINVAL, "epoch starts at 1");
  if (x->raise_from_push && !x->tickets)
    return fail(FWD_EB_EINVAL, "raise_from_push needs the ticket words");
  if (x->stage) {
    if (x->raise_from_push) return fail(FWD_EB_EINVAL, "staged rows are shipped: the flag follows the ship kernel");
    if (x->layout == FWD_EB_LAYOUT_TABLE_WISE &&
        (x->stage_tables < 1 || x->stage_tables > kShipMaxTables || x->stage_slot < 0 ||
         x->stage_slot >= x->stage_tables))
      return fail(FWD_EB_EINVAL, "stage_slot %d outside %d staged tables (at most %d)", x->stage_slot,
                  x->stage_tables, kShipMaxTables);
    if (reinterpret_cast<uintptr_t>(x->stage) & 15u) return fail(FWD_EB_EALIGN, "stage must be 16-byte aligned");
  }
  if (!x->status) return fail(FWD_EB_EINVAL, "status word is null");
  for (int r = 0; r < x->world; ++r) {
    if (!x->peer_slots[r] || !x->peer_flags[r])
      return fail(FWD_EB_EINVAL, "peer %d has no mapped slots / flags", r);
  }
  if (x->layout != FWD_EB_LAYOUT_ROW_SHARD && x->layout != FWD_EB_LAYOUT_TABLE_WISE)
    return fail(FWD_EB_EINVAL, "unknown layout %d", x->layout);
  if (x->layout == FWD_EB_LAYOUT_TABLE_WISE &&
      (x->num_tables < 1 || x->table_index < 0 || x->table_index >= x->num_tables))
    return fail(FWD_EB_EINVAL, "table_index %d outside %d tables", x->table_index, x->num_tables);
  return 0;
}

static size_t part_bytes(const fwd_eb_shard_exchange* x, int dim) {
  const size_t blocks = x->layout == FWD_EB_LAYOUT_TABLE_WISE ? (size_t)x->num_tables : (size_t)x->world;
  return blocks * (size_t)x->bags_per_rank * (size_t)dim * wire_bytes(x->wire_dtype);
}

static void fill_push(const fwd_eb_shard_exchange* x, int dim, PushArgs* out) {
  memset(out, 0, sizeof(*out));
  const size_t part = part_bytes(x, dim) * (x->epoch % FWD_EB_SHARD_BUFFERS);
  for (int r = 0; r < x->world; ++r) {
    out->peer_slots[r] = static_cast<char*>(x->peer_slots[r]) + part;
    out->peer_flags[r] = x->peer_flags[r];
  }
  if (x->layout == FWD_EB_LAYOUT_TABLE_WISE) {
    out->row_base = 0;
    out->col_offset = (long long)x->table_index * dim;
  } else {
    out->row_base = (long long)x->rank * x->bags_per_rank;
    out->col_offset = 0;
  }
  if (x->stage) {
    // every owner's rows go to the local staging scratch, laid out [owner][bag][staged table][dim]
    const int S = x->layout == FWD_EB_LAYOUT_TABLE_WISE ? x->stage_tables : 1;
    const size_t block = (size_t)x->bags_per_rank * S * dim * wire_bytes(x->wire_dtype);
    char* base = static_cast<char*>(x->stage) + block * x->world * (x->epoch % FWD_EB_SHARD_BUFFERS);
    for (int r = 0; r < x->world; ++r) out->peer_slots[r] = base + block * r;
    out->row_base = 0;
    out->col_offset = x->layout == FWD_EB_LAYOUT_TABLE_WISE ? (long long)x->stage_slot * dim : 0;
  }
  out->bags_per_rank = x->bags_per_rank;
  out->world = x->world;
  out->rank = x->rank;
  out->epoch = x->epoch;
  out->ticket = (x->raise_from_push && x->tickets) ? x->tickets + (x->epoch % FWD_EB_SHARD_BUFFERS) : nullptr;
}

static FlagSet flag_set(const fwd_eb_shard_exchange* x) {
  FlagSet f;
  memset(&f, 0, sizeof(f));
  for (int r = 0; r < x->world; ++r) f.peer_flags[r] = x->peer_flags[r];
  return f;
}

template <typename TW, int VE, int CPL, int U, int IPL>
static cudaError_t launch_push(const PoolArgs& a, const PushArgs& x, int tiles, bool weighted,
                               cudaStream_t st) {
  const long long threads = a.num_bags << a.lanes_log2;
  const int cta = group_cta_threads(a.lanes_log2);
  const long long blocks = (threads + cta - 1) / cta;
  if (blocks == 0) return cudaSuccess;
  if (blocks > INT_MAX) return cudaErrorInvalidConfiguration;
  dim3 grid((unsigned)blocks, (unsigned)tiles);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3((unsigned)cta);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];  // see launch_pool in eb_api.cu
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = weighted
      ? cudaLaunchKernelEx(&cfg, eb_pool_push_kernel<TW, VE, CPL, kOpWeighted, U, IPL>, a, x)
      : cudaLaunchKernelEx(&cfg, eb_pool_push_kernel<TW, VE, CPL, kOpSum, U, IPL>, a, x);
  count_launch();
  return e != cudaSuccess ? e : cudaGetLastError();
}

template <typename TW>
static cudaError_t launch_push_shape(const PoolArgs& a, const PushArgs& x, bool vec, int cpl,
                                     int tiles, bool weighted, cudaStream_t st) {
  constexpr int VE = 16 / (int)sizeof(TW);
  if (!vec) return launch_push<TW, 1, 4, 4, 1>(a, x, tiles, weighted, st);
  if (cpl == 1 && a.lanes_log2 == 4) return launch_push<TW, VE, 1, FWD_EB_U1, 2>(a, x, tiles, weighted, st);
  if (cpl == 1 && a.lanes_log2 == 3) return launch_push<TW, VE, 1, FWD_EB_U1, 4>(a, x, tiles, weighted, st);
  if (cpl == 1) return launch_push<TW, VE, 1, FWD_EB_U1, 1>(a, x, tiles, weighted, st);
  if (cpl == 2) return launch_push<TW, VE, 2, 4, 1>(a, x, tiles, weighted, st);
  return launch_push<TW, VE, 4, 2, 1>(a, x, tiles, weighted, st);
}

// The streaming kernel (eb_stream.cuh) with the push epilogue.
template <typename TW, int LL>
static cudaError_t launch_push_stream_ll(const PoolArgs& a, const PushArgs& x, bool weighted,
                                         cudaStream_t st) {
  constexpr int VE = 16 / (int)sizeof(TW);
  const long long groups = (a.num_bags + a.stream_k - 1) / a.stream_k;
  const long long blocks = ((groups << LL) + kCtaThreads - 1) / kCtaThreads;
  if (blocks == 0) return cudaSuccess;
  if (blocks > INT_MAX) return cudaErrorInvalidConfiguration;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3((unsigned)kCtaThreads);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];  // see launch_pool in eb_api.cu
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = weighted
      ? cudaLaunchKernelEx(&cfg, eb_pool_stream_kernel<TW, VE, LL, kOpWeighted, stream_u(LL), true>, a, x)
      : cudaLaunchKernelEx(&cfg, eb_pool_stream_kernel<TW, VE, LL, kOpSum, stream_u(LL), true>, a, x);
  count_launch();
  return e != cudaSuccess ? e : cudaGetLastError();
}

template <typename TW>
static cudaError_t launch_push_stream(const PoolArgs& a, const PushArgs& x, bool weighted,
                                      cudaStream_t st) {
  if (a.lanes_log2 == 3) return launch_push_stream_ll<TW, 3>(a, x, weighted, st);
  if (a.lanes_log2 == 4) return launch_push_stream_ll<TW, 4>(a, x, weighted, st);
  return launch_push_stream_ll<TW, 5>(a, x, weighted, st);
}

// CTA size of the lean kernel when its rows go to peers (a CTA's registers and warp slots are
// released only when its last warp has retired, and a warp that stored to a peer retires only
// when the store has been acknowledged).
constexpr int kPushCtaThreads = kCtaThreads;

// The lean kernel (eb_lite.cuh) with the push epilogue.
template <typename TW, int LL>
static cudaError_t launch_push_lite_ll(const PoolArgs& a, const PushArgs& x, bool weighted,
                                       cudaStream_t st) {
  constexpr int VE = 16 / (int)sizeof(TW);
  // One bag per lane group.  (A warp must wait for its peer stores before it can exit, and a
  // second bag to walk would hide that wait; but two bags per group also halve the number of
  // groups, and on two B200s the step got slower, not faster: 32.5 against 24.5 us table-wise,
  // 150 against 133 us on config 5.  The hardware's hand-out of CTAs balances ragged bags better.)
  const PoolArgs& b = a;
  int cta = kPushCtaThreads;
#ifdef FWD_EB_TUNE
  if (const char* env = getenv("FWD_EB_PUSH_CTA")) cta = atoi(env) >= 32 ? atoi(env) : cta;
#endif
  const long long blocks = ((a.num_bags << LL) + cta - 1) / cta;
  if (blocks == 0) return cudaSuccess;
  if (blocks > INT_MAX) return cudaErrorInvalidConfiguration;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3((unsigned)cta);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];  // see launch_pool in eb_api.cu
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = weighted
      ? cudaLaunchKernelEx(&cfg, eb_pool_lite_kernel<TW, VE, LL, kOpWeighted, true>, b, x)
      : cudaLaunchKernelEx(&cfg, eb_pool_lite_kernel<TW, VE, LL, kOpSum, true>, b, x);
  count_launch();
  return e != cudaSuccess ? e : cudaGetLastError();
}

template <typename TW>
static cudaError_t launch_push_lite(const PoolArgs& a, const PushArgs& x, bool weighted, cudaStream_t st) {
  if (a.lanes_log2 == 3) return launch_push_lite_ll<TW, 3>(a, x, weighted, st);
  if (a.lanes_log2 == 4) return launch_push_lite_ll<TW, 4>(a, x, weighted, st);
  return launch_push_lite_ll<TW, 5>(a, x, weighted, st);
}

static_assert(FWD_EB_MAX_PEERS == 16, "PushArgs (eb_stream.cuh) holds 16 peers");

}  // namespace fwd_eb

using namespace fwd_eb;

extern "C" {

size_t fwd_eb_shard_slots_bytes(int32_t world, int64_t bags_per_rank, int32_t dim,
                                int32_t wire_dtype) {
  if (world < 1 || bags_per_rank < 1 || dim < 1) return 0;
  return (size_t)FWD_EB_SHARD_BUFFERS * (size_t)world * (size_t)bags_per_rank * (size_t)dim * wire_bytes(wire_dtype);
}

int fwd_eb_shard_push(const fwd_eb_params* p, const fwd_eb_shard_exchange* x, void* stream) {
  int rc = check_exchange(x);
  if (rc) return rc;
  if (!p) return fail(FWD_EB_EINVAL, "params is null");
  if (p->mode != FWD_EB_MODE_SUM && p->mode != FWD_EB_MODE_MEAN)
    return fail(FWD_EB_EUNSUPPORTED, "pushed pooling supports SUM and MEAN (got mode %d); a sharded "
                "MAX goes through the staged exchange", p->mode);
  if (x->wire_dtype == FWD_EB_F32_POS)
    return fail(FWD_EB_EINVAL, "the value + position wire type belongs to MAX (staged exchange)");
  if (p->num_bags > x->bags_per_rank * x->world)
    return fail(FWD_EB_EINVAL, "%lld bags do not fit %d ranks x %lld bags", (long long)p->num_bags,
                x->world, (long long)x->bags_per_rank);
  // Reuse the single-GPU planner for shapes and checks; the output it plans for is replaced.
  fwd_eb_params q = *p;
  q.out = x->peer_slots[x->rank];
  q.out_dtype = x->wire_dtype;
  if (x->layout == FWD_EB_LAYOUT_ROW_SHARD) {
    q.flags |= FWD_EB_FLAG_MEAN_SINGLE_ROUNDING;  // a partial is not the final fp16 mean torch would round
    // a row window filters most indices away unless they were compacted first: the group
    // kernel's survivor ring is the one built for that (every rank, rank 0 included)
    if (!(q.flags & FWD_EB_FLAG_OFFSET_PAIRS) && q.strategy == FWD_EB_STRATEGY_AUTO)
      q.strategy = FWD_EB_STRATEGY_GROUP;
  }
  q.out_stride = x->layout == FWD_EB_LAYOUT_TABLE_WISE
                     ? (int64_t)(x->stage ? x->stage_tables : x->num_tables) * p->dim : 0;
  if (x->stage && ((size_t)p->dim * wire_bytes(x->wire_dtype)) % 16 != 0)
    return fail(FWD_EB_EUNSUPPORTED, "shipping needs rows that are a multiple of 16 bytes on the wire");
  PoolArgs a;
  int vec = 0, cpl = 0, tiles = 0, stream_kernel = 0;
  rc = plan_group(&q, &a, &vec, &cpl, &tiles, &stream_kernel);
  if (rc) return rc;
  PushArgs px;
  fill_push(x, p->dim, &px);
  px.first_bag = (long long)((x->rank + 1) % x->world) * x->bags_per_rank;
  if (px.first_bag >= p->num_bags) px.first_bag = 0;
  px.small = p->num_bags <= 0x7fffffffLL && x->bags_per_rank <= 0x7fffffffLL;
  const bool weighted = p->per_sample_weights != nullptr;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (stream_kernel == 1) {
    e = p->table_dtype == FWD_EB_F16 ? launch_push_stream<__half>(a, px, weighted, st)
                                     : launch_push_stream<float>(a, px, weighted, st);
  } else if (stream_kernel == 2) {
    e = p->table_dtype == FWD_EB_F16 ? launch_push_lite<__half>(a, px, weighted, st)
                                     : launch_push_lite<float>(a, px, weighted, st);
  } else {
    e = p->table_dtype == FWD_EB_F16
            ? launch_push_shape<__half>(a, px, vec != 0, cpl, tiles, weighted, st)
            : launch_push_shape<float>(a, px, vec != 0, cpl, tiles, weighted, st);
  }
  if (e != cudaSuccess) return cuda_fail(e, "push kernel launch");
  clear_error();
  return 0;
}

int fwd_eb_shard_pool_local(const fwd_eb_params* p, const fwd_eb_shard_exchange* x, void* stream) {
  int rc = check_exchange(x);
  if (rc) return rc;
  if (!p) return fail(FWD_EB_EINVAL, "params is null");
  if (x->layout != FWD_EB_LAYOUT_TABLE_WISE)
    return fail(FWD_EB_EINVAL, "a replicated table belongs to the table-wise layout");
  if (p->mode == FWD_EB_MODE_GATHER) return fail(FWD_EB_EUNSUPPORTED, "GATHER has no pooled row to place");
  if (x->wire_dtype != FWD_EB_F32 && x->wire_dtype != FWD_EB_F16)
    return fail(FWD_EB_EINVAL, "the table-wise buffer holds fp32 or fp16 rows");
  if (p->num_bags > x->bags_per_rank)
    return fail(FWD_EB_EINVAL, "%lld bags, but a rank owns at most %lld", (long long)p->num_bags,
                (long long)x->bags_per_rank);
  fwd_eb_params q = *p;
  const size_t part = part_bytes(x, p->dim) * (x->epoch % FWD_EB_SHARD_BUFFERS);
  q.out = static_cast<char*>(x->peer_slots[x->rank]) + part +
          (size_t)x->table_index * (size_t)p->dim * wire_bytes(x->wire_dtype);
  q.out_dtype = x->wire_dtype;
  q.out_stride = (int64_t)x->num_tables * p->dim;
  return fwd_eb_forward(&q, stream);
}

size_t fwd_eb_shard_stage_bytes(int32_t world, int64_t bags_per_rank, int32_t stage_tables, int32_t dim,
                                int32_t wire_dtype) {
  if (world < 1 || bags_per_rank < 1 || stage_tables < 1 || dim < 1) return 0;
  return (size_t)FWD_EB_SHARD_BUFFERS * (size_t)world * (size_t)bags_per_rank * (size_t)stage_tables *
         (size_t)dim * wire_bytes(wire_dtype);
}

int fwd_eb_shard_ship(const fwd_eb_shard_exchange* x, int32_t dim, int64_t num_bags,
                      const int32_t* table_ids, void* stream) {
  int rc = check_exchange(x);
  if (rc) return rc;
  if (!x->stage) return fail(FWD_EB_EINVAL, "nothing was staged: x->stage is null");
  if (dim <= 0 || num_bags < 0 || num_bags > x->bags_per_rank * x->world)
    return fail(FWD_EB_EINVAL, "bad ship arguments");
  const bool tw = x->layout == FWD_EB_LAYOUT_TABLE_WISE;
  if (tw && !table_ids) return fail(FWD_EB_EINVAL, "table_ids is null");
  const size_t seg = (size_t)dim * wire_bytes(x->wire_dtype);
  if (seg % 16 != 0 || seg > 0x7fffffffu)
    return fail(FWD_EB_EUNSUPPORTED, "shipping needs rows that are a multiple of 16 bytes on the wire");
  if (num_bags == 0) return 0;
  ShipArgs a;
  memset(&a, 0, sizeof(a));
  a.S = tw ? x->stage_tables : 1;
  a.seg_bytes = (int)seg;
  a.per = x->bags_per_rank;
  a.num_bags = num_bags;
  a.world = x->world;
  a.rank = x->rank;
  const size_t block = (size_t)x->bags_per_rank * a.S * seg;
  a.stage = static_cast<const char*>(x->stage) + block * x->world * (x->epoch % FWD_EB_SHARD_BUFFERS);
  const size_t part = part_bytes(x, dim) * (size_t)(x->epoch % FWD_EB_SHARD_BUFFERS);
  for (int r = 0; r < x->world; ++r) a.peer[r] = static_cast<char*>(x->peer_slots[r]) + part;
  if (tw) {
    a.dst_row_stride = (long long)x->num_tables * (long long)seg;
    a.dst_row_base = 0;
    for (int j = 0; j < a.S; ++j) {
      if (table_ids[j] < 0 || table_ids[j] >= x->num_tables)
        return fail(FWD_EB_EINVAL, "table_ids[%d] = %d outside %d tables", j, table_ids[j], x->num_tables);
      a.col_bytes[j] = (int)(table_ids[j] * (long long)seg);
    }
  } else {
    a.dst_row_stride = (long long)seg;
    a.dst_row_base = (long long)x->rank * x->bags_per_rank;
  }
  const long long vectors = (long long)x->bags_per_rank * x->world * a.S * (long long)(seg / 16);
  long long blocks = (vectors + 256 * 4 - 1) / (256 * 4);
  const long long cap = sm_count() / 2 > 0 ? sm_count() / 2 : 1;   // a corner of the GPU: the pooling has the rest
  if (blocks > cap) blocks = cap;
  eb_shard_ship_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "ship kernel launch");
  clear_error();
  return 0;
}

size_t fwd_eb_shard_tablewise_bytes(int64_t bags_per_rank, int32_t num_tables, int32_t dim,
                                    int32_t wire_dtype) {
  if (num_tables < 1 || bags_per_rank < 1 || dim < 1) return 0;
  return (size_t)FWD_EB_SHARD_BUFFERS * (size_t)num_tables * (size_t)bags_per_rank * (size_t)dim * (wire_dtype == FWD_EB_F16 ? 2u : 4u);
}

int fwd_eb_shard_wait(const fwd_eb_shard_exchange* x, int32_t dim, void** d_result, void* stream) {
  int rc = check_exchange(x);
  if (rc) return rc;
  if (dim <= 0) return fail(FWD_EB_EINVAL, "dim must be positive");
  const long long spins = x->max_spins > 0 ? x->max_spins : (1LL << 22);
  eb_shard_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      flag_set(x), x->rank, x->world, x->epoch, x->status, spins, x->raise_from_push ? 0 : 1);
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "wait kernel launch");
  if (d_result)
    *d_result = static_cast<char*>(x->peer_slots[x->rank]) + part_bytes(x, dim) * (x->epoch % FWD_EB_SHARD_BUFFERS);
  return 0;
}

int fwd_eb_shard_signal(const fwd_eb_shard_exchange* x, void* stream) {
  int rc = check_exchange(x);
  if (rc) return rc;
  eb_shard_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flag_set(x), x->world,
                                                                          x->rank, x->epoch);
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "signal kernel launch");
  return 0;
}

int fwd_eb_shard_combine(const fwd_eb_shard_exchange* x, int32_t dim, int64_t num_bags,
                         void* d_out, int32_t out_dtype, void* stream) {
  return fwd_eb_shard_combine_div(x, dim, num_bags, nullptr, d_out, out_dtype, stream);
}

int fwd_eb_shard_combine_div(const fwd_eb_shard_exchange* x, int32_t dim, int64_t num_bags,
                             const int32_t* d_counts, void* d_out, int32_t out_dtype, void* stream) {
  int rc = check_exchange(x);
  if (rc) return rc;
  if (dim <= 0 || num_bags < 0 || num_bags > x->bags_per_rank || (num_bags > 0 && !d_out))
    return fail(FWD_EB_EINVAL, "bad combine arguments");
  if (out_dtype != FWD_EB_F32 && out_dtype != FWD_EB_F16)
    return fail(FWD_EB_EINVAL, "unknown out_dtype %d", out_dtype);
  const long long count = (long long)num_bags * dim;
  const long long slot_stride = (long long)x->bags_per_rank * dim;
  const char* slots = static_cast<const char*>(x->peer_slots[x->rank]) + part_bytes(x, dim) * (x->epoch % FWD_EB_SHARD_BUFFERS);
  const FlagSet flags = flag_set(x);
  const long long spins = x->max_spins > 0 ? x->max_spins : (1LL << 22);
  const bool wire16 = x->wire_dtype == FWD_EB_F16, out16 = out_dtype == FWD_EB_F16;
  if (x->wire_dtype == FWD_EB_F32_POS) {
    if (d_counts) return fail(FWD_EB_EINVAL, "a divisor makes no sense for a sharded MAX");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    long long blocks = (count + kCtaThreads - 1) / kCtaThreads;
    if (blocks > sm_count() * 8) blocks = sm_count() * 8;
    if (blocks < 1) blocks = 1;
    eb_shard_wait_kernel<<<1, 32, 0, st>>>(flags, x->rank, x->world, x->epoch, x->status, spins,
                                         x->raise_from_push ? 0 : 1);
    count_launch();
    if (out16) {
      eb_shard_combine_max_kernel<__half><<<(unsigned)blocks, kCtaThreads, 0, st>>>(
          reinterpret_cast<const int2*>(slots), x->world, slot_stride, count,
          static_cast<__half*>(d_out), x->status);
    } else {
      eb_shard_combine_max_kernel<float><<<(unsigned)blocks, kCtaThreads, 0, st>>>(
          reinterpret_cast<const int2*>(slots), x->world, slot_stride, count,
          static_cast<float*>(d_out), x->status);
    }
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "max fold kernel launch");
    clear_error();
    return 0;
  }
  const int pk = wire16 ? 8 : 4;
  const bool vec = count % pk == 0 && slot_stride % pk == 0 && dim % pk == 0 &&
                   (reinterpret_cast<uintptr_t>(slots) & 15u) == 0 &&
                   (reinterpret_cast<uintptr_t>(d_out) & 15u) == 0;
  const long long packets = vec ? count / pk : count;
  long long blocks = (packets + kCtaThreads - 1) / kCtaThreads;
  if (blocks > sm_count() * 4) blocks = sm_count() * 4;
  if (blocks < 1) blocks = 1;
  const unsigned g = (unsigned)blocks;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // flag exchange first, in a one-warp kernel of its own
  eb_shard_wait_kernel<<<1, 32, 0, st>>>(flags, x->rank, x->world, x->epoch, x->status, spins,
                                         x->raise_from_push ? 0 : 1);
  count_launch();
#define FWD_EB_COMBINE(TP, TO, V)                                                                \
  eb_shard_combine_kernel<TP, TO, V><<<g, kCtaThreads, 0, st>>>(                                 \
      reinterpret_cast<const TP*>(slots), x->world, slot_stride, count, static_cast<TO*>(d_out), \
      x->status, d_counts, dim)
  if (vec) {
    if (!wire16 && !out16) FWD_EB_COMBINE(float, float, true);
    else if (!wire16 && out16) FWD_EB_COMBINE(float, __half, true);
    else if (wire16 && !out16) FWD_EB_COMBINE(__half, float, true);
    else FWD_EB_COMBINE(__half, __half, true);
  } else {
    if (!wire16 && !out16) FWD_EB_COMBINE(float, float, false);
    else if (!wire16 && out16) FWD_EB_COMBINE(float, __half, false);
    else if (wire16 && !out16) FWD_EB_COMBINE(__half, float, false);
    else FWD_EB_COMBINE(__half, __half, false);
  }
#undef FWD_EB_COMBINE
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "combine kernel launch");
  clear_error();
  return 0;
}

// ---- pipeline: a step's stream / event choreography ------------------------------------------------

}  // extern "C"

struct fwd_eb_pipeline {
  cudaStream_t side = nullptr;
  cudaEvent_t pushed[FWD_EB_SHARD_BUFFERS] = {};
  cudaEvent_t done[FWD_EB_SHARD_BUFFERS] = {};
  uint32_t epoch = 0;
  uint32_t every = FWD_EB_PIPELINE_WAIT_EVERY;
  uint32_t depth = FWD_EB_PIPELINE_WAIT_DEPTH;
  // Replicated tables of a hybrid table-wise step are pooled on these streams, beside the pushes
  // on the caller's stream: the launches are independent of each other, and a rank's share of a
  // batch is a grid of one or two waves whose ramp and tail another grid can fill.
  cudaStream_t aux[FWD_EB_PIPELINE_LOCAL_STREAMS] = {};
  cudaEvent_t fork = nullptr;
  cudaEvent_t joined[FWD_EB_PIPELINE_LOCAL_STREAMS] = {};
  int32_t local_streams = FWD_EB_PIPELINE_LOCAL_STREAMS;
  // Steps may be issued on more than one caller stream (consecutive steps are independent
  // batches, and on two alternating streams one step's grid runs beside the tail of the step
  // before).  The look-back is a property of the stream a step is issued on: for each stream
  // seen, the newest fold it has been made to wait for.
  struct Seen {
    cudaStream_t stream;
    uint32_t waited;
    bool used;
  } seen[FWD_EB_PIPELINE_MAIN_STREAMS] = {};
};

// A step that fails its host-side checks before anything was launched must not leave this rank
// one call number ahead of its peers (their next wait would accept this rank's NEXT flag and
// fold a buffer part it never wrote): such a return takes the number back.
static int pipeline_abort(fwd_eb_pipeline* pl, int rc) {
  pl->epoch -= 1;
  return rc;
}

static int pipeline_begin(fwd_eb_pipeline* pl, fwd_eb_shard_exchange* x, cudaStream_t main) {
  // Call numbers are 32-bit flag values and pick the buffer part by a modulo: refuse the step that
  // would wrap them (2^32 steps: more than a day at 25 us a step) instead of going out of phase.
  if (pl->epoch >= 0xfffffff0u)
    return fail(FWD_EB_ETOOBIG, "this pipeline has run 2^32 steps: drain it on every rank and create a new one");
  pl->epoch += 1;
  x->epoch = pl->epoch;
  static_assert(FWD_EB_PIPELINE_WAIT_EVERY + FWD_EB_PIPELINE_WAIT_DEPTH <= FWD_EB_SHARD_BUFFERS, "k + d parts");
  static_assert(2 * (FWD_EB_PIPELINE_WAIT_EVERY_TICKETS - 1) + 2 * FWD_EB_PIPELINE_WAIT_DEPTH <= FWD_EB_SHARD_BUFFERS,
                "2(k-1) + 2d parts");
  const uint32_t every = x->tickets ? FWD_EB_PIPELINE_WAIT_EVERY_TICKETS : pl->every;
  const uint32_t depth = x->tickets ? FWD_EB_PIPELINE_WAIT_DEPTH : pl->depth;
  // Step e may start only behind this rank's fold of some step >= e - (every - 1) - depth (see
  // FWD_EB_SHARD_BUFFERS for why that is enough with the buffer parts there are).  On one stream
  // that is a wait on every `every`-th step, inherited by the steps queued behind it; a stream
  // that was not seen before, or when the table of streams is full, waits now.
  fwd_eb_pipeline::Seen* slot = nullptr;
  for (auto& sn : pl->seen)
    if (sn.used && sn.stream == main) slot = &sn;
  if (!slot) {
    for (auto& sn : pl->seen)
      if (!sn.used && !slot) slot = &sn;
    if (slot) {
      slot->used = true;
      slot->stream = main;
      slot->waited = 0;
    }
  }
  const uint32_t waited = slot ? slot->waited : 0;
  if (pl->epoch > depth && (uint64_t)waited + (every - 1) + depth < pl->epoch) {
    cudaError_t e = cudaStreamWaitEvent(main, pl->done[(pl->epoch - depth) % FWD_EB_SHARD_BUFFERS], 0);
    if (e != cudaSuccess) {
      pl->epoch -= 1;
      return cuda_fail(e, "cudaStreamWaitEvent (main)");
    }
    if (slot) slot->waited = pl->epoch - depth;
  }
  return 0;
}

// The side stream must not run ahead of the main stream's work of this step (staged exchange:
// the copies read what the pooling wrote).  Steps whose pooling grid raises the flag itself need
// no such hand-over: their side-stream kernel waits for flags, this rank's own included.
static int pipeline_handover(fwd_eb_pipeline* pl, cudaStream_t main) {
  const int k = pl->epoch % FWD_EB_SHARD_BUFFERS;
  cudaError_t e = cudaEventRecord(pl->pushed[k], main);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(pl->side, pl->pushed[k], 0);
  if (e != cudaSuccess) return cuda_fail(e, "handing a step to the side stream");
  return 0;
}

extern "C" {

int fwd_eb_pipeline_create(fwd_eb_pipeline** out) {
  if (!out) return fail(FWD_EB_EINVAL, "out pointer is null");
  *out = nullptr;
  fwd_eb_pipeline* pl = new (std::nothrow) fwd_eb_pipeline();
  if (!pl) return fail(FWD_EB_EINVAL, "out of host memory");
  int lo = 0, hi = 0;
  cudaError_t e = cudaDeviceGetStreamPriorityRange(&lo, &hi);  // hi = numerically lowest = most urgent
  if (e == cudaSuccess) e = cudaStreamCreateWithPriority(&pl->side, cudaStreamNonBlocking, hi);
  for (int k = 0; k < FWD_EB_SHARD_BUFFERS && e == cudaSuccess; ++k) {
    e = cudaEventCreateWithFlags(&pl->pushed[k], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&pl->done[k], cudaEventDisableTiming);
  }
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&pl->fork, cudaEventDisableTiming);
  for (int k = 0; k < FWD_EB_PIPELINE_LOCAL_STREAMS && e == cudaSuccess; ++k) {
    e = cudaStreamCreateWithFlags(&pl->aux[k], cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&pl->joined[k], cudaEventDisableTiming);
  }
  if (e != cudaSuccess) {
    int rc = cuda_fail(e, "creating the pipeline's stream and events");
    fwd_eb_pipeline_destroy(pl);
    return rc;
  }
  *out = pl;
  return 0;
}

void fwd_eb_pipeline_destroy(fwd_eb_pipeline* pl) {
  if (!pl) return;
  if (pl->side) cudaStreamSynchronize(pl->side);
  for (int k = 0; k < FWD_EB_SHARD_BUFFERS; ++k) {
    if (pl->pushed[k]) cudaEventDestroy(pl->pushed[k]);
    if (pl->done[k]) cudaEventDestroy(pl->done[k]);
  }
  for (int k = 0; k < FWD_EB_PIPELINE_LOCAL_STREAMS; ++k) {
    if (pl->aux[k]) {
      cudaStreamSynchronize(pl->aux[k]);
      cudaStreamDestroy(pl->aux[k]);
    }
    if (pl->joined[k]) cudaEventDestroy(pl->joined[k]);
  }
  if (pl->fork) cudaEventDestroy(pl->fork);
  if (pl->side) cudaStreamDestroy(pl->side);
  delete pl;
}

void* fwd_eb_pipeline_side_stream(fwd_eb_pipeline* pl) { return pl ? pl->side : nullptr; }

int fwd_eb_pipeline_set_local_streams(fwd_eb_pipeline* pl, int32_t streams) {
  if (!pl) return fail(FWD_EB_EINVAL, "null pipeline");
  if (streams < 0 || streams > FWD_EB_PIPELINE_LOCAL_STREAMS)
    return fail(FWD_EB_EINVAL, "0..%d streams for replicated tables (got %d)", FWD_EB_PIPELINE_LOCAL_STREAMS, streams);
  pl->local_streams = streams;
  return 0;
}

int fwd_eb_pipeline_set_lookback(fwd_eb_pipeline* pl, int32_t every, int32_t depth) {
  if (!pl) return fail(FWD_EB_EINVAL, "null pipeline");
  if (every < 1 || depth < 2 || every + depth > FWD_EB_SHARD_BUFFERS)
    return fail(FWD_EB_EINVAL, "lookback needs every >= 1, depth >= 2 and every + depth <= %d (got %d, %d)",
                FWD_EB_SHARD_BUFFERS, every, depth);
  if (pl->epoch != 0) return fail(FWD_EB_EINVAL, "set the lookback before the first step");
  pl->every = (uint32_t)every;
  pl->depth = (uint32_t)depth;
  return 0;
}

int fwd_eb_pipeline_step_rowshard(fwd_eb_pipeline* pl, const fwd_eb_params* p,
                                  fwd_eb_shard_exchange* x, int64_t num_bags_owned,
                                  void* const d_out[FWD_EB_SHARD_BUFFERS], int32_t out_dtype,
                                  void* main_stream, int32_t* which) {
  NvtxRange range("fwd_eb_pipeline_step_rowshard");
  if (!pl || !p || !x || !d_out) return fail(FWD_EB_EINVAL, "null argument");
  cudaStream_t main = static_cast<cudaStream_t>(main_stream);
  int rc = pipeline_begin(pl, x, main);
  if (rc) return rc;
  x->raise_from_push = (x->tickets && !x->stage) ? 1 : 0;
  rc = fwd_eb_shard_push(p, x, main);   // validates before it launches
  if (rc) return pipeline_abort(pl, rc);
  if (!x->raise_from_push) {
    rc = pipeline_handover(pl, main);
    if (rc) return rc;
  }
  if (x->stage) {   // the staged rows go to their owners from the side stream
    rc = fwd_eb_shard_ship(x, p->dim, p->num_bags, nullptr, pl->side);
    if (rc) return rc;
  }
  const int k = pl->epoch % FWD_EB_SHARD_BUFFERS;
  rc = fwd_eb_shard_combine(x, p->dim, num_bags_owned, d_out[k], out_dtype, pl->side);
  if (rc) return rc;
  cudaError_t e = cudaEventRecord(pl->done[k], pl->side);
  if (e != cudaSuccess) return cuda_fail(e, "cudaEventRecord (side)");
  if (which) *which = k;
  return 0;
}

int fwd_eb_pipeline_step_rowshard_compact(fwd_eb_pipeline* pl, const fwd_eb_params* p,
                                          fwd_eb_shard_exchange* x, int64_t num_bags_owned,
                                          const fwd_eb_compact_scratch* scratch,
                                          void* const d_out[FWD_EB_SHARD_BUFFERS], int32_t out_dtype,
                                          void* main_stream, int32_t* which) {
  NvtxRange range("fwd_eb_pipeline_step_rowshard_compact");
  if (!pl || !p || !x || !d_out || !scratch) return fail(FWD_EB_EINVAL, "null argument");
  if (x->layout != FWD_EB_LAYOUT_ROW_SHARD)
    return fail(FWD_EB_EINVAL, "window compaction is for the row-shard layout");
  if (p->mode != FWD_EB_MODE_SUM && p->mode != FWD_EB_MODE_MEAN)
    return fail(FWD_EB_EUNSUPPORTED, "compacted row shards support SUM and MEAN (got mode %d); a sharded "
                "MAX goes through the staged exchange", p->mode);
  const bool mean = p->mode == FWD_EB_MODE_MEAN;
  if (!scratch->kept || !scratch->bounds || (mean && !scratch->counts) ||
      (p->per_sample_weights && !scratch->kept_weights))
    return fail(FWD_EB_EINVAL, "compaction scratch is incomplete");
  cudaStream_t main = static_cast<cudaStream_t>(main_stream);
  int rc = pipeline_begin(pl, x, main);
  if (rc) return rc;
  const int k = pl->epoch % FWD_EB_SHARD_BUFFERS;
  if (!d_out[k]) return pipeline_abort(pl, fail(FWD_EB_EINVAL, "null output buffer"));
  // 1. the window filter as one streaming pass; a mean also keeps each bag's full count, in the
  //    part of `counts` that belongs to this step (the fold reads it beside the next step)
  const int64_t all_bags = (int64_t)x->world * x->bags_per_rank;
  int32_t* counts = mean ? scratch->counts + (int64_t)k * all_bags : nullptr;
  rc = fwd_eb_compact_window(p, scratch->kept, scratch->kept_weights, scratch->bounds, counts, main);
  if (rc) return pipeline_abort(pl, rc);
  // 2. pool the dense sub-bags, partial rows pushed to their owners (partials of a mean are sums)
  fwd_eb_params q = *p;
  q.indices = scratch->kept;
  q.index_dtype = FWD_EB_I32;
  q.offsets = scratch->bounds;
  q.flags = (p->flags | FWD_EB_FLAG_OFFSET_PAIRS | FWD_EB_FLAG_PAIRS_RUN16);
  q.fixed_len = 0;
  q.include_last_offset = 0;
  q.row_lo = 0;
  q.padding_idx = -1;
  q.mode = FWD_EB_MODE_SUM;
  if (p->per_sample_weights) q.per_sample_weights = scratch->kept_weights;
  if (q.strategy != FWD_EB_STRATEGY_GROUP && q.strategy != FWD_EB_STRATEGY_STREAM &&
      q.strategy != FWD_EB_STRATEGY_LITE)
    q.strategy = FWD_EB_STRATEGY_AUTO;
  x->raise_from_push = (x->tickets && !x->stage) ? 1 : 0;
  rc = fwd_eb_shard_push(&q, x, main);
  if (rc) return rc;   // the compaction has run: the step cannot be taken back
  if (!x->raise_from_push) {
    rc = pipeline_handover(pl, main);
    if (rc) return rc;
  }
  if (x->stage) {   // the staged rows go to their owners from the side stream
    rc = fwd_eb_shard_ship(x, p->dim, p->num_bags, nullptr, pl->side);
    if (rc) return rc;
  }
  // 3. flags, bounded wait, fold (and the mean's division) on the side stream
  rc = fwd_eb_shard_combine_div(x, p->dim, num_bags_owned,
                                mean ? counts + (int64_t)x->rank * x->bags_per_rank : nullptr, d_out[k],
                                out_dtype, pl->side);
  if (rc) return rc;
  cudaError_t e = cudaEventRecord(pl->done[k], pl->side);
  if (e != cudaSuccess) return cuda_fail(e, "cudaEventRecord (side)");
  if (which) *which = k;
  return 0;
}

int fwd_eb_shard_send_staged(const fwd_eb_shard_exchange* x, int32_t dim, int64_t num_bags,
                             const void* d_stage, void* stream) {
  int rc = check_exchange(x);
  if (rc) return rc;
  if (x->layout != FWD_EB_LAYOUT_ROW_SHARD)
    return fail(FWD_EB_EINVAL, "the staged exchange is for the row-shard layout");
  if (dim <= 0 || num_bags < 0 || num_bags > x->bags_per_rank * x->world || !d_stage)
    return fail(FWD_EB_EINVAL, "bad send_staged arguments");
  const size_t row_bytes = (size_t)dim * wire_bytes(x->wire_dtype);
  const size_t part = part_bytes(x, dim) * (size_t)(x->epoch % FWD_EB_SHARD_BUFFERS);
  for (int i = 0; i < x->world; ++i) {
    const int r = (x->rank + 1 + i) % x->world;  // peers first, own block last
    long long rows = num_bags - (long long)r * x->bags_per_rank;
    if (rows > x->bags_per_rank) rows = x->bags_per_rank;
    if (rows <= 0) continue;
    const char* src = static_cast<const char*>(d_stage) + (size_t)r * x->bags_per_rank * row_bytes;
    char* dst = static_cast<char*>(x->peer_slots[r]) + part + (size_t)x->rank * x->bags_per_rank * row_bytes;
    cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)rows * row_bytes, cudaMemcpyDefault,
                                    static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e, "copying a block of partial bags to its owner");
  }
  return 0;
}

int fwd_eb_pipeline_step_rowshard_staged(fwd_eb_pipeline* pl, const fwd_eb_params* p,
                                         fwd_eb_shard_exchange* x, int64_t num_bags_owned,
                                         void* const d_stage[FWD_EB_SHARD_BUFFERS],
                                         void* const d_out[FWD_EB_SHARD_BUFFERS], int32_t out_dtype,
                                         void* main_stream, int32_t* which) {
  NvtxRange range("fwd_eb_pipeline_step_rowshard_staged");
  if (!pl || !p || !x || !d_out || !d_stage) return fail(FWD_EB_EINVAL, "null argument");
  int rc = 0;
  if (x->layout != FWD_EB_LAYOUT_ROW_SHARD)
    return fail(FWD_EB_EINVAL, "the staged exchange is for the row-shard layout");
  const bool is_max = p->mode == FWD_EB_MODE_MAX;
  if (p->mode != FWD_EB_MODE_SUM && p->mode != FWD_EB_MODE_MEAN && !is_max)
    return fail(FWD_EB_EUNSUPPORTED, "sharded pooling supports SUM, MEAN and MAX (got mode %d)", p->mode);
  if (is_max != (x->wire_dtype == FWD_EB_F32_POS))
    return fail(FWD_EB_EINVAL, "MAX needs wire_dtype FWD_EB_F32_POS, and only MAX does");
  if (p->num_bags > x->bags_per_rank * x->world)
    return fail(FWD_EB_EINVAL, "%lld bags do not fit %d ranks x %lld bags", (long long)p->num_bags,
                x->world, (long long)x->bags_per_rank);
  cudaStream_t main = static_cast<cudaStream_t>(main_stream);
  rc = pipeline_begin(pl, x, main);
  if (rc) return rc;
  x->raise_from_push = 0;   // the flag follows the copies: raised by the kernel behind them
  rc = check_exchange(x);
  if (rc) return pipeline_abort(pl, rc);
  const int k = pl->epoch % FWD_EB_SHARD_BUFFERS;
  if (!d_stage[k] || !d_out[k]) return pipeline_abort(pl, fail(FWD_EB_EINVAL, "null staging or output buffer"));
  // 1. pool every bag's partial into local staging (the plain lane-group kernel)
  fwd_eb_params q = *p;
  q.strategy = FWD_EB_STRATEGY_GROUP;
  q.out = d_stage[k];
  q.out_dtype = x->wire_dtype;  // fp32 / fp16 partial sums, or {value, position} pairs for MAX
  q.out_stride = 0;
  q.flags |= FWD_EB_FLAG_MEAN_SINGLE_ROUNDING;  // a partial is not the final fp16 mean
  rc = fwd_eb_forward(&q, main);   // validates before it launches
  if (rc) return pipeline_abort(pl, rc);
  rc = pipeline_handover(pl, main);
  if (rc) return rc;
  // 2. one copy-engine transfer per owner: its block of partial bags -> slot [rank] over there
  rc = fwd_eb_shard_send_staged(x, p->dim, p->num_bags, d_stage[k], pl->side);
  if (rc) return rc;
  // 3. flags (raised by the kernel that follows the copies on the stream), bounded wait, fold
  rc = fwd_eb_shard_combine(x, p->dim, num_bags_owned, d_out[k], out_dtype, pl->side);
  if (rc) return rc;
  cudaError_t e = cudaEventRecord(pl->done[k], pl->side);
  if (e != cudaSuccess) return cuda_fail(e, "cudaEventRecord (side)");
  if (which) *which = k;
  return 0;
}

int fwd_eb_pipeline_step_tablewise_hybrid(fwd_eb_pipeline* pl, const fwd_eb_params* const* params,
                                          const int32_t* table_index, int32_t count,
                                          const fwd_eb_params* const* local_params,
                                          const int32_t* local_table_index, int32_t local_count,
                                          fwd_eb_shard_exchange* x, int32_t dim, void* main_stream,
                                          void** d_result) {
  NvtxRange range("fwd_eb_pipeline_step_tablewise_hybrid");
  if (!pl || !x || count < 0 || (count > 0 && (!params || !table_index)) || local_count < 0 ||
      (local_count > 0 && (!local_params || !local_table_index)))
    return fail(FWD_EB_EINVAL, "null argument");
  if (local_count > 0 && x->tickets)
    return fail(FWD_EB_EUNSUPPORTED, "replicated tables need the flag raised behind the step's last "
                "kernel (x->tickets must be null)");
  cudaStream_t main = static_cast<cudaStream_t>(main_stream);
  int rc = pipeline_begin(pl, x, main);
  if (rc) return rc;
  const bool from_push = x->tickets != nullptr && count > 0 && !x->stage;
  if (x->stage && count > kShipMaxTables)   // nothing launched yet: take the call number back
    return pipeline_abort(pl, fail(FWD_EB_ETOOBIG, "shipping takes at most %d tables per rank and step (got %d)",
                                   kShipMaxTables, count));
  // The step's launches are independent of each other (one table each): they are spread over
  // the caller's stream and the auxiliary streams, which start where the caller's stream stands
  // now and are joined before the hand-over, so that a grid of one or two waves runs beside
  // another's ramp and tail, and local stores beside peer stores.  Pushes leave the caller's
  // stream only when the flag is raised behind the step (with tickets the last push grid raises
  // it, and must be the last to complete) and there are no replicated tables to fill the other
  // streams with (config 4 on two GPUs, 4 pushes + 18 replicated tables per rank: 595 us per step
  // with the pushes kept together, 603 us spread; 13 pushes and nothing else: 651 against 734).
  const bool spread_pushes = x->tickets == nullptr && local_count == 0;
  const int jobs = (spread_pushes ? count : 0) + local_count;
  int aux = (jobs > 1 || (jobs == 1 && count > 0 && !spread_pushes)) ? pl->local_streams : 0;
  if (aux > jobs) aux = jobs;
  if (aux > 0) {
    cudaError_t e = cudaEventRecord(pl->fork, main);
    for (int k = 0; k < aux && e == cudaSuccess; ++k) e = cudaStreamWaitEvent(pl->aux[k], pl->fork, 0);
    if (e != cudaSuccess) return pipeline_abort(pl, cuda_fail(e, "forking the auxiliary streams"));
  }
  int next = 0;   // round robin over the caller's stream (lane 0) and the auxiliary ones
  // replicated tables stay off the caller's stream while it carries this rank's pushes
  const bool main_is_busy = !spread_pushes && count > 0;
  auto lane_stream = [&](bool may_leave_main) -> cudaStream_t {
    if (!may_leave_main || aux == 0) return main;
    if (main_is_busy) return pl->aux[next++ % aux];
    const int lane = next++ % (aux + 1);
    return lane == 0 ? main : pl->aux[lane - 1];
  };
  int64_t batch = 0;
  for (int i = 0; i < count; ++i) {
    x->table_index = table_index[i];
    x->stage_tables = count;
    x->stage_slot = i;
    if (params[i] && params[i]->num_bags > batch) batch = params[i]->num_bags;
    x->raise_from_push = (from_push && i == count - 1) ? 1 : 0;   // the step's last grid raises the flag
    rc = fwd_eb_shard_push(params[i], x, lane_stream(spread_pushes));
    if (rc) return i == 0 ? pipeline_abort(pl, rc) : rc;   // nothing launched yet: take the number back
  }
  x->raise_from_push = from_push ? 1 : 0;
  for (int i = 0; i < local_count; ++i) {
    x->table_index = local_table_index[i];
    rc = fwd_eb_shard_pool_local(local_params[i], x, lane_stream(true));
    if (rc) return (count == 0 && i == 0) ? pipeline_abort(pl, rc) : rc;   // nothing launched yet
  }
  for (int k = 0; k < aux; ++k) {
    cudaError_t e = cudaEventRecord(pl->joined[k], pl->aux[k]);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(main, pl->joined[k], 0);
    if (e != cudaSuccess) return cuda_fail(e, "joining the auxiliary streams");
  }
  if (!from_push) {
    rc = pipeline_handover(pl, main);
    if (rc) return rc;
  }
  if (x->stage && count > 0) {   // the staged rows go to their owners from the side stream
    rc = fwd_eb_shard_ship(x, dim, batch, table_index, pl->side);
    if (rc) return rc;
  }
  rc = fwd_eb_shard_wait(x, dim, d_result, pl->side);
  if (rc) return rc;
  cudaError_t e = cudaEventRecord(pl->done[pl->epoch % FWD_EB_SHARD_BUFFERS], pl->side);
  if (e != cudaSuccess) return cuda_fail(e, "cudaEventRecord (side)");
  return 0;
}

int fwd_eb_pipeline_step_tablewise(fwd_eb_pipeline* pl, const fwd_eb_params* const* params,
                                   const int32_t* table_index, int32_t count,
                                   fwd_eb_shard_exchange* x, int32_t dim, void* main_stream,
                                   void** d_result) {
  return fwd_eb_pipeline_step_tablewise_hybrid(pl, params, table_index, count, nullptr, nullptr, 0, x, dim,
                                               main_stream, d_result);
}

int fwd_eb_pipeline_sync_result(fwd_eb_pipeline* pl, void* stream) {
  if (!pl) return fail(FWD_EB_EINVAL, "null pipeline");
  if (pl->epoch == 0) return 0;
  cudaError_t e = cudaStreamWaitEvent(static_cast<cudaStream_t>(stream),
                                      pl->done[pl->epoch % FWD_EB_SHARD_BUFFERS], 0);
  if (e != cudaSuccess) return cuda_fail(e, "cudaStreamWaitEvent (result)");
  return 0;
}

int fwd_eb_pipeline_drain(fwd_eb_pipeline* pl) {
  if (!pl) return fail(FWD_EB_EINVAL, "null pipeline");
  cudaError_t e = cudaStreamSynchronize(pl->side);
  if (e != cudaSuccess) return cuda_fail(e, "draining the side stream");
  return 0;
}

// ---- CUDA IPC ----------------------------------------------------------------------------------

int fwd_eb_ipc_alloc(size_t bytes, void** d_ptr, unsigned char handle[FWD_EB_IPC_HANDLE_BYTES]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == FWD_EB_IPC_HANDLE_BYTES, "handle size");
  if (!d_ptr || !handle || bytes == 0) return fail(FWD_EB_EINVAL, "bad ipc_alloc arguments");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc (ipc)");
  e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) {
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, p);
    if (e == cudaSuccess) memcpy(handle, &h, sizeof(h));
  }
  if (e != cudaSuccess) {
    cudaFree(p);
    return cuda_fail(e, "cudaIpcGetMemHandle");
  }
  *d_ptr = p;
  return 0;
}

int fwd_eb_ipc_open(const unsigned char handle[FWD_EB_IPC_HANDLE_BYTES], void** d_peer_ptr) {
  if (!handle || !d_peer_ptr) return fail(FWD_EB_EINVAL, "bad ipc_open arguments");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(d_peer_ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return cuda_fail(e, "cudaIpcOpenMemHandle");
  return 0;
}

int fwd_eb_ipc_close(void* d_peer_ptr) {
  cudaError_t e = cudaIpcCloseMemHandle(d_peer_ptr);
  if (e != cudaSuccess) return cuda_fail(e, "cudaIpcCloseMemHandle");
  return 0;
}

int fwd_eb_ipc_free(void* d_ptr) {
  cudaError_t e = cudaFree(d_ptr);
  if (e != cudaSuccess) return cuda_fail(e, "cudaFree (ipc)");
  return 0;
}

}  // extern "C"
