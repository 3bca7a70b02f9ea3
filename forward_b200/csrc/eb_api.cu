// Host side of the C ABI declared in include/fwd_eb.h: argument checks,
// strategy choice and kernel launches.  No allocation, no synchronisation.
//
// Replaces the launch code of Forward's EmbeddingBag plugin
// (source/trt_engine/trt_network_crt/plugins/embedding_bag_plugin/
// embedding_bag_plugin.cu:182-206) and the rank / op dispatch of
// EmbeddingBagPlugin::enqueue (embedding_bag_plugin.cpp:146-189).
#include <atomic>
#include <climits>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include <cstdlib>
#include <mutex>

#include "eb_compact.cuh"
#include "eb_internal.h"
#include "eb_kernels.cuh"
#include "eb_lite.cuh"
#include "eb_lite_staged.cuh"
#include "eb_stream.cuh"
#include "fwd_eb.h"

namespace fwd_eb {

static thread_local char g_err[512] = "";
static std::atomic<uint64_t> g_launches{0};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  snprintf(g_err, sizeof(g_err), "%s: %s", what, cudaGetErrorString(e));
  return (int)e;
}

void clear_error() { g_err[0] = '\0'; }
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Shape-derived launch plan.
struct Plan {
  PoolArgs a;
  bool vec;      // 16-byte chunks (else one element per chunk)
  int ve;        // elements per chunk
  int cpl;       // chunks per lane: 1, 2 or 4
  int tiles;     // column tiles (grid.y)
  int op;        // Op
  int strategy;  // resolved FWD_EB_STRATEGY_*
  bool table_f16;
};

static int ceil_log2(int x) {
  int l = 0;
  while ((1 << l) < x) ++l;
  return l;
}

// Streaming multiprocessors of the current device, asked once per device ordinal (grid caps
// and the split / run-length heuristics scale with it); 148 (B200) if the query fails.
int sm_count() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  cached[dev].store(n, std::memory_order_relaxed);
  return n;
}

// Split factor for the SPLIT strategy: enough CTAs for about four per SM, no
// slice shorter than 256 indices, at most 64 splits.
static int choose_splits(const fwd_eb_params* p) {
  if (p->num_bags <= 0) return 1;
  long long avg = p->fixed_len > 0 ? p->fixed_len : p->num_indices / p->num_bags;
  long long want = (4LL * sm_count() + p->num_bags - 1) / p->num_bags;
  long long cap = avg / 256;
  if (want > cap) want = cap;
  if (want > 64) want = 64;
  if (want < 1) want = 1;
  return (int)want;
}

static size_t split_workspace_bytes(const fwd_eb_params* p, int splits) {
  if (splits <= 1) return 0;
  size_t slots = (size_t)p->num_bags * (size_t)splits;
  size_t acc = slots * (size_t)p->dim * sizeof(float);
  acc = (acc + 255) & ~(size_t)255;
  return acc + slots * 2 * sizeof(int);
}

static int validate(const fwd_eb_params* p) {
  if (!p) return fail(FWD_EB_EINVAL, "params is null");
  if (p->dim <= 0) return fail(FWD_EB_EINVAL, "dim must be positive (got %d)", p->dim);
  if (p->num_rows < 0 || p->num_indices < 0 || p->num_bags < 0)
    return fail(FWD_EB_EINVAL, "negative size");
  if (p->num_rows > INT_MAX)
    return fail(FWD_EB_ETOOBIG, "num_rows per device is limited to 2^31-1 (got %lld)",
                (long long)p->num_rows);
  if (p->table_dtype != FWD_EB_F32 && p->table_dtype != FWD_EB_F16)
    return fail(FWD_EB_EINVAL, "unknown table_dtype %d", p->table_dtype);
  if (p->out_dtype == FWD_EB_F32_POS) {
    if (p->mode != FWD_EB_MODE_MAX)
      return fail(FWD_EB_EINVAL, "out_dtype FWD_EB_F32_POS is defined for MODE_MAX only");
    if (p->strategy != FWD_EB_STRATEGY_AUTO && p->strategy != FWD_EB_STRATEGY_GROUP)
      return fail(FWD_EB_EUNSUPPORTED, "max with positions runs with the GROUP strategy only");
    if (reinterpret_cast<uintptr_t>(p->out) & 7u)
      return fail(FWD_EB_EALIGN, "FWD_EB_F32_POS output must be 8-byte aligned");
  } else if (p->out_dtype != FWD_EB_F32 && p->out_dtype != FWD_EB_F16) {
    return fail(FWD_EB_EINVAL, "unknown out_dtype %d", p->out_dtype);
  }
  if (p->index_dtype != FWD_EB_I32 && p->index_dtype != FWD_EB_I64)
    return fail(FWD_EB_EINVAL, "unknown index_dtype %d", p->index_dtype);
  switch (p->mode) {
    case FWD_EB_MODE_SUM:
    case FWD_EB_MODE_MEAN:
    case FWD_EB_MODE_MAX:
    case FWD_EB_MODE_SQUARE_SUM:
    case FWD_EB_MODE_GATHER:
      break;
    default:
      return fail(FWD_EB_EINVAL, "unknown mode %d", p->mode);
  }
  if (p->num_rows > 0 && !p->table) return fail(FWD_EB_EINVAL, "table is null");
  if (p->num_indices > 0 && !p->indices) return fail(FWD_EB_EINVAL, "indices is null");
  if (p->table_stride != 0 && p->table_stride < p->dim)
    return fail(FWD_EB_EINVAL, "table_stride smaller than dim");
  if (p->out_stride != 0 && p->out_stride < p->dim)
    return fail(FWD_EB_EINVAL, "out_stride smaller than dim");
  if (p->fixed_len < 0) return fail(FWD_EB_EINVAL, "fixed_len is negative");
  if (p->mode == FWD_EB_MODE_GATHER) {
    if (p->num_indices > 0 && !p->out) return fail(FWD_EB_EINVAL, "out is null");
    if (p->per_sample_weights)
      return fail(FWD_EB_EINVAL, "per_sample_weights are not defined for GATHER");
    return 0;
  }
  if (p->num_bags > 0 && !p->out) return fail(FWD_EB_EINVAL, "out is null");
  if (p->fixed_len > 0) {
    if (p->num_indices != p->num_bags * (int64_t)p->fixed_len)
      return fail(FWD_EB_EINVAL, "num_indices (%lld) != num_bags (%lld) * fixed_len (%d)",
                  (long long)p->num_indices, (long long)p->num_bags, p->fixed_len);
  } else if (p->num_bags > 0 && !p->offsets) {
    return fail(FWD_EB_EINVAL, "offsets is null and fixed_len is 0");
  }
  if (p->per_sample_weights && p->mode != FWD_EB_MODE_SUM)
    return fail(FWD_EB_EINVAL, "per_sample_weights need mode SUM (torch rule)");
  if (p->strategy < FWD_EB_STRATEGY_AUTO || p->strategy > FWD_EB_STRATEGY_LITE)
    return fail(FWD_EB_EINVAL, "unknown strategy %d", p->strategy);
  if (p->flags & FWD_EB_FLAG_OFFSET_PAIRS) {
    if (p->fixed_len > 0) return fail(FWD_EB_EINVAL, "offset pairs and fixed_len exclude each other");
    if (p->strategy == FWD_EB_STRATEGY_CTA || p->strategy == FWD_EB_STRATEGY_SPLIT)
      return fail(FWD_EB_EUNSUPPORTED, "offset pairs run with the GROUP and STREAM strategies");
  }
  return 0;
}

static int pick_strategy(const fwd_eb_params* p) {
  if (p->strategy != FWD_EB_STRATEGY_AUTO) return p->strategy;
  if (p->num_bags <= 0) return FWD_EB_STRATEGY_GROUP;
  const long long avg = p->fixed_len > 0 ? p->fixed_len : p->num_indices / p->num_bags;
  // Many bags, or bags too short to share: a lane group each keeps enough rows in flight.
  if (avg < 64 || p->num_bags >= 8192) return FWD_EB_STRATEGY_GROUP;
  // Few long bags: split them when scratch is on offer and a CTA per bag would leave SMs idle.
  if (p->num_bags < 2 * sm_count() && avg >= 1024) {
    int splits = choose_splits(p);
    if (splits > 1 && p->workspace && p->workspace_bytes >= split_workspace_bytes(p, splits))
      return FWD_EB_STRATEGY_SPLIT;
  }
  return FWD_EB_STRATEGY_CTA;
}

// Shapes the streaming kernel covers (see eb_stream.cuh).
static bool stream_ok(const fwd_eb_params* p, const Plan* pl) {
  return pl->vec && pl->cpl == 1 && pl->tiles == 1 && pl->a.lanes_log2 >= 3 &&
         p->index_dtype == FWD_EB_I32 && p->num_indices <= INT_MAX && p->num_bags <= INT_MAX &&
         p->mode != FWD_EB_MODE_GATHER && p->out_dtype != FWD_EB_F32_POS;
}

// Consecutive bags per lane group: about a hundred rows per run, so the start-up chain
// (bounds, first index block, first rows) is paid once per run instead of once per bag, but
// never so many that the grid falls below two waves of resident groups.  With offset pairs a
// run must stay inside one aligned block of 16 bags (a power of two), and only when the caller
// vouches for their contiguity.
static int choose_stream_k(const fwd_eb_params* p, int lanes_log2) {
  if (p->num_bags <= 0) return 1;
  const bool pairs = (p->flags & FWD_EB_FLAG_OFFSET_PAIRS) != 0;
  if (pairs && !(p->flags & FWD_EB_FLAG_PAIRS_RUN16)) return 1;
  long long avg = p->fixed_len > 0 ? p->fixed_len : p->num_indices / p->num_bags;
  if (avg < 1) avg = 1;
  long long k = 96 / avg;
  if (k > kStreamMaxK) k = kStreamMaxK;
  if (k < 1) k = 1;
  const long long slots = (long long)sm_count() * ((FWD_EB_STREAM_MIN_CTAS * kCtaThreads) >> lanes_log2);
  while (k > 1 && (p->num_bags + k - 1) / k < 2 * slots) --k;
#ifdef FWD_EB_TUNE
  if (const char* e = getenv("FWD_EB_STREAM_K")) k = atoi(e) > 0 ? atoi(e) : k;
  if (k > kStreamMaxK) k = kStreamMaxK;
#endif
  if (pairs) {
    long long p2 = 1;
    while (p2 * 2 <= k) p2 *= 2;
    k = p2;
  }
  return (int)k;
}

static int make_plan(const fwd_eb_params* p, Plan* pl) {
  int rc = validate(p);
  if (rc) return rc;
  memset(pl, 0, sizeof(*pl));
  PoolArgs& a = pl->a;
  const int tsize = p->table_dtype == FWD_EB_F16 ? 2 : 4;
  const int osize = p->out_dtype == FWD_EB_F16 ? 2 : 4;
  const long long tstride = p->table_stride ? p->table_stride : p->dim;
  const long long ostride = p->out_stride ? p->out_stride : p->dim;
  pl->table_f16 = p->table_dtype == FWD_EB_F16;

  const long long row_bytes = (long long)p->dim * tsize;
  pl->vec = (row_bytes % 16 == 0) && ((tstride * tsize) % 16 == 0) && aligned16(p->table);
  pl->ve = pl->vec ? 16 / tsize : 1;
  a.nchunks = pl->vec ? (int)(row_bytes / 16) : p->dim;
  a.lanes_log2 = ceil_log2(a.nchunks < 32 ? a.nchunks : 32);
#ifdef FWD_EB_TUNE_HALFWARP
  if (pl->vec && a.nchunks == 32 && p->mode != FWD_EB_MODE_GATHER &&
      p->num_bags * 32 < (long long)sm_count() * 2048)
    a.lanes_log2 = 4;
#endif
  const int lanes = 1 << a.lanes_log2;
  const int per_lane = (a.nchunks + lanes - 1) / lanes;
  if (pl->vec) {
    pl->cpl = per_lane <= 1 ? 1 : (per_lane <= 2 ? 2 : 4);
  } else {
    pl->cpl = 4;
  }
  const int tile_chunks = pl->cpl * lanes;
  pl->tiles = (a.nchunks + tile_chunks - 1) / tile_chunks;

  a.table = static_cast<const char*>(p->table);
  if (tstride * tsize > 0xffffffffLL)
    return fail(FWD_EB_ETOOBIG, "table row stride must stay below 4 GiB");
  a.row_bytes_stride = tstride * tsize;
  a.num_rows = p->num_rows;
  a.row_lo = p->row_lo;
  a.indices = p->indices;
  a.offsets = p->offsets;
  a.num_indices = p->num_indices;
  a.num_bags = p->num_bags;
  a.psw = p->per_sample_weights;
  a.padding_idx = p->padding_idx;
  a.out = static_cast<char*>(p->out);
  a.out_stride = ostride;
  a.dim = p->dim;
  a.fixed_len = p->fixed_len;
  a.idx64 = p->index_dtype == FWD_EB_I64;
  a.include_last = p->include_last_offset != 0;
  a.out_f16 = p->out_dtype == FWD_EB_F16;
  a.out_vec = pl->vec && aligned16(p->out) && ((ostride * osize) % 16 == 0);
  a.mean = p->mode == FWD_EB_MODE_MEAN;
  a.mean_raw_len = (p->flags & FWD_EB_FLAG_MEAN_RAW_LENGTH) != 0;
  a.mean_double_round = (p->flags & FWD_EB_FLAG_MEAN_SINGLE_ROUNDING) == 0;
  a.splits = 1;
  a.pairs = (p->flags & FWD_EB_FLAG_OFFSET_PAIRS) != 0;
  a.stream_k = 1;
  // 32-bit filter constants for int32 indices
  a.lo32 = (unsigned)p->row_lo;
  // (idx - row_lo) in wrap-around 32-bit arithmetic is exact whenever row_lo itself fits an int;
  // a window starting beyond the int range cannot contain an int32 index at all
  a.nrows32 = (p->row_lo >= INT_MIN && p->row_lo <= INT_MAX) ? (unsigned)p->num_rows : 0u;
  a.pad32_on = p->padding_idx >= 0 && p->padding_idx <= INT_MAX;
  a.pad32 = a.pad32_on ? (int)p->padding_idx : 0;

  switch (p->mode) {
    case FWD_EB_MODE_MAX:
      pl->op = kOpMax;
      break;
    case FWD_EB_MODE_SQUARE_SUM:
      pl->op = kOpSquareSum;
      break;
    default:
      pl->op = p->per_sample_weights ? kOpWeighted : kOpSum;
  }

  if (p->mode == FWD_EB_MODE_GATHER) {
    pl->strategy = FWD_EB_STRATEGY_GROUP;
    return 0;
  }
  if (p->out_dtype == FWD_EB_F32_POS) {
    pl->strategy = FWD_EB_STRATEGY_GROUP;
    return 0;
  }
  pl->strategy = pick_strategy(p);
  if (a.pairs && pl->strategy != FWD_EB_STRATEGY_STREAM && pl->strategy != FWD_EB_STRATEGY_LITE)
    pl->strategy = FWD_EB_STRATEGY_GROUP;
  // AUTO: where a lane group per bag is the plan and the shape allows, the lean kernel runs it.
  // Measured on B200 (us per call, group / stream / lite): 16384 bags of ~40 rows of 256 B, Zipf
  // 23.0 / 28.0 / 19.5, uniform 29.4 / 34.4 / 27.5; 8192 bags of 0..64 rows of 512 B (max, 5 %
  // padding) 33.8 / 32.5 / 28.8; 131072 dense bags of ~6 rows of 128 B 42.7 / 43.2 / 32.6; fixed
  // length, uniform indices over 4 M rows: 65536 x 20 weighted fp32 rows of 512 B 117.1 / 111.3 /
  // 105.9; 262144 x 8 fp16 rows of 128 B 66.5 / 60.8 / 48.5; 131072 x 6 fp16 rows of 512 B 215.3 /
  // 101.5 / 78.8; 262144 x 4 fp32 rows of 128 B 44.2 / 33.4 / 31.1.  The streaming kernel stays
  // available by name (FWD_EB_STRATEGY_STREAM).
  // A table window that starts above row 0 says "one shard of a larger table": most indices
  // will then miss the window, and both lean kernels spend a load slot on every index, kept or
  // not, where the group kernel's survivor ring does not (142 against 80 us on a 1-in-8 window).
  // Such calls stay with the group kernel unless the indices were compacted first.
  if (p->strategy == FWD_EB_STRATEGY_AUTO && pl->strategy == FWD_EB_STRATEGY_GROUP &&
      stream_ok(p, pl) && (a.pairs || p->row_lo == 0))
    pl->strategy = FWD_EB_STRATEGY_LITE;
  if (pl->strategy == FWD_EB_STRATEGY_LITE && !stream_ok(p, pl))
    return fail(FWD_EB_EUNSUPPORTED, "LITE needs 16-byte aligned rows of 128..512 bytes, int32 "
                "indices and fewer than 2^31 of them");
  if (pl->strategy == FWD_EB_STRATEGY_STREAM) {
    if (!stream_ok(p, pl)) {
      if (p->strategy == FWD_EB_STRATEGY_STREAM)
        return fail(FWD_EB_EUNSUPPORTED, "STREAM needs 16-byte aligned rows of 128..512 bytes, int32 "
                    "indices and fewer than 2^31 of them");
      pl->strategy = FWD_EB_STRATEGY_GROUP;
    } else {
      a.stream_k = choose_stream_k(p, a.lanes_log2);
    }
  }
  if (pl->strategy == FWD_EB_STRATEGY_SPLIT) {
    int splits = choose_splits(p);
    if (splits <= 1) {
      pl->strategy = FWD_EB_STRATEGY_CTA;
    } else {
      size_t need = split_workspace_bytes(p, splits);
      if (!p->workspace || p->workspace_bytes < need)
        return fail(FWD_EB_EWORKSPACE, "split strategy needs %zu bytes of workspace, got %zu", need,
                    p->workspace ? p->workspace_bytes : (size_t)0);
      if (reinterpret_cast<uintptr_t>(p->workspace) & 255u)
        return fail(FWD_EB_EALIGN, "workspace must be 256-byte aligned");
      a.splits = splits;
      size_t acc = (size_t)p->num_bags * splits * p->dim * sizeof(float);
      acc = (acc + 255) & ~(size_t)255;
      a.ws_acc = static_cast<float*>(p->workspace);
      a.ws_meta = reinterpret_cast<int*>(static_cast<char*>(p->workspace) + acc);
    }
  }
  return 0;
}

int plan_group(const fwd_eb_params* p, PoolArgs* args, int* vec, int* cpl, int* tiles, int* stream) {
  Plan pl;
  fwd_eb_params q = *p;
  q.strategy = FWD_EB_STRATEGY_GROUP;
  int rc = make_plan(&q, &pl);
  if (rc) return rc;
  // the same choice AUTO makes between the lane-group kernels
  int want = 0;
  if (p->strategy == FWD_EB_STRATEGY_STREAM) want = 1;
  else if (p->strategy == FWD_EB_STRATEGY_LITE) want = 2;
  else if (p->strategy == FWD_EB_STRATEGY_AUTO && (pl.a.pairs || p->row_lo == 0))
    want = 2;
  *stream = 0;
  if (want && stream_ok(&q, &pl)) {
    if (want == 1) pl.a.stream_k = choose_stream_k(&q, pl.a.lanes_log2);
    *stream = want;
  }
  *args = pl.a;
  *vec = pl.vec ? 1 : 0;
  *cpl = pl.cpl;
  *tiles = pl.tiles;
  return 0;
}

// ---- kernel dispatch ---------------------------------------------------------

template <typename TW, int VE, int LL, int OP>
static cudaError_t launch_stream_ll(const Plan& pl, cudaStream_t st) {
  const PoolArgs& a = pl.a;
  const long long groups = (a.num_bags + a.stream_k - 1) / a.stream_k;
  const long long threads = groups << LL;
  const long long blocks = (threads + kCtaThreads - 1) / kCtaThreads;
  if (blocks == 0) return cudaSuccess;
  if (blocks > INT_MAX) return cudaErrorInvalidConfiguration;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3((unsigned)kCtaThreads);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  PushArgs none;
  memset(&none, 0, sizeof(none));
  cudaError_t le = cudaLaunchKernelEx(
      &cfg, eb_pool_stream_kernel<TW, VE, LL, OP, stream_u(LL), false>, a, none);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return le != cudaSuccess ? le : cudaGetLastError();
}

// CTA size of the lean kernel (the kernel reads blockDim.x).
static int lite_cta_threads(int lanes_log2) {
  (void)lanes_log2;
  return kCtaThreads;
}

template <typename TW, int VE, int LL, int OP>
static cudaError_t launch_lite_ll(const Plan& pl, cudaStream_t st) {
  const PoolArgs& a = pl.a;
  int cta = lite_cta_threads(LL);
#ifdef FWD_EB_TUNE
  if (const char* env = getenv("FWD_EB_LITE_CTA")) cta = atoi(env) >= 32 ? atoi(env) : cta;
#endif
  const long long blocks = ((a.num_bags << LL) + cta - 1) / cta;
  if (blocks == 0) return cudaSuccess;
  if (blocks > INT_MAX) return cudaErrorInvalidConfiguration;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3((unsigned)cta);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
#if defined(FWD_EB_ROW_STAGING) && FWD_EB_ROW_STAGING > 0
  // experiment build: rows staged through shared memory (eb_lite_staged.cuh)
  cudaError_t le = cudaLaunchKernelEx(&cfg, eb_pool_lite_staged_kernel<TW, VE, LL, OP>, a);
#else
  PushArgs none;
  memset(&none, 0, sizeof(none));
  cudaError_t le = cudaLaunchKernelEx(&cfg, eb_pool_lite_kernel<TW, VE, LL, OP, false>, a, none);
#endif
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return le != cudaSuccess ? le : cudaGetLastError();
}

template <typename TW, int OP>
static cudaError_t launch_lite_op(const Plan& pl, cudaStream_t st) {
  constexpr int VE = 16 / (int)sizeof(TW);
  switch (pl.a.lanes_log2) {
    case 3:
      return launch_lite_ll<TW, VE, 3, OP>(pl, st);
    case 4:
      return launch_lite_ll<TW, VE, 4, OP>(pl, st);
    default:
      return launch_lite_ll<TW, VE, 5, OP>(pl, st);
  }
}

template <typename TW>
static cudaError_t launch_lite(const Plan& pl, cudaStream_t st) {
  switch (pl.op) {
    case kOpSum:
      return launch_lite_op<TW, kOpSum>(pl, st);
    case kOpWeighted:
      return launch_lite_op<TW, kOpWeighted>(pl, st);
    case kOpMax:
      return launch_lite_op<TW, kOpMax>(pl, st);
    default:
      return launch_lite_op<TW, kOpSquareSum>(pl, st);
  }
}

template <typename TW, int OP>
static cudaError_t launch_stream_op(const Plan& pl, cudaStream_t st) {
  constexpr int VE = 16 / (int)sizeof(TW);
  switch (pl.a.lanes_log2) {
    case 3:
      return launch_stream_ll<TW, VE, 3, OP>(pl, st);
    case 4:
      return launch_stream_ll<TW, VE, 4, OP>(pl, st);
    default:
      return launch_stream_ll<TW, VE, 5, OP>(pl, st);
  }
}

template <typename TW>
static cudaError_t launch_stream(const Plan& pl, cudaStream_t st) {
  switch (pl.op) {
    case kOpSum:
      return launch_stream_op<TW, kOpSum>(pl, st);
    case kOpWeighted:
      return launch_stream_op<TW, kOpWeighted>(pl, st);
    case kOpMax:
      return launch_stream_op<TW, kOpMax>(pl, st);
    default:
      return launch_stream_op<TW, kOpSquareSum>(pl, st);
  }
}

template <typename TW, int VE, int CPL, int OP, int U, int IPL>
static cudaError_t launch_pool(const Plan& pl, cudaStream_t st) {
  const PoolArgs& a = pl.a;
  if (pl.strategy == FWD_EB_STRATEGY_GROUP) {
    const long long threads = a.num_bags << a.lanes_log2;
    const int cta = group_cta_threads(a.lanes_log2);
    const long long blocks = (threads + cta - 1) / cta;
    if (blocks == 0) return cudaSuccess;
    if (blocks > INT_MAX) return cudaErrorInvalidConfiguration;
    dim3 grid((unsigned)blocks, (unsigned)pl.tiles);
    // Programmatic stream serialization: when the launch ahead of this one on the stream is
    // also a pooling grid, this grid's CTAs take their places while that grid's last CTAs
    // drain (they wait in griddepcontrol.wait before touching memory) — 1.6-2 us per call of
    // back-to-back pooling.  After any other kind of work it is an ordinary launch.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3((unsigned)cta);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t le = cudaLaunchKernelEx(&cfg, eb_pool_group_kernel<TW, VE, CPL, OP, U, IPL>, a);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return le != cudaSuccess ? le : cudaGetLastError();
  }
  const long long blocks = a.num_bags * a.splits;
  if (blocks == 0) return cudaSuccess;
  if (blocks > INT_MAX) return cudaErrorInvalidConfiguration;
  const int groups = kCtaThreads >> a.lanes_log2;
  const size_t smem = (size_t)kCtaThreads * CPL * VE * sizeof(float) + (size_t)groups * 2 * sizeof(int);
  dim3 grid((unsigned)blocks, (unsigned)pl.tiles);
  eb_pool_cta_kernel<TW, VE, CPL, OP, U, IPL><<<grid, kCtaThreads, smem, st>>>(a);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess || a.splits <= 1) return e;
  const long long total = a.num_bags * a.dim;
  const long long fblocks = (total + kCtaThreads - 1) / kCtaThreads;
  if (fblocks > INT_MAX) return cudaErrorInvalidConfiguration;
  eb_split_finish_kernel<OP><<<(unsigned)fblocks, kCtaThreads, 0, st>>>(a, pl.table_f16 ? 1 : 0);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

template <typename TW, int VE, int CPL, int U, int IPL>
static cudaError_t launch_op(const Plan& pl, cudaStream_t st) {
  switch (pl.op) {
    case kOpSum:
      return launch_pool<TW, VE, CPL, kOpSum, U, IPL>(pl, st);
    case kOpWeighted:
      return launch_pool<TW, VE, CPL, kOpWeighted, U, IPL>(pl, st);
    case kOpMax:
      return launch_pool<TW, VE, CPL, kOpMax, U, IPL>(pl, st);
    default:
      return launch_pool<TW, VE, CPL, kOpSquareSum, U, IPL>(pl, st);
  }
}

// Row loads kept in flight per lane group: FWD_EB_U1 (4) x 16 B for one chunk per lane,
// fewer when a lane owns several chunks so the register count stays put.
template <typename TW>
static cudaError_t launch_shape(const Plan& pl, cudaStream_t st) {
  constexpr int VE = 16 / (int)sizeof(TW);
  if (!pl.vec) return launch_op<TW, 1, 4, 4, 1>(pl, st);
  switch (pl.cpl) {
    case 1:
#ifdef FWD_EB_TUNE
      if (getenv("FWD_EB_IPL1")) return launch_op<TW, VE, 1, FWD_EB_U1, 1>(pl, st);
#endif
      // rows of 256 B / 128 B: blocks of 32 indices (two / four index loads per lane)
      if (pl.a.lanes_log2 == 4) return launch_op<TW, VE, 1, FWD_EB_U1, 2>(pl, st);
      if (pl.a.lanes_log2 == 3) return launch_op<TW, VE, 1, FWD_EB_U1, 4>(pl, st);
      return launch_op<TW, VE, 1, FWD_EB_U1, 1>(pl, st);
    case 2:
      return launch_op<TW, VE, 2, 4, 1>(pl, st);
    default:
      return launch_op<TW, VE, 4, 2, 1>(pl, st);
  }
}

template <typename TW>
static cudaError_t launch_maxpos(const Plan& pl, cudaStream_t st) {
  const PoolArgs& a = pl.a;
  const long long threads = a.num_bags << a.lanes_log2;
  const long long blocks = (threads + kCtaThreads - 1) / kCtaThreads;
  if (blocks == 0) return cudaSuccess;
  if (blocks > INT_MAX) return cudaErrorInvalidConfiguration;
  const int lanes = 1 << a.lanes_log2;
  dim3 grid((unsigned)blocks, (unsigned)((a.nchunks + lanes - 1) / lanes));
  if (pl.vec) {
    eb_pool_maxpos_kernel<TW, 16 / (int)sizeof(TW)><<<grid, kCtaThreads, 0, st>>>(a);
  } else {
    eb_pool_maxpos_kernel<TW, 1><<<grid, kCtaThreads, 0, st>>>(a);
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

template <typename TW>
static cudaError_t launch_gather(const Plan& pl, bool keep, cudaStream_t st) {
  const PoolArgs& a = pl.a;
  const long long threads = a.num_indices << a.lanes_log2;
  const long long blocks = (threads + kCtaThreads - 1) / kCtaThreads;
  if (blocks == 0) return cudaSuccess;
  if (blocks > INT_MAX) return cudaErrorInvalidConfiguration;
  if (pl.vec) {
    eb_gather_kernel<TW, 16 / (int)sizeof(TW)><<<(unsigned)blocks, kCtaThreads, 0, st>>>(a, keep);
  } else {
    eb_gather_kernel<TW, 1><<<(unsigned)blocks, kCtaThreads, 0, st>>>(a, keep);
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

}  // namespace fwd_eb

using namespace fwd_eb;

extern "C" {

int fwd_eb_version(void) { return FWD_EB_ABI_VERSION; }

size_t fwd_eb_params_size(void) { return sizeof(fwd_eb_params); }

const char* fwd_eb_last_error_string(void) { return g_err; }

uint64_t fwd_eb_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int fwd_eb_pick_strategy(const fwd_eb_params* p) {
  if (!p) return fail(FWD_EB_EINVAL, "params is null");
  fwd_eb_params q = *p;
  if (q.strategy == FWD_EB_STRATEGY_SPLIT) q.strategy = FWD_EB_STRATEGY_AUTO;
  Plan pl;
  int rc = make_plan(&q, &pl);
  if (rc) return rc;
  return pl.strategy;
}

size_t fwd_eb_workspace_size(const fwd_eb_params* p) {
  if (!p || validate(p) != 0 || p->mode == FWD_EB_MODE_GATHER) return 0;
  if (p->strategy == FWD_EB_STRATEGY_GROUP || p->strategy == FWD_EB_STRATEGY_CTA ||
      p->strategy == FWD_EB_STRATEGY_STREAM || p->strategy == FWD_EB_STRATEGY_LITE)
    return 0;
  // AUTO: what SPLIT would need if AUTO could choose it for this shape.
  if (p->strategy == FWD_EB_STRATEGY_AUTO) {
    if (p->num_bags <= 0) return 0;
    const long long avg = p->fixed_len > 0 ? p->fixed_len : p->num_indices / p->num_bags;
    if (avg < 64 || p->num_bags >= 8192) return 0;
    if (!(p->num_bags < 2 * sm_count() && avg >= 1024)) return 0;
  }
  return split_workspace_bytes(p, choose_splits(p));
}

int fwd_eb_forward(const fwd_eb_params* p, void* stream) {
  NvtxRange range("fwd_eb_forward");
  Plan pl;
  int rc = make_plan(p, &pl);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (p->mode == FWD_EB_MODE_GATHER) {
    const bool keep = (p->flags & FWD_EB_FLAG_GATHER_KEEP_SKIPPED) != 0;
    e = pl.table_f16 ? launch_gather<__half>(pl, keep, st) : launch_gather<float>(pl, keep, st);
  } else if (p->out_dtype == FWD_EB_F32_POS) {
    e = pl.table_f16 ? launch_maxpos<__half>(pl, st) : launch_maxpos<float>(pl, st);
  } else if (pl.strategy == FWD_EB_STRATEGY_STREAM) {
    e = pl.table_f16 ? launch_stream<__half>(pl, st) : launch_stream<float>(pl, st);
  } else if (pl.strategy == FWD_EB_STRATEGY_LITE) {
    e = pl.table_f16 ? launch_lite<__half>(pl, st) : launch_lite<float>(pl, st);
  } else {
    e = pl.table_f16 ? launch_shape<__half>(pl, st) : launch_shape<float>(pl, st);
  }
  if (e != cudaSuccess) return cuda_fail(e, "kernel launch");
  g_err[0] = '\0';
  return 0;
}

// Auxiliary streams of fwd_eb_forward_many, per GPU, created on first use and kept.
namespace {
struct ManyStreams {
  bool ready = false;
  cudaStream_t aux[FWD_EB_MANY_STREAMS] = {};
  cudaEvent_t fork = nullptr;
  cudaEvent_t joined[FWD_EB_MANY_STREAMS] = {};
};
constexpr int kManyDevices = 64;
std::mutex g_many_lock;
ManyStreams g_many[kManyDevices];
}  // namespace

int fwd_eb_forward_many(const fwd_eb_params* const* params, int32_t count, void* stream) {
  NvtxRange range("fwd_eb_forward_many");
  if (count < 0 || (count > 0 && !params)) return fail(FWD_EB_EINVAL, "bad argument list");
  for (int i = 0; i < count; ++i) {   // everything is checked before anything is launched
    if (!params[i]) return fail(FWD_EB_EINVAL, "params[%d] is null", i);
    Plan pl;
    int rc = make_plan(params[i], &pl);
    if (rc) return rc;
  }
  if (count <= 1) return count == 1 ? fwd_eb_forward(params[0], stream) : 0;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= kManyDevices) {   // no slot for this ordinal: one after the other
    for (int i = 0; i < count; ++i) {
      int rc = fwd_eb_forward(params[i], stream);
      if (rc) return rc;
    }
    return 0;
  }
  std::lock_guard<std::mutex> hold(g_many_lock);
  ManyStreams& m = g_many[dev];
  if (!m.ready) {
    e = cudaEventCreateWithFlags(&m.fork, cudaEventDisableTiming);
    for (int k = 0; k < FWD_EB_MANY_STREAMS && e == cudaSuccess; ++k) {
      e = cudaStreamCreateWithFlags(&m.aux[k], cudaStreamNonBlocking);
      if (e == cudaSuccess) e = cudaEventCreateWithFlags(&m.joined[k], cudaEventDisableTiming);
    }
    if (e != cudaSuccess) return cuda_fail(e, "creating the auxiliary streams");
    m.ready = true;
  }
  cudaStream_t main = static_cast<cudaStream_t>(stream);
  const int aux = count - 1 < FWD_EB_MANY_STREAMS ? count - 1 : FWD_EB_MANY_STREAMS;
  e = cudaEventRecord(m.fork, main);
  for (int k = 0; k < aux && e == cudaSuccess; ++k) e = cudaStreamWaitEvent(m.aux[k], m.fork, 0);
  if (e != cudaSuccess) return cuda_fail(e, "forking the auxiliary streams");
  int rc = 0;
  for (int i = 0; i < count && rc == 0; ++i) {
    const int lane = i % (aux + 1);
    rc = fwd_eb_forward(params[i], lane == 0 ? stream : static_cast<void*>(m.aux[lane - 1]));
  }
  // joined even after a failed launch: `stream` must stay ordered behind what did start
  for (int k = 0; k < aux; ++k) {
    e = cudaEventRecord(m.joined[k], m.aux[k]);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(main, m.joined[k], 0);
    if (e != cudaSuccess && rc == 0) rc = cuda_fail(e, "joining the auxiliary streams");
  }
  return rc;
}

int fwd_eb_compact_window(const fwd_eb_params* p, int32_t* d_kept, float* d_kept_weights,
                          int32_t* d_bounds, int32_t* d_counts, void* stream) {
  NvtxRange range("fwd_eb_compact_window");
  if (!p) return fail(FWD_EB_EINVAL, "params is null");
  if (p->num_rows < 0 || p->num_indices < 0 || p->num_bags < 0) return fail(FWD_EB_EINVAL, "negative size");
  if (p->num_rows > INT_MAX)
    return fail(FWD_EB_ETOOBIG, "num_rows per device is limited to 2^31-1 (got %lld)", (long long)p->num_rows);
  if (p->num_indices > INT_MAX)
    return fail(FWD_EB_ETOOBIG, "window compaction takes fewer than 2^31 indices per call (got %lld)",
                (long long)p->num_indices);
  if (p->index_dtype != FWD_EB_I32 && p->index_dtype != FWD_EB_I64)
    return fail(FWD_EB_EINVAL, "unknown index_dtype %d", p->index_dtype);
  if (p->flags & FWD_EB_FLAG_OFFSET_PAIRS)
    return fail(FWD_EB_EUNSUPPORTED, "window compaction reads plain offsets or fixed_len, not pairs");
  if (p->fixed_len < 0) return fail(FWD_EB_EINVAL, "fixed_len is negative");
  if (p->fixed_len > 0 && p->num_indices != p->num_bags * (int64_t)p->fixed_len)
    return fail(FWD_EB_EINVAL, "num_indices (%lld) != num_bags (%lld) * fixed_len (%d)",
                (long long)p->num_indices, (long long)p->num_bags, p->fixed_len);
  if (p->num_bags == 0) return 0;
  if (p->fixed_len == 0 && !p->offsets) return fail(FWD_EB_EINVAL, "offsets is null and fixed_len is 0");
  if (p->num_indices > 0 && (!p->indices || !d_kept)) return fail(FWD_EB_EINVAL, "indices / d_kept is null");
  if (!d_bounds) return fail(FWD_EB_EINVAL, "d_bounds is null");
  if (reinterpret_cast<uintptr_t>(d_bounds) & 7u) return fail(FWD_EB_EALIGN, "d_bounds must be 8-byte aligned");
  if (p->per_sample_weights && !d_kept_weights)
    return fail(FWD_EB_EINVAL, "per_sample_weights given but d_kept_weights is null");
  CompactArgs c;
  memset(&c, 0, sizeof(c));
  c.indices = p->indices;
  c.offsets = p->offsets;
  c.psw = p->per_sample_weights;
  c.num_indices = p->num_indices;
  c.num_bags = p->num_bags;
  c.row_lo = p->row_lo;
  c.num_rows = p->num_rows;
  c.padding_idx = p->padding_idx;
  c.fixed_len = p->fixed_len;
  c.idx64 = p->index_dtype == FWD_EB_I64;
  c.include_last = p->include_last_offset != 0;
  c.kept = d_kept;
  c.kept_w = d_kept_weights;
  c.bounds = d_bounds;
  c.counts = d_counts;
  const long long warps = (p->num_bags + kCompactRun - 1) / kCompactRun;
  const long long blocks = (warps * 32 + kCtaThreads - 1) / kCtaThreads;
  if (blocks > INT_MAX) return fail(FWD_EB_ETOOBIG, "too many bags for one compaction launch");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3((unsigned)kCtaThreads);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];  // see launch_pool: overlaps its launch with the drain of a pooling grid ahead
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e;
  if (c.psw)
    e = c.idx64 ? cudaLaunchKernelEx(&cfg, eb_window_compact_kernel<long long, true>, c)
                : cudaLaunchKernelEx(&cfg, eb_window_compact_kernel<int, true>, c);
  else
    e = c.idx64 ? cudaLaunchKernelEx(&cfg, eb_window_compact_kernel<long long, false>, c)
                : cudaLaunchKernelEx(&cfg, eb_window_compact_kernel<int, false>, c);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "compaction kernel launch");
  g_err[0] = '\0';
  return 0;
}

// ---- the reference's three launchers, same argument order --------------------

static void legacy_params(fwd_eb_params* p, const int* d_input, float* d_output,
                          const float* d_data, int count, int dim, int data_offset, int op_type) {
  memset(p, 0, sizeof(*p));
  p->table = d_data;
  p->table_dtype = FWD_EB_F32;
  p->dim = dim;
  p->num_rows = count;
  p->row_lo = data_offset;
  p->indices = d_input;
  p->index_dtype = FWD_EB_I32;
  p->mode = op_type;
  p->padding_idx = -1;
  p->out = d_output;
  p->out_dtype = FWD_EB_F32;
}

int fwd_eb_gather_f32(const int* d_input, float* d_output, int batch_size, int offset,
                      const float* d_data, int count, int dim, int data_offset, void* stream) {
  if (batch_size < 0 || offset < 0) return fail(FWD_EB_EINVAL, "negative size");
  fwd_eb_params p;
  legacy_params(&p, d_input, d_output, d_data, count, dim, data_offset, FWD_EB_MODE_GATHER);
  p.num_indices = (int64_t)batch_size * offset;
  return fwd_eb_forward(&p, stream);
}

int fwd_eb_bag_fixed_f32(const int* d_input, float* d_output, int batch_size, int offset,
                         const float* d_data, int count, int dim, int data_offset, int op_type,
                         void* stream) {
  if (batch_size < 0 || offset <= 0) return fail(FWD_EB_EINVAL, "bad batch_size / offset");
  fwd_eb_params p;
  legacy_params(&p, d_input, d_output, d_data, count, dim, data_offset, op_type);
  p.fixed_len = offset;
  p.num_bags = batch_size;
  p.num_indices = (int64_t)batch_size * offset;
  return fwd_eb_forward(&p, stream);
}

int fwd_eb_bag_f32(const int* d_input, const int* d_offsets, float* d_output, int input_size,
                   int block_size, const float* d_data, int count, int dim, int data_offset,
                   int op_type, void* stream) {
  if (input_size < 0 || block_size < 0) return fail(FWD_EB_EINVAL, "negative size");
  fwd_eb_params p;
  legacy_params(&p, d_input, d_output, d_data, count, dim, data_offset, op_type);
  p.offsets = d_offsets;
  p.num_bags = block_size;
  p.num_indices = input_size;
  return fwd_eb_forward(&p, stream);
}

// ---- helpers -----------------------------------------------------------------

int fwd_eb_fill_table(void* d_table, int32_t table_dtype, int64_t num_rows, int32_t dim,
                      int64_t row_lo, uint64_t seed, float scale, void* stream) {
  if (!d_table || num_rows < 0 || dim <= 0) return fail(FWD_EB_EINVAL, "bad table arguments");
  if (table_dtype != FWD_EB_F32 && table_dtype != FWD_EB_F16)
    return fail(FWD_EB_EINVAL, "unknown table_dtype %d", table_dtype);
  if (num_rows == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long total = (long long)num_rows * dim;
  long long blocks = (total + kCtaThreads - 1) / kCtaThreads;
  const long long cap = (long long)sm_count() * 32;
  if (blocks > cap) blocks = cap;
  if (table_dtype == FWD_EB_F16) {
    eb_fill_table_kernel<__half><<<(unsigned)blocks, kCtaThreads, 0, st>>>(
        static_cast<__half*>(d_table), num_rows, dim, row_lo, seed, scale);
  } else {
    eb_fill_table_kernel<float><<<(unsigned)blocks, kCtaThreads, 0, st>>>(
        static_cast<float*>(d_table), num_rows, dim, row_lo, seed, scale);
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "fill_table launch");
  return 0;
}

int fwd_eb_cast_i64_to_i32(const void* d_src, void* d_dst, int64_t count, void* stream) {
  if (count < 0 || (count > 0 && (!d_src || !d_dst))) return fail(FWD_EB_EINVAL, "bad cast arguments");
  if (count == 0) return 0;
  long long blocks = (count + kCtaThreads - 1) / kCtaThreads;
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  eb_cast_i64_i32_kernel<<<(unsigned)blocks, kCtaThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const long long*>(d_src), static_cast<int*>(d_dst), count);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "cast launch");
  return 0;
}

int fwd_eb_combine_partials(const void* d_parts, int32_t part_dtype, int32_t num_parts,
                            int64_t part_stride_elems, int64_t count, void* d_out,
                            int32_t out_dtype, void* stream) {
  if (!d_parts || !d_out || num_parts <= 0 || count < 0 || part_stride_elems < count)
    return fail(FWD_EB_EINVAL, "bad combine arguments");
  if (count == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  long long blocks = (count + kCtaThreads - 1) / kCtaThreads;
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  const unsigned g = (unsigned)blocks;
  if (part_dtype == FWD_EB_F32 && out_dtype == FWD_EB_F32) {
    eb_combine_partials_kernel<float, float><<<g, kCtaThreads, 0, st>>>(
        static_cast<const float*>(d_parts), num_parts, part_stride_elems, count,
        static_cast<float*>(d_out));
  } else if (part_dtype == FWD_EB_F32 && out_dtype == FWD_EB_F16) {
    eb_combine_partials_kernel<float, __half><<<g, kCtaThreads, 0, st>>>(
        static_cast<const float*>(d_parts), num_parts, part_stride_elems, count,
        static_cast<__half*>(d_out));
  } else if (part_dtype == FWD_EB_F16 && out_dtype == FWD_EB_F32) {
    eb_combine_partials_kernel<__half, float><<<g, kCtaThreads, 0, st>>>(
        static_cast<const __half*>(d_parts), num_parts, part_stride_elems, count,
        static_cast<float*>(d_out));
  } else if (part_dtype == FWD_EB_F16 && out_dtype == FWD_EB_F16) {
    eb_combine_partials_kernel<__half, __half><<<g, kCtaThreads, 0, st>>>(
        static_cast<const __half*>(d_parts), num_parts, part_stride_elems, count,
        static_cast<__half*>(d_out));
  } else {
    return fail(FWD_EB_EINVAL, "unknown dtype in combine");
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "combine launch");
  return 0;
}

}  // extern "C"
