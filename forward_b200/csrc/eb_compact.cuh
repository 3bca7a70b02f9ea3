// Window compaction: the filter of the reference's bag loop
// (source/trt_engine/trt_network_crt/plugins/embedding_bag_plugin/embedding_bag_plugin.cu:94,
// `data_offset <= index < data_offset + count`) taken out of the pooling kernel and run once,
// as a coalesced streaming pass over the index array.
//
// A rank that holds one row window of a sharded table finds only a fraction of a batch's
// indices inside its window.  Filtering inside the pooling loop makes every lane group read
// and test all of a bag's indices to find its few rows: latency-bound work that does not
// shrink with the window.  Here one warp takes a run of 16 consecutive bags — whose indices
// are consecutive in memory — reads them 32 at a time (several blocks in flight), votes, and
// writes the surviving indices, as local row numbers, densely from the run's own first
// position in a second array.  Within a run the surviving sub-bags are therefore back to back
// and in bag order; the hole is at the run's end.  Each lane also notes how many survivors lie
// before the start of "its" bag of the run, which gives the sub-bags' {start, end} pairs; the
// pooling kernels read those pairs instead of offsets.
#pragma once

#include <type_traits>

#include "eb_kernels.cuh"

namespace fwd_eb {

struct CompactArgs {
  const void* indices;      // [num_indices] int32 or int64
  const void* offsets;      // [num_bags] (+1 with include_last), same type
  const float* psw;         // optional per-sample weights
  long long num_indices;
  long long num_bags;
  long long row_lo;
  long long num_rows;
  long long padding_idx;
  int fixed_len;
  int idx64;
  int include_last;
  int* kept;                // [num_indices] local row numbers of the survivors
  float* kept_w;            // [num_indices] their weights (when psw is given)
  int* bounds;              // [num_bags][2] {start, end} of every sub-bag inside `kept`
  int* counts;              // optional [num_bags]: non-padding entries of the whole bag (mean's divisor)
};

constexpr int kCompactRun = 16;     // bags per warp; sub-bags of a run are contiguous in `kept`
constexpr int kCompactUnroll = 8;   // index blocks (of 32 positions) in flight per warp

// TI = int (32-bit indices and offsets: the whole filter in 32-bit arithmetic, as in
// pool_range) or long long.
// The common case (32-bit indices, no weights) is compiled for 16 resident CTAs per SM (32
// registers): 8192 warps of config 5's batch then run as one wave instead of one and a half.
template <typename TI, bool WEIGHTED>
__global__ void __launch_bounds__(kCtaThreads, (sizeof(TI) == 4 && !WEIGHTED) ? 16 : 10)
eb_window_compact_kernel(const CompactArgs c) {
  const unsigned lane = threadIdx.x & 31u;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long b0 = warp * kCompactRun;
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (b0 >= c.num_bags) return;
  const long long left = c.num_bags - b0;
  const int nb = left < kCompactRun ? (int)left : kCompactRun;
  const int n_idx = (int)c.num_indices;  // checked on the host: below 2^31
  const TI* __restrict__ indices = reinterpret_cast<const TI*>(c.indices);
  const TI* __restrict__ offsets = reinterpret_cast<const TI*>(c.offsets);

  // this lane's bag of the run (lanes nb.. hold an empty bag at the run's end)
  int s = 0, e = 0;
  if ((int)lane < nb) {
    const long long b = b0 + lane;
    if (c.fixed_len > 0) {
      s = (int)b * c.fixed_len;
      e = s + c.fixed_len;
    } else {
      s = (int)__ldg(offsets + b);
      e = (c.include_last || b + 1 < c.num_bags) ? (int)__ldg(offsets + b + 1) : n_idx;
    }
    s = s < 0 ? 0 : (s > n_idx ? n_idx : s);
    e = e < s ? s : (e > n_idx ? n_idx : e);
  }
  const int p0 = __shfl_sync(kFull, s, 0);
  int p1 = __shfl_sync(kFull, e, nb - 1);
  if (p1 < p0) p1 = p0;

  // the filter's constants in the index type
  const TI pad = (TI)c.padding_idx;
  const bool pad_on = c.padding_idx >= 0 && (long long)pad == c.padding_idx;
  const TI row_lo = (TI)c.row_lo;
  // (idx - row_lo) compared unsigned covers both ends of the window; a window that starts
  // outside the index type's range holds no index at all
  using TU = typename std::conditional<sizeof(TI) == 4, unsigned, unsigned long long>::type;
  const TU nrows = ((long long)row_lo == c.row_lo) ? (TU)c.num_rows : (TU)0;

  // Per-bag bookkeeping by prefix: K(p) = survivors among positions [p0, p).  Lane j needs K at
  // the start of its bag; bags are back to back, so its bag's survivors are K(next start) - K(own
  // start), taken from lane j+1 (the run's total for the last bag).  K(s) is known while the
  // block that holds position s is processed: survivors before the block + those below s in it.
  const unsigned lt = (1u << lane) - 1u;
  int carry = 0;    // survivors of the run so far
  int ccarry = 0;   // non-padding entries of the run so far
  int k_start = 0;  // K at this lane's bag start
  int c_start = 0;  // the same for non-padding entries
  for (int base = p0; base < p1; base += 32 * kCompactUnroll) {
    TI idx[kCompactUnroll];
    float w[WEIGHTED ? kCompactUnroll : 1];
#pragma unroll
    for (int k = 0; k < kCompactUnroll; ++k) {
      const int pos = base + 32 * k + (int)lane;
      idx[k] = 0;
      if (WEIGHTED) w[k] = 0.0f;
      if (pos < p1) {
        idx[k] = __ldg(indices + pos);
        if (WEIGHTED) w[k] = __ldg(c.psw + pos);
      }
    }
#pragma unroll
    for (int k = 0; k < kCompactUnroll; ++k) {
      const int bb = base + 32 * k;  // first position of this block
      if (bb >= p1) break;           // warp-uniform
      const int pos = bb + (int)lane;
      const bool counted = pos < p1 && !(pad_on && idx[k] == pad);
      const TU r = (TU)idx[k] - (TU)row_lo;
      const bool keep = counted && r < nrows;
      const unsigned m = __ballot_sync(kFull, keep);
      const unsigned cm = c.counts ? __ballot_sync(kFull, counted) : 0u;  // warp-uniform condition
      if (keep) {
        const int at = p0 + carry + __popc(m & lt);
        c.kept[at] = (int)r;
        if (WEIGHTED) c.kept_w[at] = w[k];
      }
      const unsigned off = (unsigned)(s - bb);  // this lane's bag starts inside the block?
      if (off < 32u) {
        const unsigned below = (1u << off) - 1u;
        k_start = carry + __popc(m & below);
        c_start = ccarry + __popc(cm & below);
      }
      carry += __popc(m);
      ccarry += __popc(cm);
    }
  }
  // a bag that starts at the run's end (an empty tail bag, or lanes past the run) saw no block
  if (s >= p1) {
    k_start = carry;
    c_start = ccarry;
  }
  int k_next = __shfl_down_sync(kFull, k_start, 1);
  int c_next = __shfl_down_sync(kFull, c_start, 1);
  if ((int)lane == nb - 1) {
    k_next = carry;
    c_next = ccarry;
  }
  if ((int)lane < nb) {
    reinterpret_cast<int2*>(c.bounds)[b0 + lane] = make_int2(p0 + k_start, p0 + k_next);
    if (c.counts) c.counts[b0 + lane] = c_next - c_start;
  }
}

}  // namespace fwd_eb
