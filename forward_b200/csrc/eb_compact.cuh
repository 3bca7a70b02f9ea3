// Window compaction: the filter of the reference's bag loop
// (source/trt_engine/trt_network_crt/plugins/embedding_bag_plugin/embedding_bag_plugin.cu:94,
// `data_offset <= index < data_offset + count`) taken out of the pooling kernel and run once,
// as a coalesced streaming pass over the index array.
//
// A rank that holds one row window of a sharded table finds only a fraction of a batch's
// indices inside its window.  Filtering inside the pooling loop makes every lane group read
// and test all of a bag's indices to find its few rows: latency-bound work that does not
// shrink with the window.  Here one warp takes a run of 32 consecutive bags — whose indices
// are consecutive in memory — reads them 32 at a time (several blocks in flight), votes, and
// writes the surviving indices, as local row numbers, densely from the run's own first
// position in a second array.  Within a run the surviving sub-bags are therefore back to back
// and in bag order; the hole is at the run's end.  Each lane also counts the survivors of "its"
// bag of the run (block overlap x vote mask), a shuffle scan turns the counts into the sub-bags'
// {start, end} pairs, and the pooling kernels read those pairs instead of offsets.
#pragma once

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

constexpr int kCompactRun = 32;     // bags per warp; sub-bags of a run are contiguous in `kept`
constexpr int kCompactUnroll = 4;   // index blocks in flight per warp

__global__ void __launch_bounds__(kCtaThreads)
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

  // this lane's bag of the run
  int s = 0, e = 0;
  if ((int)lane < nb) {
    const long long b = b0 + lane;
    if (c.fixed_len > 0) {
      s = (int)b * c.fixed_len;
      e = s + c.fixed_len;
    } else {
      s = (int)load_index(c.offsets, c.idx64, b);
      e = (c.include_last || b + 1 < c.num_bags) ? (int)load_index(c.offsets, c.idx64, b + 1) : n_idx;
    }
    s = s < 0 ? 0 : (s > n_idx ? n_idx : s);
    e = e < s ? s : (e > n_idx ? n_idx : e);
  }
  const int p0 = __shfl_sync(kFull, s, 0);
  int p1 = __shfl_sync(kFull, e, nb - 1);
  if (p1 < p0) p1 = p0;

  const unsigned lt = (1u << lane) - 1u;
  int carry = 0;         // survivors of the run so far
  int mine = 0;          // survivors of this lane's bag
  int mine_counted = 0;  // non-padding entries of this lane's bag
  for (int base = p0; base < p1; base += 32 * kCompactUnroll) {
    long long idx[kCompactUnroll];
    float w[kCompactUnroll];
#pragma unroll
    for (int k = 0; k < kCompactUnroll; ++k) {
      const int pos = base + 32 * k + (int)lane;
      idx[k] = 0;
      w[k] = 0.0f;
      if (pos < p1) {
        idx[k] = load_index(c.indices, c.idx64, pos);
        if (c.psw) w[k] = __ldg(c.psw + pos);
      }
    }
#pragma unroll
    for (int k = 0; k < kCompactUnroll; ++k) {
      const int bb = base + 32 * k;  // first position of this block
      if (bb >= p1) break;           // warp-uniform
      const int pos = bb + (int)lane;
      const bool counted = pos < p1 && (c.padding_idx < 0 || idx[k] != c.padding_idx);
      const long long r = idx[k] - c.row_lo;
      const bool keep = counted && r >= 0 && r < c.num_rows;
      const unsigned m = __ballot_sync(kFull, keep);
      const unsigned cm = __ballot_sync(kFull, counted);
      if (keep) {
        const int at = p0 + carry + __popc(m & lt);
        c.kept[at] = (int)r;
        if (c.psw) c.kept_w[at] = w[k];
      }
      carry += __popc(m);
      // the part of this lane's bag that lies inside the block
      const int lo = (s > bb ? s : bb) - bb;
      const int hi = (e < bb + 32 ? e : bb + 32) - bb;
      if (hi > lo) {
        const unsigned span = (hi - lo >= 32 ? kFull : ((1u << (hi - lo)) - 1u)) << lo;
        mine += __popc(m & span);
        mine_counted += __popc(cm & span);
      }
    }
  }
  // sub-bag bounds: exclusive scan of the per-bag survivor counts
  int incl = mine;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int up = __shfl_up_sync(kFull, incl, d);
    if ((int)lane >= d) incl += up;
  }
  if ((int)lane < nb) {
    const int start = p0 + incl - mine;
    reinterpret_cast<int2*>(c.bounds)[b0 + lane] = make_int2(start, start + mine);
    if (c.counts) c.counts[b0 + lane] = mine_counted;
  }
}

}  // namespace fwd_eb
