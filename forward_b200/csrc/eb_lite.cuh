// The lean lane-group kernel: one lane group per bag, nothing but the essentials.
//
// The pooling kernels of this library are as sensitive to issued instructions as to memory
// latency (ncu on B200: issue slots 45-60 % busy while DRAM is 40 % busy), and for short bags
// the fixed work per bag dominates: eb_pool_group_kernel's blocks of 32 indices, survivor ring
// and next-block prefetch cost several hundred instructions per warp before the first row
// arrives.  This kernel keeps the same work split and the same order of additions (lane l of a
// group owns 16-byte chunk l of a row; rows are folded in bag order, so results are bit-identical
// to the other lane-group kernels) and drops the rest:
//
//   * a block is LANES indices, one coalesced load per lane (the next block is requested
//     before the current one is used);
//   * the padding / table-window filter is three 32-bit instructions on the loaded index;
//     a filtered entry simply issues no row load (no compaction inside the kernel: callers
//     with sparse windows compact first, see eb_compact.cuh);
//   * rows are fetched in passes of 4 to 7 loads per lane, the row number of slot u coming
//     from lane u of the group by shuffle, then folded in order.
//
// Shapes: 16-byte vector path, one chunk per lane (rows of 128 B to 512 B), int32 indices and
// offsets (plain, fixed-length or {start, end} pairs), fewer than 2^31 indices per call.
#pragma once

#include "eb_kernels.cuh"
#include "eb_stream.cuh"  // PushArgs

namespace fwd_eb {

#ifndef FWD_EB_LITE_PASS
#define FWD_EB_LITE_PASS 0
#endif
#ifndef FWD_EB_LITE_MIN_CTAS
#define FWD_EB_LITE_MIN_CTAS 0
#endif
// Row loads in flight per lane and pass, and resident CTAs per SM (which caps the registers: 8 CTAs
// of 128 threads = 64 registers, 10 = 48, 12 = 40).  A longer pass hides more latency per warp but
// costs 4 registers per fp16 row slot; once the kernel spills, it loses more than the pass gains, and
// short bags want warps in flight rather than loads per warp.  Measured on B200, us per call, as
// pass / CTAs:
//   fp16, 128 B rows, 131072 bags of ~6 rows     8/8 37.0   4/8 38.8   4/10 34.4   4/12 32.8   3/16 32.9
//   fp16, 256 B rows, 16384 bags of ~40 (Zipf)    6/8 19.5   7/8 23.3   8/8 22.6   6/9 20.0   6/10 21.8   4/12 22.0
//   fp16, 512 B rows, 8192 bags of 0..64, max     7/8 28.8   6/8 29.1   8/9 28.5   6/10 29.8   4/12 31.2
//   fp32, 512 B rows, 65536 bags of 20, weighted  7/8 62.9   6/9 56.1   4/10 52.0   5/10 50.9   5/12 51.7   6/12 74.9
__host__ __device__ constexpr int lite_pass(int lanes_log2, int elem_bytes) {
  return FWD_EB_LITE_PASS > 0 ? FWD_EB_LITE_PASS
         : elem_bytes == 4    ? 5
                              : (lanes_log2 == 3 ? 4 : (lanes_log2 == 5 ? 7 : 6));
}
__host__ __device__ constexpr int lite_min_ctas(int lanes_log2, int elem_bytes) {
  return FWD_EB_LITE_MIN_CTAS > 0 ? FWD_EB_LITE_MIN_CTAS
         : elem_bytes == 4        ? 10
                                  : (lanes_log2 == 3 ? 12 : FWD_EB_MIN_CTAS);
}

template <typename TW, int VE, int LL, int OP, bool PUSH>
__global__ void __launch_bounds__(kCtaThreads, lite_min_ctas(LL, (int)sizeof(TW)))
eb_pool_lite_kernel(const PoolArgs a, const PushArgs x) {
  using V = typename Chunk<TW, VE>::type;
  constexpr int LANES = 1 << LL;
  constexpr int U = lite_pass(LL, (int)sizeof(TW));
  constexpr unsigned GMASK = LANES == 32 ? kFull : ((1u << LANES) - 1u);
  const unsigned lane = threadIdx.x & 31u;
  const int lig = lane & (LANES - 1);
  const int gbase = lane & ~(LANES - 1);
  const int seq = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) >> LL);
  const bool live = seq < a.num_bags;
  int bag = seq;
  if (PUSH && live) {  // start with the next rank's bags (see eb_pool_push_kernel)
    bag += (int)x.first_bag;
    if (bag >= a.num_bags) bag -= (int)a.num_bags;
  }
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  const int* __restrict__ indices = reinterpret_cast<const int*>(a.indices);
  const int* __restrict__ offsets = reinterpret_cast<const int*>(a.offsets);
  const int n_idx = (int)a.num_indices;
  int start = 0, end = 0;
  if (live) {
    if (a.fixed_len > 0) {
      start = bag * a.fixed_len;
      end = start + a.fixed_len;
    } else if (a.pairs) {
      const int2 se = __ldg(reinterpret_cast<const int2*>(offsets) + bag);
      start = se.x;
      end = se.y;
    } else {
      start = __ldg(offsets + bag);
      end = (a.include_last || bag + 1 < a.num_bags) ? __ldg(offsets + bag + 1) : n_idx;
    }
    // a malformed offsets array must not turn into a wild read
    start = start < 0 ? 0 : start;
    end = end > n_idx ? n_idx : end;
    end = end < start ? start : end;
  }

  const bool chunk_ok = lig < a.nchunks;
  const char* __restrict__ tbase = a.table + lig * (VE * (int)sizeof(TW));
  const unsigned stride32 = (unsigned)a.row_bytes_stride;

  float acc[VE];
#pragma unroll
  for (int e = 0; e < VE; ++e) acc[e] = 0.0f;
  int counted = 0;
  bool have = false;

  // one index per lane: local row (>= 0), -1 = counted but outside the window, -2 = padding / none
  auto fetch = [&](int pos, int& row, float& w) {
    row = -2;
    w = 1.0f;
    if (pos < end) {
      const int idx = __ldg(indices + pos);
      if (!a.pad32_on || idx != a.pad32) {
        const unsigned r = (unsigned)idx - a.lo32;
        row = r < a.nrows32 ? (int)r : -1;
        if (OP == kOpWeighted) w = __ldg(a.psw + pos);
      }
    }
  };

  int row, nrow;
  float w, nw;
  fetch(start + lig, row, w);
  for (int base = start; __any_sync(kFull, base < end); base += LANES) {
    fetch(base + LANES + lig, nrow, nw);  // next block, early
    if (a.mean) counted += __popc((__ballot_sync(kFull, row >= -1) >> gbase) & GMASK);
    const int n = end - base;             // entries of this block (may exceed LANES or be <= 0)
#pragma unroll
    for (int k = 0; k < LANES; k += U) {
      if (!__any_sync(kFull, k < n)) break;
      V val[U];
      float wu[U];
      unsigned ok = 0u;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int r = __shfl_sync(kFull, row, gbase + ((k + u) & (LANES - 1)));
        if (OP == kOpWeighted) wu[u] = __shfl_sync(kFull, w, gbase + ((k + u) & (LANES - 1)));
        const bool take = k + u < n && k + u < LANES && r >= 0;
        ok |= (take ? 1u : 0u) << u;
        if (take && chunk_ok) val[u] = load_chunk<V>(tbase + (unsigned long long)(unsigned)r * stride32);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (((ok >> u) & 1u) && chunk_ok) {
          fold_chunk<OP>(acc, val[u], OP == kOpWeighted ? wu[u] : 1.0f, !have);
          have = true;
        }
      }
    }
    row = nrow;
    w = nw;
  }

  float v[1][VE];
#pragma unroll
  for (int e = 0; e < VE; ++e) v[0][e] = acc[e];
  if (OP == kOpMax && VE == 8) unpack_half_max(reinterpret_cast<float(&)[8]>(v[0]));
  const bool tf16 = sizeof(TW) == 2;
#pragma unroll
  for (int e = 0; e < VE; ++e) v[0][e] = finish(a, v[0][e], counted, (long long)(end - start), tf16);
  if (PUSH) {
    long long owner = 0;
    if (live) owner = (long long)((unsigned)bag / (unsigned)x.bags_per_rank);
    if (owner >= x.world) owner = x.world - 1;
    char* base = x.peer_slots[owner] + x.col_offset * (a.out_f16 ? 2 : 4);
    store_row<VE, 1, true>(a, base, x.row_base + (bag - owner * x.bags_per_rank), 0, v, live);
    push_grid_done(x);
  } else {
    store_row<VE, 1, true>(a, a.out, bag, 0, v, live);
  }
}

}  // namespace fwd_eb
