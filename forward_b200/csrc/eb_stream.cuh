// The streaming lane-group kernel: a lane group walks a RUN of consecutive bags as one
// index stream.
//
// Same work split as eb_pool_group_kernel (lane l of a group owns 16-byte chunk l of a row;
// every column is accumulated in fp32 registers in bag order), but built around two queues so
// that no bag restarts the latency chain:
//
//   * index queue: the indices of the group's bags are consecutive in memory, so they are
//     fetched as blocks of 32 positions, one block ahead of use, filtered (padding / table
//     window) and parked in a small shared-memory ring addressed by position.  A bag boundary
//     does not interrupt the stream: the first rows of bag b+1 are requested while the last
//     rows of bag b are still being added.
//   * rows: a pass issues U row loads back to back and then folds them in order.  (A rolling
//     queue — re-arm a slot as soon as its row is folded — was built first and ran 2-3x
//     slower: a warp has only a handful of scoreboards for outstanding loads, so waiting for
//     the oldest load also waited for younger ones that shared its scoreboard.)
//
// Bag boundaries are found by position: the group keeps the end position of its current bag
// and a pass never crosses it; when a pass has reached it, the accumulators are finished,
// stored and cleared, and the bag counter moves on (an empty bag is a pass of zero rows that
// stores the cleared accumulators, i.e. zeros).  All loops are warp-uniform; a group whose
// run has ended runs with its predicates off.
//
// Shapes: 16-byte vector path, one chunk per lane (rows of 128 B to 512 B: groups of 8, 16
// or 32 lanes), int32 indices and offsets, fewer than 2^31 indices per call.  Everything else
// stays with eb_pool_group_kernel.
#pragma once

#include <climits>

#include "eb_kernels.cuh"

namespace fwd_eb {

constexpr int kStreamRing = 64;  // ring entries per group: two blocks of 32 positions
constexpr int kStreamMaxK = 16;  // bags per group at most (their end positions sit in shared memory)

// Rows per pass, by group width (measured on B200: 128-byte rows, short bags: 6 beats 4 and 5;
// 512-byte rows: 5 beats 4, 6 and 8, which spill at 64 registers).
#ifndef FWD_EB_STREAM_U
#define FWD_EB_STREAM_U 0
#endif
constexpr int stream_u(int lanes_log2) {
  return FWD_EB_STREAM_U > 0 ? FWD_EB_STREAM_U : (lanes_log2 == 3 ? 6 : 5);
}
#ifndef FWD_EB_STREAM_MIN_CTAS
#define FWD_EB_STREAM_MIN_CTAS 8
#endif

// Destination of the output rows when the pooling kernel itself hands them to other ranks
// (row shards / table-wise placement; see eb_shard.cu).
struct PushArgs {
  char* peer_slots[16];    // already offset to this call's buffer part
  uint32_t* peer_flags[16];
  long long bags_per_rank;
  long long row_base;    // destination row of this rank's first bag inside the owner's buffer
  long long col_offset;  // destination column of this call's first column
  long long first_bag;   // bag the grid starts with; later bags follow, wrapping at num_bags
  int world;
  int rank;
  int small;             // bag numbers and bags_per_rank fit 32 bits
  uint32_t epoch;
  unsigned* ticket;      // non-null: the grid's last CTA raises this rank's flag on every peer
};

// End of a pooling grid that pushes its rows to peers: the CTA that finishes last publishes
// `epoch` in this rank's flag word on every peer.  Every CTA makes its own stores visible system
// wide (fence) before it takes a ticket; the CTA that draws the last ticket therefore knows that
// all stores of the grid have been performed, fences again and writes the flags with release
// semantics.  It also clears the ticket word for the next grid that uses it (grids that share a
// word never overlap: a dependent grid's CTAs wait in griddepcontrol.wait until this grid has
// completed).  Called by every thread of the CTA.
__device__ __forceinline__ void push_grid_done(const PushArgs& x) {
  if (!x.ticket) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned total = gridDim.x * gridDim.y * gridDim.z;
    const unsigned t = atomicAdd(x.ticket, 1u);
    if (t == total - 1u) {
      *x.ticket = 0u;
      __threadfence_system();
      for (int r = 0; r < x.world; ++r)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(x.peer_flags[r] + x.rank), "r"(x.epoch)
                     : "memory");
    }
  }
}

template <typename TW, int VE, int LL, int OP, int U, bool PUSH>
__global__ void __launch_bounds__(kCtaThreads, FWD_EB_STREAM_MIN_CTAS)
eb_pool_stream_kernel(const PoolArgs a, const PushArgs x) {
  using V = typename Chunk<TW, VE>::type;
  constexpr int LANES = 1 << LL;
  constexpr int IPL = 32 / LANES;  // index loads per lane and block of 32 positions
  constexpr int GW = 32 / LANES;   // groups per warp
  constexpr int kWarps = kCtaThreads / 32;
  __shared__ int s_ring[kWarps * GW * kStreamRing];
  __shared__ float s_ringw[OP == kOpWeighted ? kWarps * GW * kStreamRing : 1];
  __shared__ int s_ends[kWarps * GW * kStreamMaxK];

  const unsigned lane = threadIdx.x & 31u;
  const int lig = lane & (LANES - 1);
  const int slot = (threadIdx.x >> 5) * GW + (lane >> LL);  // group within the CTA
  int* ring = s_ring + slot * kStreamRing;
  float* ringw = s_ringw + (OP == kOpWeighted ? slot * kStreamRing : 0);
  int* ends = s_ends + slot * kStreamMaxK;

  const int K = a.stream_k;
  long long gid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> LL;
  const long long ngroups = (a.num_bags + K - 1) / K;
  const bool live_group = gid < ngroups;
  if (PUSH && live_group) {  // start with the groups of the next rank's bags (see eb_pool_push_kernel)
    gid += x.first_bag / K;
    if (gid >= ngroups) gid -= ngroups;
  }
  const int b0 = (int)(gid * K);  // the host sends at most 2^31-1 bags this way
  const int nb = live_group ? (int)((a.num_bags - b0) < K ? (a.num_bags - b0) : K) : 0;

  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  const int* __restrict__ indices = reinterpret_cast<const int*>(a.indices);
  const int* __restrict__ offsets = reinterpret_cast<const int*>(a.offsets);
  const int n_idx = (int)a.num_indices;

  // ---- bag bounds of the run: start of the first bag, end of every bag -----------------
  int p0 = 0;
  if (nb > 0) {
    if (a.fixed_len > 0) p0 = b0 * a.fixed_len;
    else if (a.pairs) p0 = __ldg(offsets + 2LL * b0);
    else p0 = __ldg(offsets + b0);
    p0 = p0 < 0 ? 0 : (p0 > n_idx ? n_idx : p0);
  }
  for (int j = lig; j < nb; j += LANES) {
    const int b = b0 + j;
    int e;
    if (a.fixed_len > 0) e = (b + 1) * a.fixed_len;
    else if (a.pairs) e = __ldg(offsets + 2LL * b + 1);
    else e = (a.include_last || b + 1 < a.num_bags) ? __ldg(offsets + b + 1) : n_idx;
    ends[j] = e > n_idx ? n_idx : e;  // a malformed offsets array must not turn into a wild read
  }
  __syncwarp();
  int p1 = nb > 0 ? ends[nb - 1] : p0;
  if (p1 < p0) p1 = p0;
  const int len = p1 - p0;  // positions this group streams

  const bool chunk_ok = lig < a.nchunks;
  const char* __restrict__ tbase = a.table + lig * (VE * (int)sizeof(TW));
  const unsigned stride32 = (unsigned)a.row_bytes_stride;

  // ---- index queue ------------------------------------------------------------------
  // Ring entries: local row (>= 0), -1 = counted but outside the table window, -2 = padding
  // or past the end of the stream.
  int nx_idx[IPL];
  float nx_w[IPL];
  auto fetch = [&](int relbase) {
#pragma unroll
    for (int j = 0; j < IPL; ++j) {
      const int rel = relbase + j * LANES + lig;
      nx_idx[j] = 0;
      if (rel < len) {
        nx_idx[j] = __ldg(indices + p0 + rel);
        if (OP == kOpWeighted) nx_w[j] = __ldg(a.psw + p0 + rel);
      }
    }
  };
  auto park = [&](int relbase) {
#pragma unroll
    for (int j = 0; j < IPL; ++j) {
      const int rel = relbase + j * LANES + lig;
      int r = -2;
      if (rel < len) {
        const int idx = nx_idx[j];
        if (!a.pad32_on || idx != a.pad32) {
          const unsigned rr = (unsigned)idx - a.lo32;
          r = rr < a.nrows32 ? (int)rr : -1;
        }
      }
      ring[rel & (kStreamRing - 1)] = r;
      if (OP == kOpWeighted) ringw[rel & (kStreamRing - 1)] = nx_w[j];
    }
  };

  // ---- accumulators and the bag cursor ---------------------------------------------------
  float acc[VE];
#pragma unroll
  for (int e = 0; e < VE; ++e) acc[e] = 0.0f;
  int counted = 0;
  bool have = false;
  int bag = 0;
  int cur_end = nb > 0 ? ends[0] : INT_MAX;
  const bool tf16 = sizeof(TW) == 2;

  // ---- passes ---------------------------------------------------------------------------------
  // A pass takes up to U rows of the group's CURRENT bag: it reads their ring entries, issues the
  // row loads back to back (the loads of a pass share one wait, which is how the hardware's few
  // per-warp scoreboards want it) and folds them in order.  When the pass reached the bag's end
  // the accumulators are finished, stored and cleared and the cursor moves to the next bag,
  // whose first rows are already waiting in the ring: a bag boundary costs no round trip to
  // memory.  Groups of a warp advance independently; the loop is warp-uniform.
  fetch(0);
  park(0);
  fetch(32);
  int parked = 32;  // positions [0, parked) are in the ring; the block at `parked` is in registers
  int rel = 0;      // next position of the stream, relative to p0
  __syncwarp();

  while (__any_sync(kFull, bag < nb)) {
    const bool active = bag < nb;
    const bool need = active && rel + U > parked && parked < len;
    if (__any_sync(kFull, need)) {
      __syncwarp();
      if (need) {
        park(parked);
        parked += 32;
        fetch(parked);
      }
      __syncwarp();
    }
    int n = active ? cur_end - (p0 + rel) : 0;  // rows of the current bag taken by this pass
    n = n < 0 ? 0 : (n > U ? U : n);
    V val[U];
    float w[U];
    unsigned okmask = 0u, cntmask = 0u;  // bit u: slot u holds a row / a counted entry
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int q = rel + u;
      const bool in = u < n && q < len;
      const int r = in ? ring[q & (kStreamRing - 1)] : -2;
      okmask |= (r >= 0 ? 1u : 0u) << u;
      cntmask |= (r >= -1 ? 1u : 0u) << u;
      if (OP == kOpWeighted) w[u] = in ? ringw[q & (kStreamRing - 1)] : 0.0f;
      if (r >= 0 && chunk_ok)
        val[u] = load_chunk<V>(tbase + (unsigned long long)(unsigned)r * stride32);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (((okmask >> u) & 1u) && chunk_ok) {
        fold_chunk<OP>(acc, val[u], OP == kOpWeighted ? w[u] : 1.0f, !have);
        have = true;
      }
    }
    counted += __popc(cntmask);
    rel += n;
    const bool hit = active && p0 + rel >= cur_end;  // the bag is complete (an empty bag at once)
    if (__any_sync(kFull, hit)) {
      float v[1][VE];
#pragma unroll
      for (int e = 0; e < VE; ++e) v[0][e] = acc[e];
      if (OP == kOpMax && VE == 8) unpack_half_max(reinterpret_cast<float(&)[8]>(v[0]));
#pragma unroll
      for (int e = 0; e < VE; ++e)
        v[0][e] = finish(a, v[0][e], counted, (long long)(cur_end - (bag > 0 ? ends[bag - 1] : p0)), tf16);
      const long long b = (long long)b0 + bag;
      if (PUSH) {
        long long owner = 0;
        if (hit)
          owner = x.small ? (long long)((unsigned)b / (unsigned)x.bags_per_rank) : b / x.bags_per_rank;
        if (owner >= x.world) owner = x.world - 1;
        char* base = x.peer_slots[owner] + x.col_offset * (a.out_f16 ? 2 : 4);
        store_row<VE, 1, true>(a, base, x.row_base + (b - owner * x.bags_per_rank), 0, v, hit);
      } else {
        store_row<VE, 1, true>(a, a.out, b, 0, v, hit);
      }
      if (hit) {
#pragma unroll
        for (int e = 0; e < VE; ++e) acc[e] = 0.0f;
        counted = 0;
        have = false;
        ++bag;
        cur_end = bag < nb ? ends[bag] : INT_MAX;
      }
    }
  }
  if (PUSH) push_grid_done(x);
}

}  // namespace fwd_eb
