// Device code of the EmbeddingBag gather-and-pool path for sm_100a.
//
// Replaces the three kernels of Forward's EmbeddingBag plugin
// (source/trt_engine/trt_network_crt/plugins/embedding_bag_plugin/
// embedding_bag_plugin.cu:66-181).  The reference pools through shared-memory
// atomics with one column per thread; here a *lane group* owns a bag:
//
//   * a table row is cut into 16-byte chunks and lane l of the group loads
//     chunk l (and l + lanes, ... when the row is wider than the group), so one
//     warp-wide load instruction fetches 32/lanes whole rows with every sector
//     fully used;
//   * the group reads `lanes` indices with one coalesced load, the warp votes
//     (ballot) on which of them survive the padding / table-window filter, and
//     the survivors are walked in bag order by shuffling the row number from
//     the lane that loaded it; U row loads are issued before the first add so
//     U * row_bytes per group are in flight;
//   * every column is accumulated in fp32 registers in bag order, which is the
//     order torch CPU uses, so sum / mean / weighted sum / max reproduce it
//     exactly; max keeps the first of equal values because the comparison is
//     strict and rows arrive in order.
//
// Three strategies share that inner loop: a group per bag (many bags), a CTA
// per bag (long bags; groups take consecutive slices and are folded in slice
// order through shared memory) and split bags (several CTAs per bag, partial
// results in caller-provided scratch, folded in order by a second kernel).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fwd_eb {

constexpr unsigned kFull = 0xffffffffu;
#ifndef FWD_EB_CTA_THREADS
#define FWD_EB_CTA_THREADS 128
#endif
constexpr int kCtaThreads = FWD_EB_CTA_THREADS;

// CTA size of the lane-group kernels.  When a bag takes a whole warp (rows of 512 B and more) a
// CTA is one warp, so a finished bag frees its slot at once instead of waiting for the longest
// of four (3-4 % on ragged 512-byte-row bags; the SM holds 32 such CTAs, the same 32 warps).
// Narrower groups keep kCtaThreads.  The kernels read blockDim.x.
#ifndef FWD_EB_WARP_CTA
#define FWD_EB_WARP_CTA 32
#endif
inline int group_cta_threads(int lanes_log2) { return lanes_log2 >= 5 ? FWD_EB_WARP_CTA : kCtaThreads; }
// Resident CTAs per SM the pooling kernels are compiled for (caps registers per thread).
#ifndef FWD_EB_MIN_CTAS
#define FWD_EB_MIN_CTAS 8
#endif
// Row loads in flight per lane group and pass (one 16-byte chunk per lane): 6 measured best on
// B200 for 256-byte rows (4: 31.6 us, 5: 30.1, 6: 29.3 on 16384 bags of ~40 uniform indices).
#ifndef FWD_EB_U1
#define FWD_EB_U1 6
#endif

enum Op { kOpSum = 0, kOpWeighted = 1, kOpMax = 2, kOpSquareSum = 3 };

struct PoolArgs {
  const char* table;        // device bytes
  long long row_bytes_stride;  // bytes between rows
  long long num_rows;
  long long row_lo;
  const void* indices;
  const void* offsets;
  long long num_indices;
  long long num_bags;
  const float* psw;
  long long padding_idx;
  char* out;
  long long out_stride;     // elements between output rows
  float* ws_acc;            // split strategy: [num_bags, splits, dim] fp32
  int* ws_meta;             // split strategy: [num_bags, splits, 2] {counted, have}
  int dim;
  int nchunks;              // chunks per row (16 B vectors, or elements in scalar mode)
  int lanes_log2;           // lanes per group
  int fixed_len;
  int idx64;
  int include_last;
  int out_f16;
  int out_vec;              // output rows are 16 B aligned: vector stores allowed
  int mean;                 // divide by the bag's count at the end
  int mean_raw_len;         // ... by the raw bag length instead of the non-padding count
  int mean_double_round;    // fp16 mean the way torch CPU rounds it
  int splits;               // split strategy: CTAs per bag
  int pairs;                // offsets hold a {start, end} pair per bag instead of one start
  int stream_k;             // streaming kernel: consecutive bags per lane group
  // 32-bit form of the filter for int32 indices (set by the host; see fetch in pool_range)
  unsigned lo32;            // row_lo
  unsigned nrows32;         // num_rows, or 0 when the window lies beyond the int32 range
  int pad32;                // padding_idx, or INT_MIN-like sentinel that matches nothing counted
  int pad32_on;             // padding_idx is set and fits an int
};

template <typename TW, int VE>
struct Chunk;
template <>
struct Chunk<float, 4> { using type = float4; };
template <>
struct Chunk<__half, 8> { using type = uint4; };
template <>
struct Chunk<float, 1> { using type = float; };
template <>
struct Chunk<__half, 1> { using type = __half; };

__device__ __forceinline__ void unpack(const float4& v, float (&f)[4]) {
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
__device__ __forceinline__ void unpack(const uint4& v, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __half22float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void unpack(const float& v, float (&f)[1]) { f[0] = v; }
__device__ __forceinline__ void unpack(const __half& v, float (&f)[1]) { f[0] = __half2float(v); }

template <typename V>
__device__ __forceinline__ V load_chunk(const char* p) {
  return __ldg(reinterpret_cast<const V*>(p));
}

template <int OP>
__device__ __forceinline__ void fold(float& acc, float x, float w, bool first) {
  if (OP == kOpSum) {
    acc = __fadd_rn(acc, x);
  } else if (OP == kOpWeighted) {
    acc = __fmaf_rn(w, x, acc);
  } else if (OP == kOpSquareSum) {
    acc = __fadd_rn(acc, __fmul_rn(x, x));
  } else {  // max: the first row is taken as is, later rows only when strictly greater
    acc = (first || x > acc) ? x : acc;
  }
}

// acc += float(h), one rounding: sm_100's mixed-precision add takes the half operand as is,
// which saves the separate conversion (same result as convert-then-add: the conversion is
// exact).
__device__ __forceinline__ void add_half(float& acc, unsigned short h) {
  asm("add.rn.f32.f16 %0, %1, %0;" : "+f"(acc) : "h"(h));
}

// Two fp32 adds in one instruction (sm_100 packed fp32 pipe); each lane rounds on its own.
__device__ __forceinline__ void add_pair(float& a0, float& a1, float x0, float x1) {
  unsigned long long acc, x;
  asm("mov.b64 %0, {%1, %2};" : "=l"(acc) : "f"(a0), "f"(a1));
  asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "f"(x0), "f"(x1));
  asm("add.rn.f32x2 %0, %0, %1;" : "+l"(acc) : "l"(x));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a0), "=f"(a1) : "l"(acc));
}

// Fold one loaded chunk into the accumulators.
// Max over fp16 rows is kept in fp16 while a bag is walked: the eight running values sit as
// four packed pairs in acc[0..3] (bit patterns), a row replaces a value only where it is
// strictly greater (one packed compare producing a lane mask, one bit select), and the first
// row is taken whole.  Comparing halves orders exactly as comparing their float values, the
// winner's bits are carried unchanged (so -0.0 / +0.0 and the first of equals survive), and a
// NaN never wins over an earlier value.  unpack_half_max() turns the pairs into floats once
// the bag is done.
__device__ __forceinline__ void max_half2(float& acc_bits, unsigned x, bool first) {
  const unsigned a = __float_as_uint(acc_bits);
  unsigned gt;  // 0xffff in each half where x > a
  asm("set.gt.u32.f16x2 %0, %1, %2;" : "=r"(gt) : "r"(x), "r"(a));
  const unsigned m = first ? 0xffffffffu : gt;
  acc_bits = __uint_as_float((x & m) | (a & ~m));
}
__device__ __forceinline__ void unpack_half_max(float (&acc)[8]) {
  unsigned w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) w[i] = __float_as_uint(acc[i]);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    acc[2 * i] = t.x;
    acc[2 * i + 1] = t.y;
  }
}

template <int OP>
__device__ __forceinline__ void fold_chunk(float (&acc)[8], const uint4& v, float w, bool first) {
  if (OP == kOpMax) {
    max_half2(acc[0], v.x, first);
    max_half2(acc[1], v.y, first);
    max_half2(acc[2], v.z, first);
    max_half2(acc[3], v.w, first);
  } else if (OP == kOpSum) {
    const unsigned wd[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      add_half(acc[2 * i], (unsigned short)(wd[i] & 0xffffu));
      add_half(acc[2 * i + 1], (unsigned short)(wd[i] >> 16));
    }
  } else {
    float f[8];
    unpack(v, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) fold<OP>(acc[e], f[e], w, first);
  }
}
template <int OP>
__device__ __forceinline__ void fold_chunk(float (&acc)[4], const float4& v, float w, bool first) {
  if (OP == kOpSum) {
    add_pair(acc[0], acc[1], v.x, v.y);
    add_pair(acc[2], acc[3], v.z, v.w);
  } else {
    float f[4];
    unpack(v, f);
#pragma unroll
    for (int e = 0; e < 4; ++e) fold<OP>(acc[e], f[e], w, first);
  }
}
template <int OP>
__device__ __forceinline__ void fold_chunk(float (&acc)[1], const float& v, float w, bool first) {
  fold<OP>(acc[0], v, w, first);
}
template <int OP>
__device__ __forceinline__ void fold_chunk(float (&acc)[1], const __half& v, float w, bool first) {
  fold<OP>(acc[0], __half2float(v), w, first);
}

__device__ __forceinline__ long long load_index(const void* p, int idx64, long long i) {
  return idx64 ? __ldg(reinterpret_cast<const long long*>(p) + i)
               : static_cast<long long>(__ldg(reinterpret_cast<const int*>(p) + i));
}

__device__ __forceinline__ void bag_bounds(const PoolArgs& a, long long bag, long long& start,
                                           long long& end) {
  if (a.fixed_len > 0) {
    start = bag * a.fixed_len;
    end = start + a.fixed_len;
  } else if (a.pairs) {
    start = load_index(a.offsets, a.idx64, 2 * bag);
    end = load_index(a.offsets, a.idx64, 2 * bag + 1);
  } else {
    start = load_index(a.offsets, a.idx64, bag);
    end = (a.include_last || bag + 1 < a.num_bags) ? load_index(a.offsets, a.idx64, bag + 1)
                                                    : a.num_indices;
  }
  // a malformed offsets array must not turn into a wild read
  if (start < 0) start = 0;
  if (end > a.num_indices) end = a.num_indices;
  if (end < start) end = start;
}

// State one lane group carries while it walks a range of a bag.
template <int CPL, int VE>
struct Accum {
  float v[CPL][VE];
  int counted;  // non-padding indices seen (inside or outside the table window)
  bool have;    // at least one row was folded in
  bool seeded;  // max only: the accumulators start at -inf and every row is compared strictly
};

// One lane's share of walking indices [start, end) of a bag.  All 32 lanes of
// the warp must call this together (the loops are warp-uniform; a group with
// nothing left simply has its predicates off).
//
// IPL = index loads per lane and block.  A block is lanes * IPL consecutive indices of the
// bag; with IPL = 32 / lanes (groups of 16 or 8 lanes) every block is 32 indices, so a bag of
// 50 indices costs two index round trips whatever the row width.
template <typename TW, int VE, int CPL, int OP, int U, int IPL>
__device__ __forceinline__ void pool_range(const PoolArgs& a, long long start, long long end,
                                           int chunk0, Accum<CPL, VE>& s) {
  using V = typename Chunk<TW, VE>::type;
  const int lanes = 1 << a.lanes_log2;
  const unsigned lane = threadIdx.x & 31u;
  const int lig = lane & (lanes - 1);
  const int gbase = lane & ~(lanes - 1);
  const unsigned gmask = lanes == 32 ? kFull : ((1u << lanes) - 1u);
  const int vbytes = VE * (int)sizeof(TW);
  const unsigned stride32 = (unsigned)a.row_bytes_stride;  // checked on the host: < 2^32
  const int block = lanes * IPL;

  bool chunk_ok[CPL];
  int chunk_off[CPL];
#pragma unroll
  for (int c = 0; c < CPL; ++c) {
    int chunk = chunk0 + c * lanes + lig;
    chunk_ok[c] = chunk < a.nchunks;
    chunk_off[c] = chunk * vbytes;
  }

  // fetch one index: local row (>= 0) or -1 for "skip"
  auto fetch = [&](long long pos, int& row, float& w, bool& counted) {
    row = -1;
    w = 1.0f;
    counted = false;
    if (pos < end) {
      if (!a.idx64) {
        // int32 indices: the whole filter in 32-bit arithmetic.  (unsigned)(idx - lo) < rows
        // is the window test; a negative or too-small index wraps to a value >= 2^31.
        const int idx = __ldg(reinterpret_cast<const int*>(a.indices) + pos);
        if (!a.pad32_on || idx != a.pad32) {
          counted = true;
          const unsigned r = (unsigned)idx - a.lo32;
          if (r < a.nrows32) {
            row = (int)r;
            if (OP == kOpWeighted) w = __ldg(a.psw + pos);
          }
        }
        return;
      }
      long long idx = load_index(a.indices, a.idx64, pos);
      if (a.padding_idx < 0 || idx != a.padding_idx) {
        counted = true;
        long long r = idx - a.row_lo;
        if (r >= 0 && r < a.num_rows) {
          row = (int)r;
          if (OP == kOpWeighted) w = __ldg(a.psw + pos);
        }
      }
    }
  };

  // Issue U row loads, then fold them in order; ok[u] switches a slot off.
  auto consume = [&](const int (&row)[U], const float (&w)[U], const bool (&ok)[U]) {
    V val[U][CPL];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (ok[u]) {
        const char* rp = a.table + (unsigned long long)(unsigned)row[u] * stride32;
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
          if (chunk_ok[c]) val[u][c] = load_chunk<V>(rp + chunk_off[c]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (ok[u]) {
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
          if (chunk_ok[c])
            fold_chunk<OP>(s.v[c], val[u][c], OP == kOpWeighted ? w[u] : 1.0f, !s.have && !s.seeded);
        }
        s.have = true;
      }
    }
  };

  // Survivors of a block (everything that is not padding and lies inside the table window)
  // wait in a per-group ring in shared memory until U of them are there, so a row-load pass
  // is as full for a 1-in-8 window as for a dense bag, and blocks without enough survivors
  // cost no row round trip of their own.  Capacity 2 * block per group.  Groups narrower than
  // 8 lanes (rows under 128 B) keep their survivors in registers and walk the mask instead.
  constexpr int kRingPerWarp = 64 * (IPL > 1 ? IPL : 1);
  __shared__ int ring_row[(kCtaThreads / 32) * kRingPerWarp];
  __shared__ float ring_w[OP == kOpWeighted ? (kCtaThreads / 32) * kRingPerWarp : 1];
  const bool use_ring = IPL > 1 || lanes >= 8;
  const int ring_cap = 2 * block;
  const int ring_base = (threadIdx.x >> 5) * kRingPerWarp + 2 * IPL * gbase;
  int ring_head = 0, ring_tail = 0;  // same value in every lane of a group

  long long base = start;
  int cur_row[IPL], nxt_row[IPL];
  float cur_w[IPL], nxt_w[IPL];
  bool cur_counted[IPL], nxt_counted[IPL];
#pragma unroll
  for (int j = 0; j < IPL; ++j) fetch(base + j * lanes + lig, cur_row[j], cur_w[j], cur_counted[j]);

  while (__any_sync(kFull, base < end)) {
#pragma unroll
    for (int j = 0; j < IPL; ++j)  // next block of indices, early
      fetch(base + block + j * lanes + lig, nxt_row[j], nxt_w[j], nxt_counted[j]);
    long long left = end - base;
    const int n = left <= 0 ? 0 : (left < block ? (int)left : block);  // entries of this block
    const bool last_block = left <= block;
    const unsigned want = n >= 32 ? kFull : ((1u << n) - 1u);
    unsigned m = 0;  // bit e = entry e of the block survived; e = j * lanes + lane-in-group
#pragma unroll
    for (int j = 0; j < IPL; ++j) {
      m |= ((__ballot_sync(kFull, cur_row[j] >= 0) >> gbase) & gmask) << (j * lanes);
      if (a.mean) s.counted += __popc((__ballot_sync(kFull, cur_counted[j]) >> gbase) & gmask);
    }

    // Three ways to feed a pass of U row loads per group:
    //   dense  (IPL == 1) every entry of every group's block survived and no ring holds older
    //          rows: slot k of a pass is entry k of the block, fetched by shuffle;
    //   ring   survivors are appended to the group's ring and passes run while a ring holds
    //          U rows (or anything at all, on the group's last block);
    //   walk   narrow groups: the set bits of the survivor mask are walked directly.
    const bool dense = IPL == 1 && __all_sync(kFull, m == want && ring_head == ring_tail);
    const bool ring = !dense && use_ring;
    if (ring) {
#pragma unroll
      for (int j = 0; j < IPL; ++j) {
        if (cur_row[j] >= 0) {
          const int e = j * lanes + lig;
          const int at = ring_base + ((ring_tail + __popc(m & ((1u << e) - 1u))) & (ring_cap - 1));
          ring_row[at] = cur_row[j];
          if (OP == kOpWeighted) ring_w[at] = cur_w[j];
        }
      }
      ring_tail += __popc(m);
      __syncwarp();
    }
    const int nmax = __reduce_max_sync(kFull, n);
    for (int k = 0;; k += U) {
      const int pending = ring_tail - ring_head;
      bool more;
      if (dense) {
        more = k < nmax;
      } else if (ring) {
        more = __any_sync(kFull, last_block ? pending > 0 : pending >= U);
      } else {
        more = __any_sync(kFull, m != 0u);
      }
      if (!more) break;
      int row[U];
      float w[U];
      bool ok[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (ring) {
          ok[u] = u < pending;
          const int at = ring_base + ((ring_head + u) & (ring_cap - 1));
          row[u] = ring_row[at];
          if (OP == kOpWeighted) w[u] = ring_w[at];
        } else {
          int src;
          if (dense) {
            src = (k + u) & (lanes - 1);
            ok[u] = (k + u) < n;
          } else {
            ok[u] = m != 0u;
            src = ok[u] ? (__ffs(m) - 1) : 0;
            m &= (m - 1u);  // clears the lowest set bit; 0 stays 0
          }
          row[u] = __shfl_sync(kFull, cur_row[0], gbase + src);
          if (OP == kOpWeighted) w[u] = __shfl_sync(kFull, cur_w[0], gbase + src);
        }
      }
      if (ring) ring_head += pending < U ? pending : U;
      consume(row, w, ok);
    }
    if (ring) __syncwarp();  // all reads of the ring are done before the next block is appended
#pragma unroll
    for (int j = 0; j < IPL; ++j) {
      cur_row[j] = nxt_row[j];
      cur_w[j] = nxt_w[j];
      cur_counted[j] = nxt_counted[j];
    }
    base += block;
  }
  if (OP == kOpMax && VE == 8) {  // fp16 max ran on packed pairs: back to one float per column
#pragma unroll
    for (int c = 0; c < CPL; ++c) unpack_half_max(reinterpret_cast<float(&)[8]>(s.v[c]));
  }
}

// Final value of one column: mean division and rounding rules.
__device__ __forceinline__ float finish(const PoolArgs& a, float acc, int counted,
                                        long long raw_len, bool table_f16) {
  if (!a.mean) return acc;
  long long d = a.mean_raw_len ? raw_len : (long long)counted;
  if (d < 1) d = 1;
  float denom = (float)d;
  if (a.out_f16 && table_f16 && a.mean_double_round) {
    acc = __half2float(__float2half_rn(acc));
  }
  return __fdiv_rn(acc, denom);
}

// Write this lane's chunks of one output row.
//
// With EXCHANGE (pooling kernels) the call must be made by all 32 lanes of the warp — lanes
// with nothing to write pass live = false — because 32-byte-per-lane fp32 rows are written
// through a neighbour swap: a lane holds 8 floats = 32 B, and storing them as two 16-byte
// halves would have every lane touch half a sector twice.  Neighbouring lanes swap one quad
// so each store instruction writes whole 32-byte sectors (even lane: its quad 0, then the odd
// lane's quad 0; odd lane: the even lane's quad 1, then its own quad 1).  This matters most
// for stores that cross NVLink.
template <int VE, int CPL, bool EXCHANGE>
__device__ __forceinline__ void store_row(const PoolArgs& a, char* out_base, long long out_row,
                                          int chunk0, const float (&v)[CPL][VE], bool live) {
  const int lanes = 1 << a.lanes_log2;
  const int lig = (threadIdx.x & 31u) & (lanes - 1);
#pragma unroll
  for (int c = 0; c < CPL; ++c) {
    const int chunk = chunk0 + c * lanes + lig;
    const bool swap = EXCHANGE && VE == 8 && !a.out_f16 && a.out_vec && lanes >= 2;
    float x4[4];
    if (swap) {  // warp-uniform condition: every lane takes part in the shuffles
      const bool odd = lig & 1;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        x4[e] = __shfl_xor_sync(kFull, odd ? v[c][e < VE ? e : 0] : v[c][4 + e < VE ? 4 + e : 0], 1);
      }
    }
    if (!live || chunk >= a.nchunks) continue;
    long long col = (long long)chunk * VE;
    if (a.out_f16) {
      __half* o = reinterpret_cast<__half*>(out_base) + out_row * a.out_stride + col;
      if (VE == 8 && a.out_vec) {
        uint4 pk;
        __half2* h = reinterpret_cast<__half2*>(&pk);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(v[c][(2 * e) % VE], v[c][(2 * e + 1) % VE]);
        *reinterpret_cast<uint4*>(o) = pk;
      } else if (VE == 4 && a.out_vec) {
        uint2 pk;
        __half2* h = reinterpret_cast<__half2*>(&pk);
        h[0] = __floats2half2_rn(v[c][0], v[c][1 % VE]);
        h[1] = __floats2half2_rn(v[c][2 % VE], v[c][3 % VE]);
        *reinterpret_cast<uint2*>(o) = pk;
      } else {
#pragma unroll
        for (int e = 0; e < VE; ++e) o[e] = __float2half_rn(v[c][e]);
      }
    } else {
      float* o = reinterpret_cast<float*>(out_base) + out_row * a.out_stride + col;
      if (swap && ((chunk | 1) < a.nchunks)) {
        const bool odd = lig & 1;
        float* pair = o - (odd ? 8 : 0);  // first float of the lane pair's 16
        if (!odd) {
          *reinterpret_cast<float4*>(pair) = make_float4(v[c][0], v[c][1 % VE], v[c][2 % VE], v[c][3 % VE]);
          *reinterpret_cast<float4*>(pair + 8) = make_float4(x4[0], x4[1], x4[2], x4[3]);
        } else {
          *reinterpret_cast<float4*>(pair + 4) = make_float4(x4[0], x4[1], x4[2], x4[3]);
          *reinterpret_cast<float4*>(pair + 12) =
              make_float4(v[c][4 % VE], v[c][5 % VE], v[c][6 % VE], v[c][7 % VE]);
        }
      } else if (VE >= 4 && a.out_vec) {
#pragma unroll
        for (int e = 0; e < VE; e += 4) {
          *reinterpret_cast<float4*>(o + e) = make_float4(v[c][e], v[c][(e + 1) % VE],
                                                          v[c][(e + 2) % VE], v[c][(e + 3) % VE]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < VE; ++e) o[e] = v[c][e];
      }
    }
  }
}

template <int CPL, int VE>
__device__ __forceinline__ void clear(Accum<CPL, VE>& s) {
#pragma unroll
  for (int c = 0; c < CPL; ++c)
#pragma unroll
    for (int e = 0; e < VE; ++e) s.v[c][e] = 0.0f;
  s.counted = 0;
  s.have = false;
  s.seeded = false;
}

// MAX over a slice of a bag that is not the bag's first slice: torch's sequential rule takes the
// bag's first entry as is (a NaN there sticks) and every later entry only when strictly
// greater (a later NaN is ignored).  A slice that took ITS first row as is would keep a NaN
// that torch ignores, and the fold across slices would then drop the whole slice, larger values
// included.  Such a slice therefore starts from -inf and compares every row strictly.
// (One corner stays: a NaN that is the bag's first non-padding entry but sits in a later slice,
// every slice before it holding padding only, is ignored where torch keeps it.)
template <int CPL, int VE, typename TW>
__device__ __forceinline__ void seed_max_slice(Accum<CPL, VE>& s) {
#pragma unroll
  for (int c = 0; c < CPL; ++c) {
    if (sizeof(TW) == 2 && VE == 8) {  // fp16 rows: four packed pairs of -inf halves
#pragma unroll
      for (int e = 0; e < 4; ++e) s.v[c][e] = __uint_as_float(0xFC00FC00u);
    } else {
#pragma unroll
      for (int e = 0; e < VE; ++e) s.v[c][e] = -INFINITY;
    }
  }
  s.seeded = true;
}

// ---- strategy 1: one lane group per bag -------------------------------------
// grid.x covers bags (kCtaThreads / lanes bags per CTA), grid.y covers column
// tiles of 32 * CPL chunks for rows wider than one tile.
template <typename TW, int VE, int CPL, int OP, int U, int IPL>
__global__ void __launch_bounds__(kCtaThreads, FWD_EB_MIN_CTAS)
eb_pool_group_kernel(const PoolArgs a) {
  const int lanes_log2 = a.lanes_log2;
  const long long bag =
      ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> lanes_log2;
  const int chunk0 = blockIdx.y * (CPL << lanes_log2);
  const bool live = bag < a.num_bags;
  // Programmatic dependent launch: let the next grid on the stream (if it was launched with
  // programmatic stream serialization) place its CTAs while this grid's last ones drain, and
  // touch no memory before every grid ahead of this one has completed.  Both are no-ops for
  // an ordinary launch.
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
  store_row<VE, CPL, true>(a, a.out, bag, chunk0, s.v, live);
}

// ---- max with the winner's position (output type FWD_EB_F32_POS) ---------------
// out[bag][col] = {value as fp32, position inside the bag of the index that supplied it}, 8
// bytes per column; {0, kNoPos} where no row of the bag lies inside the table window.  This is
// what a row shard sends to a bag's owner: the owner keeps the greater value and, among equal
// ones (+0.0 / -0.0), the earlier position, which is torch's first-of-equals rule across shards.
// NaN follows the sequential rule "the bag's first non-padding entry is taken as is, later
// entries only when strictly greater": a NaN is taken only when its entry is that first one
// (every shard scans every index, so each knows where the bag's first non-padding entry is).
// One lane group per bag, the survivor mask of a block of `lanes` indices walked four rows at
// a time; rows wider than the group are covered by further column tiles (blockIdx.y).
constexpr int kNoPos = 0x7fffffff;

template <typename TW, int VE>
__global__ void __launch_bounds__(kCtaThreads, FWD_EB_MIN_CTAS)
eb_pool_maxpos_kernel(const PoolArgs a) {
  using V = typename Chunk<TW, VE>::type;
  const int lanes_log2 = a.lanes_log2;
  const int lanes = 1 << lanes_log2;
  const unsigned lane = threadIdx.x & 31u;
  const int lig = lane & (lanes - 1);
  const int gbase = lane & ~(lanes - 1);
  const unsigned gmask = lanes == 32 ? kFull : ((1u << lanes) - 1u);
  const long long bag = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> lanes_log2;
  const bool live = bag < a.num_bags;
  const int chunk = blockIdx.y * lanes + lig;
  const bool chunk_ok = chunk < a.nchunks;
  long long start = 0, end = 0;
  if (live) bag_bounds(a, bag, start, end);

  float acc[VE];
  int pos[VE];
#pragma unroll
  for (int e = 0; e < VE; ++e) {
    acc[e] = 0.0f;
    pos[e] = kNoPos;
  }
  bool seen = false;  // a non-padding entry lies before the current block (same in a group)
  const unsigned stride32 = (unsigned)a.row_bytes_stride;
  for (long long base = start; __any_sync(kFull, base < end); base += lanes) {
    const long long at = base + lig;
    int row = -1;
    bool counted = false;
    if (at < end) {
      const long long idx = load_index(a.indices, a.idx64, at);
      if (a.padding_idx < 0 || idx != a.padding_idx) {
        counted = true;
        const long long r = idx - a.row_lo;
        if (r >= 0 && r < a.num_rows) row = (int)r;
      }
    }
    unsigned m = (__ballot_sync(kFull, row >= 0) >> gbase) & gmask;
    const unsigned cm = (__ballot_sync(kFull, counted) >> gbase) & gmask;
    while (__any_sync(kFull, m != 0u)) {
      int r4[4], e4[4];
      bool ok[4];
      V val[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        ok[u] = m != 0u;
        e4[u] = ok[u] ? (__ffs(m) - 1) : 0;
        m &= (m - 1u);
        r4[u] = __shfl_sync(kFull, row, gbase + e4[u]);
        if (ok[u] && chunk_ok)
          val[u] = load_chunk<V>(a.table + (unsigned long long)(unsigned)r4[u] * stride32 +
                                 (size_t)chunk * (VE * sizeof(TW)));
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (ok[u] && chunk_ok) {
          float f[VE];
          unpack(val[u], f);
          // is this entry the bag's first non-padding one?
          const bool first_entry = !seen && (cm & ((1u << e4[u]) - 1u)) == 0u;
          const int p = (int)(base - start) + e4[u];
#pragma unroll
          for (int e = 0; e < VE; ++e) {
            const bool take = pos[e] == kNoPos ? (f[e] == f[e] || first_entry) : f[e] > acc[e];
            acc[e] = take ? f[e] : acc[e];
            pos[e] = take ? p : pos[e];
          }
        }
      }
    }
    seen = seen || cm != 0u;
  }
  if (live && chunk_ok) {
    int2* dst = reinterpret_cast<int2*>(a.out) + bag * a.out_stride + (long long)chunk * VE;
#pragma unroll
    for (int e = 0; e < VE; ++e) dst[e] = make_int2(__float_as_int(acc[e]), pos[e]);
  }
}

// ---- strategies 2 and 3: a CTA (or `splits` CTAs) per bag --------------------
// Lane groups take consecutive slices of the bag (of the split's part of it),
// stage their fp32 partials in shared memory and thread t folds column t over
// the groups in slice order, which keeps both the summation order fixed and the
// first-of-equals rule for max.  With splits > 1 the folded partial goes to the
// scratch arrays instead of the output and eb_split_finish_kernel completes it.
template <typename TW, int VE, int CPL, int OP, int U, int IPL>
__global__ void __launch_bounds__(kCtaThreads, FWD_EB_MIN_CTAS)
eb_pool_cta_kernel(const PoolArgs a) {
  extern __shared__ float smem[];  // [groups][tile_cols] then int[groups][2]
  const int lanes_log2 = a.lanes_log2;
  const int lanes = 1 << lanes_log2;
  const int groups = kCtaThreads >> lanes_log2;
  const int tile_chunks = CPL << lanes_log2;
  const int tile_cols = tile_chunks * VE;
  const int chunk0 = blockIdx.y * tile_chunks;
  const long long bag = blockIdx.x / a.splits;
  const int split = blockIdx.x % a.splits;
  const int g = threadIdx.x >> lanes_log2;
  const int lig = (threadIdx.x & 31u) & (lanes - 1);

  long long bstart, bend;
  bag_bounds(a, bag, bstart, bend);
  const long long blen = bend - bstart;
  // slice of this split, then of this group: whole multiples of U indices (a pass), so short
  // bags still spread over several groups
  const long long total_slices = (long long)a.splits * groups;
  long long per = (blen + total_slices - 1) / total_slices;
  per = (per + U - 1) / U * U;
  const long long slot = (long long)split * groups + g;
  long long start = bstart + slot * per;
  long long end = start + per;
  if (start > bend) start = bend;
  if (end > bend) end = bend;

  Accum<CPL, VE> s;
  clear(s);
  if (OP == kOpMax && slot > 0) seed_max_slice<CPL, VE, TW>(s);
  pool_range<TW, VE, CPL, OP, U, IPL>(a, start, end, chunk0, s);

  float* part = smem;
  int* meta = reinterpret_cast<int*>(smem + (size_t)groups * tile_cols);
#pragma unroll
  for (int c = 0; c < CPL; ++c) {
    int chunk_in_tile = c * lanes + lig;
#pragma unroll
    for (int e = 0; e < VE; ++e) part[(size_t)g * tile_cols + chunk_in_tile * VE + e] = s.v[c][e];
  }
  if (lig == 0) {
    meta[2 * g] = s.counted;
    meta[2 * g + 1] = s.have ? 1 : 0;
  }
  __syncthreads();

  int counted = 0;
  for (int k = 0; k < groups; ++k) counted += meta[2 * k];
  const bool tf16 = sizeof(TW) == 2;
  for (int col = threadIdx.x; col < tile_cols; col += kCtaThreads) {
    const long long gcol = (long long)chunk0 * VE + col;
    if (gcol >= a.dim) continue;
    float acc = 0.0f;
    bool have = false;
    for (int k = 0; k < groups; ++k) {
      if (!meta[2 * k + 1]) continue;
      float x = part[(size_t)k * tile_cols + col];
      if (OP == kOpMax) {
        acc = (!have || x > acc) ? x : acc;
      } else {
        acc = have ? __fadd_rn(acc, x) : x;
      }
      have = true;
    }
    if (a.splits > 1) {
      a.ws_acc[(bag * a.splits + split) * a.dim + gcol] = acc;
    } else {
      acc = finish(a, acc, counted, blen, tf16);
      if (a.out_f16) {
        reinterpret_cast<__half*>(a.out)[bag * a.out_stride + gcol] = __float2half_rn(acc);
      } else {
        reinterpret_cast<float*>(a.out)[bag * a.out_stride + gcol] = acc;
      }
    }
  }
  if (a.splits > 1 && threadIdx.x == 0 && blockIdx.y == 0) {
    int have_any = 0;
    for (int k = 0; k < groups; ++k) have_any |= meta[2 * k + 1];
    a.ws_meta[(bag * a.splits + split) * 2] = counted;
    a.ws_meta[(bag * a.splits + split) * 2 + 1] = have_any;
  }
}

// Folds the `splits` partials of every bag in split order; one thread per
// output element.
template <int OP>
__global__ void __launch_bounds__(kCtaThreads)
eb_split_finish_kernel(const PoolArgs a, int table_f16) {
  const long long t = (long long)blockIdx.x * kCtaThreads + threadIdx.x;
  if (t >= a.num_bags * a.dim) return;
  const long long bag = t / a.dim;
  const int col = (int)(t - bag * a.dim);
  float acc = 0.0f;
  bool have = false;
  int counted = 0;
  for (int sidx = 0; sidx < a.splits; ++sidx) {
    const long long slot = bag * a.splits + sidx;
    counted += a.ws_meta[2 * slot];
    if (!a.ws_meta[2 * slot + 1]) continue;
    float x = a.ws_acc[slot * a.dim + col];
    if (OP == kOpMax) {
      acc = (!have || x > acc) ? x : acc;
    } else {
      acc = have ? __fadd_rn(acc, x) : x;
    }
    have = true;
  }
  long long bstart, bend;
  bag_bounds(a, bag, bstart, bend);
  acc = finish(a, acc, counted, bend - bstart, table_f16 != 0);
  if (a.out_f16) {
    reinterpret_cast<__half*>(a.out)[bag * a.out_stride + col] = __float2half_rn(acc);
  } else {
    reinterpret_cast<float*>(a.out)[bag * a.out_stride + col] = acc;
  }
}

// ---- gather: out[t, :] = table[indices[t] - row_lo, :] -----------------------
// One lane group per index; skipped indices give a zero row (or are left alone
// when keep_skipped is set, the reference behaviour).
template <typename TW, int VE>
__global__ void __launch_bounds__(kCtaThreads)
eb_gather_kernel(const PoolArgs a, int keep_skipped) {
  using V = typename Chunk<TW, VE>::type;
  const int lanes = 1 << a.lanes_log2;
  const int lig = (threadIdx.x & 31u) & (lanes - 1);
  const long long t = ((long long)blockIdx.x * kCtaThreads + threadIdx.x) >> a.lanes_log2;
  if (t >= a.num_indices) return;
  const long long idx = load_index(a.indices, a.idx64, t);
  const long long r = idx - a.row_lo;
  const bool ok = (a.padding_idx < 0 || idx != a.padding_idx) && r >= 0 && r < a.num_rows;
  if (!ok && keep_skipped) return;
  const char* rp = a.table + (ok ? r : 0) * a.row_bytes_stride;
  for (int chunk = lig; chunk < a.nchunks; chunk += lanes) {
    float f[1][VE];
    if (ok) {
      V v = load_chunk<V>(rp + (long long)chunk * VE * (int)sizeof(TW));
      unpack(v, f[0]);
    } else {
#pragma unroll
      for (int e = 0; e < VE; ++e) f[0][e] = 0.0f;
    }
    // store_row addresses chunk0 + lig; hand it the chunk minus this lane's slot
    store_row<VE, 1, false>(a, a.out, t, chunk - lig, f, true);
  }
}

// ---- helpers ---------------------------------------------------------------

__host__ __device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// Sum of eight 16-bit uniforms, centred and scaled to unit variance: integer
// arithmetic up to the last two multiplies, so the host twin gives the same bits.
__host__ __device__ __forceinline__ float table_value(unsigned long long seed, long long row,
                                                      int col, float scale) {
  unsigned long long a =
      mix64(seed ^ mix64((unsigned long long)row * 0xD1342543DE82EF95ull + (unsigned)col));
  unsigned long long b = mix64(a);
  int s = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    s += (int)((a >> (16 * i)) & 0xFFFFu);
    s += (int)((b >> (16 * i)) & 0xFFFFu);
  }
  s -= 4 * 65535;
  const float inv_sigma = 1.0f / 53509.92f;
#ifdef __CUDA_ARCH__
  return __fmul_rn(__fmul_rn((float)s, inv_sigma), scale);
#else
  float unit = (float)s * inv_sigma;
  return unit * scale;
#endif
}

template <typename TW>
__global__ void __launch_bounds__(kCtaThreads)
eb_fill_table_kernel(TW* table, long long num_rows, int dim, long long row_lo,
                     unsigned long long seed, float scale) {
  const long long total = num_rows * dim;
  for (long long t = (long long)blockIdx.x * kCtaThreads + threadIdx.x; t < total;
       t += (long long)gridDim.x * kCtaThreads) {
    const long long r = t / dim;
    const int c = (int)(t - r * dim);
    const float v = table_value(seed, row_lo + r, c, scale);
    if (sizeof(TW) == 2) {
      reinterpret_cast<__half*>(table)[t] = __float2half_rn(v);
    } else {
      reinterpret_cast<float*>(table)[t] = v;
    }
  }
}

static __global__ void __launch_bounds__(kCtaThreads)
eb_cast_i64_i32_kernel(const long long* src, int* dst, long long count) {
  for (long long i = (long long)blockIdx.x * kCtaThreads + threadIdx.x; i < count;
       i += (long long)gridDim.x * kCtaThreads) {
    const long long v = src[i];
    dst[i] = (v >= -2147483647LL - 1 && v <= 2147483647LL) ? (int)v : -1;
  }
}

template <typename TP, typename TO>
__global__ void __launch_bounds__(kCtaThreads)
eb_combine_partials_kernel(const TP* parts, int num_parts, long long part_stride, long long count,
                           TO* out) {
  for (long long i = (long long)blockIdx.x * kCtaThreads + threadIdx.x; i < count;
       i += (long long)gridDim.x * kCtaThreads) {
    float s = 0.0f;
    for (int r = 0; r < num_parts; ++r) {
      float x;
      if (sizeof(TP) == 2) {
        x = __half2float(reinterpret_cast<const __half*>(parts)[r * part_stride + i]);
      } else {
        x = reinterpret_cast<const float*>(parts)[r * part_stride + i];
      }
      s = __fadd_rn(s, x);
    }
    if (sizeof(TO) == 2) {
      reinterpret_cast<__half*>(out)[i] = __float2half_rn(s);
    } else {
      reinterpret_cast<float*>(out)[i] = s;
    }
  }
}

}  // namespace fwd_eb
