// Two variants of the lean lane-group kernel (eb_lite.cuh) that stage table rows through shared
// memory instead of loading them straight into registers.  They exist to answer one question
// with numbers: does an asynchronous copy into shared memory (cp.async, or the bulk copy engine,
// cp.async.bulk = TMA's 1-D form) buy anything for a gather of 128..512-byte rows?  It does not
// (profiles/row_staging_variants.md has the timings and counters), so the default build does not
// contain them: they are compiled only with -DFWD_EB_ROW_STAGING=1 (cp.async) or =2
// (cp.async.bulk), and then FWD_EB_STRATEGY_LITE runs the staged kernel instead of the register
// one.  Single-GPU code: every copy reads this GPU's own table and there is no multicast form.
//
//   =1  every lane issues `cp.async.cg.shared.global` of its 16-byte chunk for each of the U rows
//       of a pass, commits the group, waits for it (cp.async.wait_group 0) and folds the rows
//       from shared memory;
//   =2  lane 0 of a group arms an mbarrier with the pass's byte count and issues one
//       `cp.async.bulk.shared::cluster.global` per row (row start and size are multiples of 16
//       bytes, as the vector path guarantees); the group waits on the mbarrier's phase with a
//       bounded number of polls and folds the rows from shared memory.  When a wait runs out
//       the group skips the pass and issues no further copies — it never hangs.
//
// Same shapes, same order of additions, same results as eb_pool_lite_kernel.
#pragma once

#if defined(FWD_EB_ROW_STAGING) && FWD_EB_ROW_STAGING > 0

#include "eb_kernels.cuh"

namespace fwd_eb {

constexpr int kStagedPass = 8;              // rows per pass, as kLitePass
constexpr int kStagedSpinLimit = 1 << 20;   // mbarrier polls before a group gives a pass up

__device__ __forceinline__ unsigned smem_addr(const void* p) {
  return (unsigned)__cvta_generic_to_shared(p);
}

template <typename TW, int VE, int LL, int OP>
__global__ void __launch_bounds__(kCtaThreads, FWD_EB_MIN_CTAS)
eb_pool_lite_staged_kernel(const PoolArgs a) {
  using V = typename Chunk<TW, VE>::type;
  constexpr int LANES = 1 << LL;
  constexpr int U = kStagedPass;
  constexpr int GROUPS = kCtaThreads / LANES;
  constexpr unsigned GMASK = LANES == 32 ? kFull : ((1u << LANES) - 1u);
  // per group: U rows of LANES * 16 bytes
  __shared__ __align__(128) unsigned char s_rows[GROUPS * U * LANES * 16];
#if FWD_EB_ROW_STAGING == 2
  __shared__ __align__(8) unsigned long long s_bar[GROUPS];
#endif
  const unsigned lane = threadIdx.x & 31u;
  const int lig = lane & (LANES - 1);
  const int gbase = lane & ~(LANES - 1);
  const int group = threadIdx.x >> LL;
  unsigned char* rows = s_rows + (size_t)group * U * LANES * 16;
  const int bag = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) >> LL);
  const bool live = bag < a.num_bags;
#if FWD_EB_ROW_STAGING == 2
  if (lig == 0) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&s_bar[group])));
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  __syncwarp();
  unsigned phase = 0;
  bool dead = false;  // a wait ran out: this group issues no further copies and skips its rows
#endif
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
    start = start < 0 ? 0 : start;
    end = end > n_idx ? n_idx : end;
    end = end < start ? start : end;
  }
  const bool chunk_ok = lig < a.nchunks;
  const unsigned stride32 = (unsigned)a.row_bytes_stride;
  const unsigned row_bytes = (unsigned)a.nchunks * 16u;

  float acc[VE];
#pragma unroll
  for (int e = 0; e < VE; ++e) acc[e] = 0.0f;
  int counted = 0;
  bool have = false;

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
    fetch(base + LANES + lig, nrow, nw);
    if (a.mean) counted += __popc((__ballot_sync(kFull, row >= -1) >> gbase) & GMASK);
    const int n = end - base;
#pragma unroll
    for (int k = 0; k < LANES; k += U) {
      if (!__any_sync(kFull, k < n)) break;
      float wu[U];
      unsigned ok = 0u;
      int r[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        r[u] = __shfl_sync(kFull, row, gbase + ((k + u) & (LANES - 1)));
        if (OP == kOpWeighted) wu[u] = __shfl_sync(kFull, w, gbase + ((k + u) & (LANES - 1)));
        const bool take = k + u < n && k + u < LANES && r[u] >= 0;
        ok |= (take ? 1u : 0u) << u;
      }
      __syncwarp();  // the previous pass has been read out of the staging slots
#if FWD_EB_ROW_STAGING == 1
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (((ok >> u) & 1u) && chunk_ok) {
          const char* src = a.table + (unsigned long long)(unsigned)r[u] * stride32 + lig * 16;
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(rows + (u * LANES + lig) * 16)),
                       "l"(src)
                       : "memory");
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncwarp();
#else
      bool arrived = true;
      if (dead) ok = 0u;
      if (lig == 0 && ok) {
        const unsigned bytes = (unsigned)__popc(ok) * row_bytes;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(&s_bar[group])),
                     "r"(bytes)
                     : "memory");
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if ((ok >> u) & 1u) {
            const char* src = a.table + (unsigned long long)(unsigned)r[u] * stride32;
            asm volatile(
                "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                    smem_addr(rows + u * LANES * 16)),
                "l"(src), "r"(row_bytes), "r"(smem_addr(&s_bar[group]))
                : "memory");
          }
        }
      }
      if (ok) {  // every lane of the group waits for the phase (bounded)
        unsigned done = 0;
        // two rounds of polls: the second gives copies still in flight time to land before the
        // group gives up for good
        for (int spin = 0; spin < 2 * kStagedSpinLimit && !done; ++spin) {
          asm volatile(
              "{\n\t.reg .pred p;\n\t"
              "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
              "selp.u32 %0, 1, 0, p;\n\t}"
              : "=r"(done)
              : "r"(smem_addr(&s_bar[group])), "r"(phase)
              : "memory");
        }
        arrived = done != 0;
        phase ^= 1u;
      }
      if (!arrived) {  // gave up: the pass is skipped, nothing is read from the slots
        ok = 0u;
        dead = true;
      }
#endif
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (((ok >> u) & 1u) && chunk_ok) {
          const V val = *reinterpret_cast<const V*>(rows + (u * LANES + lig) * 16);
          fold_chunk<OP>(acc, val, OP == kOpWeighted ? wu[u] : 1.0f, !have);
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
  store_row<VE, 1, true>(a, a.out, bag, 0, v, live);
}

}  // namespace fwd_eb

#endif  // FWD_EB_ROW_STAGING
