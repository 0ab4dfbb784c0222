// Device-side building blocks of the sm_100a top-2048 selector: PTX wrappers (mbarrier, bulk
// async copy), warp/block scans that pick a threshold bin, the histogram update, and the
// single-CTA "finish" that resolves a small candidate list held in shared memory.
#pragma once
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fftopk_key.h"

namespace fftopk {

namespace cg = cooperative_groups;

constexpr int kK = 2048;               // reference: TopK (topk_indexer_radix.cu:69)
constexpr int kMaxBins = 4096;         // widest digit of the distributed rounds: 12 bits
constexpr int kSup = 64;               // super-bins per histogram (each sums kMaxBins/64 bins)
constexpr int kMaxCluster = 16;        // CTAs per row (non-portable cluster size on B200)
constexpr int kChunks = 16;            // bulk-copy chunks (one mbarrier each) per staged shard
constexpr int kFinishBits = 10;        // digit width of the single-CTA finish
constexpr int kFinishBins = 1 << kFinishBits;
constexpr int kSmall = 32;             // candidates resolved by one warp's compare-exchange network
constexpr unsigned kFull = 0xffffffffu;
constexpr int kWaitLimit = 1 << 16;    // bound on mbarrier polls before giving up on staging

#ifndef FFTOPK_HIST_POLICY
#define FFTOPK_HIST_POLICY 1           // 0 plain atomics, 1 leader-bin ballot, 2 match.any
#endif

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait: false when the limit ran out (the caller then reads global memory instead).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  for (int i = 0; i < kWaitLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}

// 1-D bulk async copy global -> this CTA's shared memory (TMA engine, no multicast). `bytes` is
// a multiple of 16 and both addresses are 16-byte aligned.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

// ---------------------------------------------------------------------------------------------
// Histogram update. Must be called by all 32 lanes of a warp together (inactive lanes pass
// valid = false). Counters are 32-bit in shared memory.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void hist_add(uint32_t* hist, uint32_t bin, bool valid) {
#if FFTOPK_HIST_POLICY == 0
  if (valid) atomicAdd(&hist[bin], 1u);
#elif FFTOPK_HIST_POLICY == 1
  // Lanes that share lane 0's bin are counted with one atomic: removes the serialisation a
  // dominant bin (a spike of equal values, a skewed exponent bucket) would otherwise cause.
  const uint32_t mine = valid ? bin : 0xffffffffu;
  const uint32_t lead = __shfl_sync(kFull, mine, 0);
  const bool same = valid && (mine == lead);
  const unsigned m = __ballot_sync(kFull, same);
  if (same) {
    if (lane_id() == 0) atomicAdd(&hist[bin], (uint32_t)__popc(m));
  } else if (valid) {
    atomicAdd(&hist[bin], 1u);
  }
#else
  const unsigned act = __ballot_sync(kFull, valid);
  if (valid) {
    const unsigned m = __match_any_sync(act, bin);
    if (lane_id() == (__ffs(m) - 1)) atomicAdd(&hist[bin], (uint32_t)__popc(m));
  }
#endif
}

// ---------------------------------------------------------------------------------------------
// Warp-level threshold pick over 64 counts in descending bin order. Lane l holds the counts of
// bins 2l (lo) and 2l+1 (hi). Finds the bin t with
//     above(t) < need <= above(t) + count[t],   above(t) = sum of count[j], j > t.
// This is the reference's "S[t] > k >= S[t+1]" rule (topk_indexer_radix.cu:555-566) computed with
// a shuffle suffix scan instead of eight block-wide doubling steps. Returns false if the counts
// sum to less than `need`.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ bool warp_pick64(uint32_t lo, uint32_t hi, uint32_t need, int& t, uint32_t& above,
                                            uint32_t& cnt) {
  const int lane = lane_id();
  const uint32_t s = lo + hi;
  uint32_t incl = s;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t v = __shfl_down_sync(kFull, incl, off);
    if (lane + off < 32) incl += v;
  }
  const uint32_t excl = incl - s;  // counts in lanes above this one
  const bool hit_hi = (excl < need) && (need <= excl + hi);
  const bool hit_lo = (excl + hi < need) && (need <= excl + hi + lo);
  const unsigned m = __ballot_sync(kFull, hit_hi || hit_lo);
  if (m == 0) return false;
  const int src = __ffs(m) - 1;
  t = __shfl_sync(kFull, hit_hi ? 2 * lane + 1 : 2 * lane, src);
  above = __shfl_sync(kFull, hit_hi ? excl : excl + hi, src);
  cnt = __shfl_sync(kFull, hit_hi ? hi : lo, src);
  return true;
}

__device__ __forceinline__ uint32_t warp_sum(uint32_t v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(kFull, v, off);
  return v;
}

// Descending bitonic compare-exchange network over one 64-bit value per lane.
__device__ __forceinline__ uint64_t warp_sort_desc(uint64_t c) {
  const int lane = lane_id();
#pragma unroll
  for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      const uint64_t other = __shfl_xor_sync(kFull, c, j);
      const bool lower = (lane & j) == 0;
      const bool desc_block = (lane & k) == 0;
      const bool keep_max = (lower == desc_block);
      const uint64_t mx = c > other ? c : other;
      const uint64_t mn = c > other ? other : c;
      c = keep_max ? mx : mn;
    }
  }
  return c;
}

// ---------------------------------------------------------------------------------------------
// Shared-memory control block (one per CTA; rank 0's counters are the cluster-wide ones).
// ---------------------------------------------------------------------------------------------
struct Ctrl {
  uint64_t mbar[kChunks];
  // cluster-wide allocation counters, meaningful in rank 0 only (targets of remote atomics)
  uint32_t win_count;
  uint32_t cand_count;
  // per-scan local slot counters
  uint32_t wslot;
  uint32_t cslot;
  uint32_t fslot;
  uint32_t small_n;
  // result of the most recent threshold search
  int32_t t;
  uint32_t above;
  uint32_t cnt;
  int32_t sup_sel;
  uint32_t sup_above;
  int32_t mode;
  uint32_t base_w;
  uint32_t base_c;
  uint32_t tie_prefix;
  uint32_t local_c;
  uint32_t stage_fail;
  uint32_t run_total;
  uint32_t wtot[32];
  uint64_t small[kSmall];
};

// Block-wide threshold pick over kFinishBins counts (descending bin order); result in ctrl->t
// (-1 if the counts sum to less than need), ctrl->above, ctrl->cnt. Ends with a barrier.
template <int NT>
__device__ __forceinline__ void block_pick(const uint32_t* hist, uint32_t need, Ctrl* ctrl) {
  constexpr int PER = (kFinishBins + NT - 1) / NT;
  constexpr int NW = NT / 32;
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  uint32_t v[PER];
  uint32_t s = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int b = tid * PER + j;
    v[j] = (b < kFinishBins) ? hist[b] : 0u;
    s += v[j];
  }
  uint32_t incl = s;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t x = __shfl_down_sync(kFull, incl, off);
    if (lane + off < 32) incl += x;
  }
  if (lane == 0) ctrl->wtot[warp] = incl;
  if (tid == 0) ctrl->t = -1;
  __syncthreads();
  const uint32_t hw = (lane > warp && lane < NW) ? ctrl->wtot[lane] : 0u;
  const uint32_t higher = warp_sum(hw);
  uint32_t run = higher + incl - s;
#pragma unroll
  for (int j = PER - 1; j >= 0; --j) {
    if (run < need && need <= run + v[j]) {
      ctrl->t = tid * PER + j;
      ctrl->above = run;
      ctrl->cnt = v[j];
    }
    run += v[j];
  }
  __syncthreads();
}

// ---------------------------------------------------------------------------------------------
// Single-CTA finish. `cand` holds n composites c = (key << 32) | ~idx in shared memory; entries
// equal to 0 are empty. All non-empty composites agree on the bits at and above `hi`
// (their value there is `pfx`; hi == 64 means no common prefix). Writes the `need` largest
// composites' indices (and keys) to out_idx[out_base ...], in unspecified order.
//
// Replaces the reference's refinement rounds on shared-memory survivors and its CAS insertion
// tail (topk_indexer_radix.cu:686-781, 109-141, 788-850). Because the index is part of the
// composite, equal values are resolved towards the lower index by the same radix passes, and
// the last <= 32 undecided candidates go through a warp compare-exchange network.
// `idx_bits`: all indices are < 2^idx_bits, so the inverted-index bits above that are all ones.
// ---------------------------------------------------------------------------------------------
template <int NT>
__device__ void cta_finish(const uint64_t* cand, int n, uint32_t need, int hi, uint64_t pfx, int idx_bits,
                           uint32_t* hist /* >= kFinishBins words */, Ctrl* ctrl, int32_t* out_idx, uint32_t* out_key,
                           uint32_t out_base, int32_t idx_offset, uint32_t* status) {
  const int tid = threadIdx.x;
  if (tid == 0) ctrl->fslot = 0;
  // (the barrier inside the first round orders this store before any use)
  auto emit = [&](uint64_t c) {
    const uint32_t pos = out_base + atomicAdd(&ctrl->fslot, 1u);
    if (pos < (uint32_t)kK) {
      out_idx[pos] = (int32_t)(~(uint32_t)c) + idx_offset;
      if (out_key) out_key[pos] = (uint32_t)(c >> 32);
    }
  };
  for (int round = 0; round < 16 && hi > 0; ++round) {
    if (hi <= 32 && hi > idx_bits) {
      // constant run of ones in the inverted index: extend the prefix without a pass
      const int skip = hi - idx_bits;
      pfx = (pfx << skip) | ((1ull << skip) - 1ull);
      hi = idx_bits;
    }
    const int w = hi < kFinishBits ? hi : kFinishBits;
    const int sh = hi - w;
    const uint32_t dmask = (1u << w) - 1u;
    for (int b = tid; b < kFinishBins; b += NT) hist[b] = 0u;
    if (tid == 0) ctrl->small_n = 0;
    __syncthreads();
    for (int i = tid; i < n; i += NT) {
      const uint64_t c = cand[i];
      const bool act = (c != 0ull) && (hi >= 64 || (c >> hi) == pfx);
      if (act) atomicAdd(&hist[(uint32_t)(c >> sh) & dmask], 1u);
    }
    __syncthreads();
    block_pick<NT>(hist, need, ctrl);
    const int t = ctrl->t;
    if (t < 0) {
      if (tid == 0 && status) atomicOr(status, 2u);
      return;
    }
    const uint32_t cnt = ctrl->cnt;
    const uint32_t need2 = need - ctrl->above;
    const bool take_all = (cnt == need2);
    const bool small = !take_all && cnt <= (uint32_t)kSmall;
    for (int i = tid; i < n; i += NT) {
      const uint64_t c = cand[i];
      const bool act = (c != 0ull) && (hi >= 64 || (c >> hi) == pfx);
      if (!act) continue;
      const uint32_t d = (uint32_t)(c >> sh) & dmask;
      if (d > (uint32_t)t) {
        emit(c);
      } else if (d == (uint32_t)t) {
        if (take_all) {
          emit(c);
        } else if (small) {
          const uint32_t s = atomicAdd(&ctrl->small_n, 1u);
          if (s < (uint32_t)kSmall) ctrl->small[s] = c;
        }
      }
    }
    if (take_all) return;
    if (small) {
      __syncthreads();
      if (tid < 32) {
        uint64_t c = (tid < (int)cnt) ? ctrl->small[tid] : 0ull;
        c = warp_sort_desc(c);
        if ((uint32_t)tid < need2) emit(c);
      }
      return;
    }
    pfx = (hi >= 64) ? (uint64_t)t : ((pfx << w) | (uint64_t)t);
    hi = sh;
    need = need2;
    __syncthreads();  // every thread has read ctrl->t/cnt/above before the next round rewrites them
  }
}

}  // namespace fftopk
