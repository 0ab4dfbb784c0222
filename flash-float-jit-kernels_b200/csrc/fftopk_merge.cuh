// Merge of per-shard top-2048 candidate lists by one thread-block cluster per row (context-parallel
// mode). Used by the stand-alone merge kernel and by the selection kernel that merges in the same
// launch.
#pragma once
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fftopk_device.cuh"

namespace fftopk {

constexpr int kMaxShards = 8;

// Where the candidates of each shard live, and (fused mode) the flag that says they are there.
struct MergeSrc {
  const int32_t* idx[kMaxShards];
  const uint32_t* key[kMaxShards];
  const uint32_t* flag[kMaxShards];  // nullptr: no wait
  uint32_t epoch;                    // epoch to wait for; 0 with own_flag set: read it from own_flag
  const uint32_t* own_flag;          // this rank's published epoch (device-side epochs)
  int64_t half_words;                // device-side epochs: idx/key point at half 0, add (e & 1) * half_words
  int64_t flag_row_stride;           // words between the flags of consecutive rows (0: one flag per launch)
  unsigned long long wait_ns;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Candidate packet of the single-launch mode: {global index, epoch, key, epoch}. The epoch tags
// make a packet self-validating: a reader that finds both tags equal to the epoch it expects has
// the index and the key of that epoch, whatever order the stores arrived in (each 8-byte half is
// written atomically), so the exchange needs neither a flag nor a fence.
__device__ __forceinline__ void st_packet(uint4* p, int32_t idx, uint32_t key, uint32_t epoch) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"((uint32_t)idx), "r"(epoch), "r"(key), "r"(epoch)
               : "memory");
}
__device__ __forceinline__ uint4 ld_packet(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Shared memory a CTA brings to the merge of one row.
struct MergeSmem {
  uint32_t* hist;  // 2 * kMaxBins words: the histogram of the top 12 key bits, then the finer one (bits [27:16])
  uint32_t* sup;   // 2 * kSup words
  uint32_t* xch;   // kMaxCluster * kSup words
  Ctrl* ctrl;
  uint64_t* cand;  // the first CTA's gather area (the same offset in every CTA)
  int32_t cand_cap;
};

// What decide_and_allocate needs to know about a merge cluster.
struct MergeCtx {
  Ctrl* ctrl;
  Ctrl* ctrl0;
  int32_t cand_cap;
};

// Merge of one row by a cluster: the selector's exact path run over candidate lists. The first G
// CTAs of the cluster (ranks 0..G-1) own one shard each; every CTA of the cluster calls this
// function, the others only take part in its two cluster barriers.
// CTA g waits (fused mode, bounded) for shard g's epoch flag and pulls that shard's 2048
// (key, global index) candidates of the row into registers - from local memory after an
// all-gather, from the owner's memory over NVLink in fused mode, G CTAs pulling in parallel - and
// histograms their top 12 key bits and, 16 times finer, key bits [27:16] (candidate lists are the
// upper tail of a row: they nearly always share their top four key bits, and then the finer
// histogram is the one searched). After ONE cluster barrier every CTA finds the threshold bin
// from its peers' histograms over distributed shared memory (cluster_pick), writes its own
// candidates above that bin straight to the output and sends those inside it to the first CTA,
// which after the second cluster barrier finishes on that one bin with a known key range - by
// direct ranking when the bin holds at most 256 candidates.
// Composites carry the inverted global index, so equal values resolve to the lower global index.
//   sidx, skey  shard g's candidates of this row (ranks >= G: unused)
//   sflag       shard g's epoch flag, or nullptr for "no wait"
//   packets     single-launch mode instead of the three above: shard g's 2048 packets of this row in
//               THIS GPU's inbox (the owner pushes them); the CTA polls them until every tag shows
//               `epoch`
// A wait that runs out fills the row with -1, raises FFTOPK_ST_PEER_TIMEOUT and returns normally.
// kTrackMin / thr_out: the key of the row's 2048-th largest candidate (or, where the whole threshold
// bin won without a finish, the bin's lower edge - a lower bound of it) is written to *thr_out.
template <int NT, bool kTrackMin = false>
__device__ __forceinline__ void merge_row(cg::cluster_group& cluster, int C, int G, int g, const MergeSmem& sm,
                                          const int32_t* sidx, const uint32_t* skey, const uint32_t* sflag,
                                          const uint4* packets, uint32_t epoch, unsigned long long wait_ns,
                                          int32_t* __restrict__ out_idx, uint32_t* __restrict__ out_key, uint32_t* status,
                                          uint32_t* thr_out = nullptr) {
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  constexpr int NW = NT / 32;
  constexpr int PER = kK / NT;
  uint32_t* hist = sm.hist;
  Ctrl* ctrl = sm.ctrl;
  if (g >= G) {  // not a shard owner: keep the cluster's barriers company
    cluster_sync(cluster, C);
    cluster_sync(cluster, C);
    return;
  }
  MergeCtx cx;
  cx.ctrl = ctrl;
  cx.ctrl0 = C == 1 ? ctrl : cluster.map_shared_rank(ctrl, 0);
  cx.cand_cap = sm.cand_cap;
  uint64_t* cand0 = C == 1 ? sm.cand : cluster.map_shared_rank(sm.cand, 0);
  {
    uint4* h4 = reinterpret_cast<uint4*>(hist);
    for (int i = tid; i < 2 * kMaxBins / 4; i += NT) h4[i] = make_uint4(0u, 0u, 0u, 0u);
    if (tid < kSup) {
      ctrl->tot[0][tid] = 0u;  // (the buffers with index 1 are cleared by the search)
      ctrl->tot2[0][tid] = 0u;
      ctrl->totb[tid] = 0u;
    }
    if (tid == 0) {
      ctrl->merge_fail = 0u;
      ctrl->win_count = 0u;   // (rank 0's counters are the cluster's; nobody adds to them before
      ctrl->cand_count = 0u;  //  the cluster barrier below)
      ctrl->wslot = 0u;
      ctrl->cslot = 0u;
      ctrl->fslot = 0u;
      if constexpr (kTrackMin) ctrl->thr_key = 0xffffffffu;
#ifdef FFTOPK_CHECKED
      ctrl->status_ptr = status;
#endif
    }
  }
  __syncthreads();
  int32_t idx[PER];
  uint32_t key[PER];
  if (packets != nullptr) {
    // Single-launch mode: poll the shard's packets in this GPU's own memory until all of them carry
    // this epoch. Bounded: when the time runs out the row is filled with -1, a status bit is raised
    // and the kernel returns normally, so a peer that never arrives cannot hang this GPU.
    const unsigned long long t0 = global_timer_ns();
    for (;;) {
      bool ok = true;
#pragma unroll
      for (int u = 0; u < PER; ++u) {
        const uint4 v = ld_packet(packets + u * NT + tid);
        idx[u] = (int32_t)v.x;
        key[u] = v.z;
        ok = ok && v.y == epoch && v.w == epoch;
      }
      if (__syncthreads_and(ok)) break;
      const bool expired = tid == 0 && (global_timer_ns() - t0 > wait_ns);
      if (__syncthreads_or(expired)) {
        if (tid == 0) ctrl->merge_fail = 1u;
        break;
      }
    }
    __syncthreads();
    if (ctrl->merge_fail != 0u) {
#pragma unroll
      for (int u = 0; u < PER; ++u) {
        idx[u] = -1;
        key[u] = 0u;
      }
    }
  } else {
    // Two-launch mode: one thread waits until the shard's owner has published this epoch (bounded
    // in the same way), then the CTA pulls the candidates.
    if (tid == 0 && sflag != nullptr) {
      const unsigned long long t0 = global_timer_ns();
      bool ok = false;
      for (;;) {
        if ((int32_t)(ld_acquire_sys(sflag) - epoch) >= 0) {
          ok = true;
          break;
        }
        if (global_timer_ns() - t0 > wait_ns) break;
        __nanosleep(64);
      }
      if (!ok) ctrl->merge_fail = 1u;
    }
    __syncthreads();
    const bool failed = ctrl->merge_fail != 0u;  // (uniform over the CTA)
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      idx[u] = -1;
      key[u] = 0u;
      if (!failed) {
        // L2-coherent loads: the data may have been written by another GPU a moment ago
        idx[u] = __ldcg(sidx + u * NT + tid);
        key[u] = __ldcg(skey + u * NT + tid);
      }
    }
  }
  FFTOPK_MARK(62);
  uint32_t cnt = 0;
#pragma unroll
  for (int u = 0; u < PER; ++u) {
    const bool v = idx[u] >= 0;
    cnt += v ? 1u : 0u;
    hist_add(hist, key[u] >> 20, v);
    hist_add(hist + kMaxBins, (key[u] >> 16) & 0xfffu, v);
  }
  cnt = __reduce_add_sync(kFull, cnt);
  if (lane == 0) ctrl->wtot[warp] = cnt;
  __syncthreads();
  compute_sup<NT>(hist, sm.sup, kMaxBins);
  compute_sup<NT>(hist + kMaxBins, sm.sup + kSup, kMaxBins);
  if (warp == 0) {
    const uint32_t c = __reduce_add_sync(kFull, lane < NW ? ctrl->wtot[lane] : 0u);
    if (lane == 0) ctrl->merge_count = c;
  }
  FFTOPK_MARK(63);
  cluster_sync(cluster, C);  // #1: every shard's histogram and record are complete
  FFTOPK_MARK(64);
  // ---- every shard owner reads all records ----------------------------------------------------
  if (warp == 0) {
    uint32_t rc = 0u, rf = 0u;
    if (lane < G) {
      const Ctrl* rctrl = C == 1 ? ctrl : cluster.map_shared_rank(ctrl, lane);
      rc = rctrl->merge_count;
      rf = rctrl->merge_fail;
    }
    const uint32_t total = __reduce_add_sync(kFull, rc);
    const uint32_t before = __reduce_add_sync(kFull, lane < g ? rc : 0u);
    const uint32_t anyfail = __reduce_max_sync(kFull, rf);
    if (lane == 0) {
      ctrl->run_total = total;
      ctrl->tie_prefix = before;
      ctrl->pub_flag = anyfail;
    }
  }
  __syncthreads();
  const uint32_t total = ctrl->run_total;
  if (ctrl->pub_flag) {
    if (g == 0) {
      for (int i = tid; i < kK; i += NT) {
        out_idx[i] = -1;
        if (out_key) out_key[i] = 0u;
      }
      if (tid == 0 && status) atomicOr(status, (uint32_t)FFTOPK_ST_PEER_TIMEOUT);
    }
    cluster_sync(cluster, C);  // nobody leaves while a peer may still be reading its record
    return;
  }
  if (total <= (uint32_t)kK) {
    // no more candidates than k: keep them all, shard after shard, pad with -1
    const uint32_t before = ctrl->tie_prefix;
    uint32_t kmin = 0xffffffffu;
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      if (idx[u] >= 0) {
        const uint32_t pos = before + warp_alloc(&ctrl->fslot);
        if (FFTOPK_CHECK(9, pos, kK, status)) {
          out_idx[pos] = idx[u];
          if (out_key) out_key[pos] = key[u];
        }
        kmin = min(kmin, key[u]);
      }
    }
    if constexpr (kTrackMin) {  // all candidates win: the smallest key is the threshold
      kmin = __reduce_min_sync(kFull, kmin);
      if (lane == 0 && kmin != 0xffffffffu) atomicMin(&cx.ctrl0->thr_key, kmin);
    }
    if (g == 0) {
      for (int i = (int)total + tid; i < kK; i += NT) {
        out_idx[i] = -1;
        if (out_key) out_key[i] = 0u;
      }
    }
    cluster_sync(cluster, C);
    if constexpr (kTrackMin) {
      if (g == 0 && tid == 0 && thr_out != nullptr) *thr_out = total == (uint32_t)kK ? ctrl->thr_key : 0u;
    }
    return;
  }
  // ---- threshold bin over the shard owners; winners out, the bin itself to the first CTA -------
  int pick_no = 0;
  cluster_pick<NT>(
      cluster, G, hist, sm.sup, sm.xch, ctrl, pick_no, kMaxBins, [&](uint32_t) { return (uint32_t)kK; },
      [&](Picked& pk) { decide_and_allocate(cx, pk, kModeAbort, false); }, hist + kMaxBins, sm.sup + kSup);
  FFTOPK_MARK(65);
  const int mode = ctrl->mode;
  // the threshold bin as a key prefix: 12 bits, or 16 when the finer histogram was searched
  const bool fine_bins = ctrl->dual_b != 0u;
  const int pshift = fine_bins ? 16 : 20;
  const uint32_t t = fine_bins ? ((ctrl->dual_g << 12) | (uint32_t)ctrl->t) : (uint32_t)ctrl->t;
  if (mode == kModeGather || mode == kModeTakeAll) {
    const uint32_t base_w = ctrl->base_w, base_c = ctrl->base_c;
    const bool take_eq = mode == kModeTakeAll;
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      if (idx[u] >= 0) {
        const uint32_t bin = key[u] >> pshift;
        if (bin > t || (take_eq && bin == t)) {
          const uint32_t pos = base_w + warp_alloc(&ctrl->wslot);
          if (FFTOPK_CHECK(12, pos, kK, status) && pos < (uint32_t)kK) {
            out_idx[pos] = idx[u];
            if (out_key) out_key[pos] = key[u];
          }
        } else if (bin == t) {
          const uint32_t slot = base_c + warp_alloc(&ctrl->cslot);
          if (FFTOPK_CHECK(8, slot, cx.cand_cap, status) && slot < (uint32_t)cx.cand_cap)
            cand0[slot] = ((uint64_t)key[u] << 32) | (uint64_t)(~(uint32_t)idx[u]);
        }
      }
    }
  }
  FFTOPK_MARK(66);
  cluster_sync(cluster, C);  // #2: the threshold bin's candidates have landed in the first CTA
  FFTOPK_MARK(67);
  if (g != 0) return;
  if (mode == kModeGather) {
    const uint32_t need = ctrl->above;
    const DenseCands<NT> bin_cands{sm.cand, (int)ctrl->cand_count};
    const uint64_t lo = (uint64_t)t << (32 + pshift);
    const uint64_t cap = lo | ((1ull << (32 + pshift)) - 1ull);
    cta_finish<NT, DenseCands<NT>, kTrackMin>(bin_cands, need, lo, cap, cap, false, 31, hist, ctrl, out_idx, out_key,
                                              (uint32_t)kK - need, (uint32_t)kK, 0, status, nullptr, ctrl->cand_count);
  } else if (mode != kModeTakeAll) {
    if (tid == 0 && status) atomicOr(status, (uint32_t)FFTOPK_ST_INTERNAL);
  }
  if constexpr (kTrackMin) {
    if (thr_out != nullptr) {
      __syncthreads();
      if (tid == 0) {
        uint32_t thr = 0u;
        if (mode == kModeGather && ctrl->thr_key != 0xffffffffu) thr = ctrl->thr_key;
        if (mode == kModeTakeAll) thr = t << pshift;  // the whole bin won: its lower edge
        *thr_out = thr;
      }
    }
  }
}

}  // namespace fftopk
