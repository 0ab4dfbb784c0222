// Device-side building blocks of the sm_100a top-2048 selector: warp/block scans that pick a
// threshold bin, the histogram update, and the single-CTA "finish" that resolves a small
// candidate list held in shared memory.
#pragma once
#include <type_traits>
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fftopk.h"
#include "fftopk_decide.h"
#include "fftopk_key.h"
#include "fftopk_trace.cuh"

namespace fftopk {

namespace cg = cooperative_groups;

constexpr int kK = 2048;               // reference: TopK (topk_indexer_radix.cu:69)
constexpr int kMaxK = 4096;            // largest k of the general entry point (fftopk_select_topk)
constexpr int kMaxBins = 4096;         // widest digit of the distributed rounds: 12 bits
constexpr int kSup = 64;               // super-bins per histogram (each sums kMaxBins/64 bins)
constexpr int kMaxCluster = 16;        // CTAs per row (non-portable cluster size on B200)
#ifndef FFTOPK_KSMALL
#define FFTOPK_KSMALL 256
#endif
constexpr int kSmall = FFTOPK_KSMALL;            // undecided candidates that are ranked directly instead of another radix round
constexpr unsigned kFull = 0xffffffffu;

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

// Checked build (-DFFTOPK_CHECKED): every index that the selection logic guarantees to be in
// range - an output slot below k, a candidate slot the decision step has made room for, a staged
// row index below the row length, the winner count of a finish - is tested before use. A failing
// test skips the access, raises FFTOPK_ST_CHECK in the status word and, if it is the first one,
// leaves (site, index, limit, block) in a device-side record that fftopk_checked_read() returns.
// Capacity limits that the algorithm handles by design (a full candidate list makes the row fall
// back to full histograms) are not violations. The production build compiles the tests away.
#ifdef FFTOPK_CHECKED
static __device__ unsigned int g_check_rec[4];
static __device__ __noinline__ void check_fail(int site, uint32_t idx, uint32_t limit, uint32_t* status) {
  if (atomicCAS(&g_check_rec[0], 0u, (unsigned)site) == 0u) {
    g_check_rec[1] = idx;
    g_check_rec[2] = limit;
    g_check_rec[3] = blockIdx.x;
  }
  if (status) atomicOr(status, (uint32_t)FFTOPK_ST_CHECK);
}
#define FFTOPK_CHECK(site, idx, limit, status) \
  (((uint32_t)(idx) < (uint32_t)(limit)) ? true : (::fftopk::check_fail((site), (uint32_t)(idx), (uint32_t)(limit), (status)), false))
#else
#define FFTOPK_CHECK(site, idx, limit, status) true
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Shared-memory atomics with the state space spelled out. Pointers into the dynamic shared
// memory block travel through structs and function arguments here, where the compiler no longer
// knows their address space and would emit generic atomics (an order of magnitude slower on the
// shared window).
__device__ __forceinline__ void red_shared_add(uint32_t* p, uint32_t v) {
  asm volatile("red.shared.add.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t atom_shared_add(uint32_t* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.shared.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(smem_u32(p)), "r"(v) : "memory");
  return old;
}

// Histogram update: a plain shared-memory reduction (no result). Measured on B200 (64K updates
// per CTA, 1024 threads): 6 to 12 updates per clock per SM whatever the bin distribution,
// all-equal bins included - the hardware combines same-address updates, and ballot / match.any
// pre-aggregation in software was 2 to 10 times slower.
__device__ __forceinline__ void hist_add(uint32_t* hist, uint32_t bin, bool valid) {
  if (valid) red_shared_add(&hist[bin], 1u);
}

// Slot allocation from a shared-memory counter (the atomic's RESULT is needed, so equal
// addresses do serialise): the lanes of a warp that are allocating together take consecutive
// slots with one atomic. May be called from divergent code.
__device__ __forceinline__ uint32_t warp_alloc(uint32_t* counter) {
  const unsigned m = __activemask();
  const int leader = __ffs(m) - 1;
  uint32_t base = 0;
  if (lane_id() == leader) base = atom_shared_add(counter, (uint32_t)__popc(m));
  base = __shfl_sync(m, base, leader);
  return base + (uint32_t)__popc(m & ((1u << lane_id()) - 1u));
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

// ---------------------------------------------------------------------------------------------
// Shared-memory control block (one per CTA; rank 0's counters are the cluster-wide ones).
// ---------------------------------------------------------------------------------------------
struct Ctrl {
  // cluster-wide allocation counters, meaningful in rank 0 only (targets of remote atomics)
  uint32_t win_count;
  uint32_t cand_count;
  uint32_t over_flag;  // rank 0 only: some CTA's candidate list overflowed (remote OR)
  uint32_t max_key;    // rank 0 only: largest key among the gathered candidates (remote max)
  // published to the peers before a cluster barrier
  uint32_t pub_flag;
  // per-pass local slot counters
  uint32_t wslot;
  uint32_t cslot;
  uint32_t fslot;
  uint32_t small_n;
  uint32_t lcount;  // entries pushed to this CTA's spill area (may exceed its capacity)
  uint32_t spill_kmax;  // largest key among the spilled entries
  // result of the most recent threshold search
  int32_t t;
  uint32_t above;
  uint32_t cnt;
  int32_t sup_sel;
  uint32_t sup_above;
  uint32_t need;
  uint32_t any_flag;
  int32_t mode;
  uint32_t base_w;
  uint32_t base_c;
  uint32_t tie_prefix;
  uint32_t local_c;
  uint32_t run_total;
  // cluster-wide super-bin totals and fine-bin totals of the threshold super-bin, double-buffered
  // by search number (each search clears the buffers of the next one)
  uint32_t tot[2][kSup];
  uint32_t tot2[2][kSup];
  uint32_t totb[kSup];  // first sample round: super-bin totals of the second (finer) histogram
  uint32_t dual_b;      // ... whether the finer histogram was usable, and for which top nibble
  uint32_t dual_g;
  int32_t focus_bin;    // first sample round of a lone CTA: bin the threshold will not lie above (-1: none)
  uint32_t wtot[32];
  uint32_t wmax[32];
  // merge of candidate lists: this CTA's record about its shard, read by the cluster's other CTAs
  uint32_t thr_key;      // warm start: smallest key among the winners of the finish
  uint32_t merge_count;  // valid candidates
  uint32_t merge_fail;   // the bounded wait for the shard's flag ran out
  uint64_t small[kSmall];
#ifdef FFTOPK_CHECKED
  uint32_t* status_ptr;  // the call's status word, for checks in code that has no other way to it
#endif
};
#ifdef FFTOPK_CHECKED
#define ctrl_status(c) ((c)->status_ptr)
#endif

// What a cluster does after a threshold search (see decide_and_allocate).
enum Mode : int { kModeNext = 0, kModeGather = 1, kModeTakeAll = 2, kModeTies = 3, kModeAbort = 4, kModeFallback = 5 };

// Sum each group of nb/64 consecutive bins into sup[0..63].
template <int NT>
__device__ __forceinline__ void compute_sup(const uint32_t* hist, uint32_t* sup, int nb) {
  const int tid = threadIdx.x;
  if (nb == kMaxBins) {
    constexpr int PER = kMaxBins / NT;            // bins per thread: 4 (1024 thr), 8 (512)
    constexpr int TPS = (kMaxBins / kSup) / PER;  // threads per super-bin: 16, 8
    uint32_t s = 0;
    const uint4* h4 = reinterpret_cast<const uint4*>(hist) + tid * (PER / 4);
#pragma unroll
    for (int j = 0; j < PER / 4; ++j) {
      const uint4 v = h4[j];
      s += v.x + v.y + v.z + v.w;
    }
#pragma unroll
    for (int off = TPS / 2; off > 0; off >>= 1) s += __shfl_xor_sync(kFull, s, off);
    if ((tid % TPS) == 0) sup[tid / TPS] = s;
  } else {  // 256 bins
    if (tid < kSup) {
      const uint4 v = reinterpret_cast<const uint4*>(hist)[tid];
      sup[tid] = v.x + v.y + v.z + v.w;
    }
  }
}

// Cluster barrier; for a cluster of one CTA a block barrier does the same job for less.
__device__ __forceinline__ void cluster_sync(cg::cluster_group& cluster, int C) {
  if (C == 1) {
    __syncthreads();
  } else {
    cluster.sync();
  }
}

// What warp 0 knows after a cluster-wide threshold search.
struct Picked {
  bool ok;            // false: the histogram holds fewer than `need` elements
  int t;              // threshold bin
  uint32_t need2;     // elements still to take from bin t
  uint32_t cnt;       // cluster-wide population of bin t
  uint32_t local_w;   // this CTA's elements in bins above t
  uint32_t local_c;   // this CTA's elements in bin t
  uint32_t total;     // cluster-wide number of histogrammed elements
  uint32_t any_flag;  // OR of the peers' published flags
  int tf;             // t's position inside its super-bin (index into xch rows)
  bool fine;          // the search ran on the second, finer histogram (see cluster_pick)
  uint32_t group;     // ... whose bins all lie under this value of the key's top four bits
};

// Cluster-wide threshold search on per-CTA histograms `h` (nb bins) with super-bin sums `s`,
// both complete and published by a cluster barrier before the call. Every CTA reads its peers'
// 64 super-bin sums, then the fine bins of the threshold super-bin, over distributed shared
// memory; warp 0 picks with shuffle scans. need_of(total) maps the cluster-wide element count
// to the rank searched for. `post(picked)` runs in warp 0 (all lanes) before the closing
// barrier; the results it wants every thread to see go through `ctrl`.
// Optionally a second histogram `hb` / `sb` of the same elements on key bits [27:16] (4096 bins, 16
// times finer) comes along: it orders the elements only if they all share the key's top four
// bits, i.e. if one group of four super-bins of `h` holds everything; then the search runs on it
// (Picked::fine, ::group) and the threshold bin is a 16-bit key prefix. ctrl->totb must be zero.
// Replaces parallel_reduce_histogram + radix_prefix_sum of the reference
// (topk_indexer_radix.cu:80-107, 232-279), which reduce to rank 0 and broadcast back with three
// cluster barriers and eight block barriers per round.
template <int NT, class NeedFn, class Post>
__device__ __forceinline__ void cluster_pick(cg::cluster_group& cluster, int C, const uint32_t* h, const uint32_t* s,
                                             uint32_t* xch, Ctrl* ctrl, int& pick_no, int nb, NeedFn&& need_of,
                                             Post&& post, const uint32_t* hb = nullptr, const uint32_t* sb = nullptr) {
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int fine = nb / kSup;
  uint32_t* tot = ctrl->tot[pick_no & 1];
  uint32_t* tot2 = ctrl->tot2[pick_no & 1];
  const bool dual = hb != nullptr;
  // (A) cluster-wide super-bin totals: one remote word per thread, summed with shared-memory
  // reductions instead of a serial loop over the ranks. (Pushing the sums into the peers before
  // the cluster barrier instead - remote reductions behind a split arrive / wait barrier - was
  // measured and was not faster: the release of the extra arrive costs what the remote loads cost.)
  for (int i = tid; i < C * kSup; i += NT) {
    const uint32_t* rs = C == 1 ? s : cluster.map_shared_rank(s, i / kSup);
    red_shared_add(&tot[i % kSup], rs[i % kSup]);
    if (dual) {
      const uint32_t* rb = C == 1 ? sb : cluster.map_shared_rank(sb, i / kSup);
      red_shared_add(&ctrl->totb[i % kSup], rb[i % kSup]);
    }
  }
  __syncthreads();
  FFTOPK_MARK(40);
  // Warp 0 picks and publishes through the control block. (Letting every warp pick for itself
  // saves the two broadcast barriers but was measured slower: 32 warps running the same shuffle
  // scans get in each other's way.)
  if (warp == 0) {
    uint32_t lo = tot[2 * lane], hi = tot[2 * lane + 1];
    const uint32_t total = warp_sum(lo + hi);
    const uint32_t need = need_of(total);
    unsigned one = 0u;
    if (dual) {
      // four super-bins = 256 bins of `h` = one value of the top four key bits
      const uint32_t pair = lo + hi;
      const uint32_t grp = pair + __shfl_xor_sync(kFull, pair, 1);
      one = __ballot_sync(kFull, fine_histogram_usable(true, total, grp));
      if (one != 0u) {
        lo = ctrl->totb[2 * lane];
        hi = ctrl->totb[2 * lane + 1];
      }
    }
    uint32_t above = 0, cnt = 0;
    int ts = -1;
    const bool ok = need > 0 && warp_pick64(lo, hi, need, ts, above, cnt);
    if (lane == 0) {
      ctrl->sup_sel = ok ? ts : -1;
      ctrl->sup_above = above;
      ctrl->need = need;
      ctrl->run_total = total;
      ctrl->dual_b = one != 0u ? 1u : 0u;
      ctrl->dual_g = one != 0u ? (uint32_t)((__ffs(one) - 1) >> 1) : 0u;
    }
  }
  __syncthreads();
  FFTOPK_MARK(41);
  const int ssel = ctrl->sup_sel;
  if (dual && ctrl->dual_b != 0u) {  // (uniform) the rest of the search runs on the finer histogram
    h = hb;
    s = sb;
  }
  // (B) fine bins of the threshold super-bin: pulled from every peer, kept per rank in xch (the
  // tie path wants them) and summed into tot2
  if (ssel >= 0) {
    for (int i = tid; i < C * kSup; i += NT) {
      const int q = i / kSup, f = i % kSup;
      uint32_t v = 0;
      if (f < fine) {
        const uint32_t* rh = C == 1 ? h : cluster.map_shared_rank(h, q);
        v = rh[ssel * fine + f];
        red_shared_add(&tot2[f], v);
      }
      xch[i] = v;
    }
  }
  __syncthreads();
  FFTOPK_MARK(42);
  // the buffers of the next search: their last readers passed the barrier above long ago
  if (tid < kSup) {
    ctrl->tot[(pick_no + 1) & 1][tid] = 0u;
    ctrl->tot2[(pick_no + 1) & 1][tid] = 0u;
  }
  ++pick_no;
  if (warp == 0) {
    Picked pk;
    pk.ok = false;
    pk.t = -1;
    pk.need2 = pk.cnt = pk.local_w = pk.local_c = 0;
    pk.total = ctrl->run_total;
    pk.any_flag = 0u;
    pk.tf = 0;
    pk.fine = dual && ctrl->dual_b != 0u;
    pk.group = ctrl->dual_g;
    if (ssel >= 0) {
      const uint32_t lo = tot2[2 * lane], hi = tot2[2 * lane + 1];
      const uint32_t need = ctrl->need, sup_above = ctrl->sup_above;
      int tf = -1;
      uint32_t above_f = 0, cnt_t = 0;
      if (warp_pick64(lo, hi, need - sup_above, tf, above_f, cnt_t)) {
        pk.ok = true;
        pk.tf = tf;
        pk.t = ssel * fine + tf;
        pk.need2 = need - sup_above - above_f;
        pk.cnt = cnt_t;
        uint32_t lw = 0;
        lw += (2 * lane > ssel) ? s[2 * lane] : 0u;
        lw += (2 * lane + 1 > ssel) ? s[2 * lane + 1] : 0u;
        lw += (2 * lane < fine && 2 * lane > tf) ? h[ssel * fine + 2 * lane] : 0u;
        lw += (2 * lane + 1 < fine && 2 * lane + 1 > tf) ? h[ssel * fine + 2 * lane + 1] : 0u;
        pk.local_w = warp_sum(lw);
        pk.local_c = h[pk.t];
      }
    }
    post(pk);  // warp 0 only; what the other warps need goes through the control block
  }
  __syncthreads();
  FFTOPK_MARK(43);
}

// Standard decision after a search with need = what is still missing of k: either the threshold
// bin is taken whole, or its population fits rank 0's buffer and is gathered there, or
// `otherwise` (a mode) applies. Output and candidate slots are allocated with one remote atomic
// each on rank 0's counters.
// `cx` is anything with the members ctrl, ctrl0 (rank 0's control block) and cand_cap.
template <class Ctx>
__device__ __forceinline__ void decide_and_allocate(const Ctx& cx, const Picked& pk, int otherwise,
                                                    bool force_otherwise) {
  int md = kModeAbort;
  uint32_t base_w = 0, base_c = 0, lw = pk.local_w;
  if (pk.ok) {
    if (force_otherwise) {
      md = otherwise;
    } else if (pk.cnt == pk.need2) {
      md = kModeTakeAll;
      lw += pk.local_c;
    } else if (pk.cnt <= (uint32_t)cx.cand_cap) {
      md = kModeGather;
    } else {
      md = otherwise;
    }
    if (lane_id() == 0 && md != kModeFallback) {
      base_w = atomicAdd(&cx.ctrl0->win_count, lw);
      if (md == kModeGather) base_c = atomicAdd(&cx.ctrl0->cand_count, pk.local_c);
    }
  }
  if (lane_id() == 0) {
    Ctrl* ctrl = cx.ctrl;
    ctrl->mode = md;
    ctrl->t = pk.t;
    ctrl->above = pk.need2;
    ctrl->cnt = pk.cnt;
    ctrl->base_w = base_w;
    ctrl->base_c = base_c;
    ctrl->local_c = pk.local_c;
    ctrl->wslot = 0u;
    ctrl->cslot = 0u;
  }
}

// ---------------------------------------------------------------------------------------------
// Candidate sources of the finish. A source tells a thread which candidates are its share:
//   for_each_key(f)     f(key) for every slot of the share (any order, any trip count)
//   for_each_uniform(f) f(composite) with the same trip count in all lanes of a warp (f may vote);
//                       lanes without a candidate get 0, which is also what an empty slot holds
//   for_each_uniform4(f4)  the same, four composites per call
// Loads are issued four at a time (a plain loop waits out the full shared-memory latency once per
// element: measured 190 cycles per element with 16 warps on the SM).
// ---------------------------------------------------------------------------------------------

// One dense array cand[0..n); slots equal to 0 are empty.
template <int NT>
struct DenseCands {
  static constexpr bool kEmpties = true;
  const uint64_t* cand;
  int n;
  template <class F>
  __device__ __forceinline__ void for_each_key(F&& f) const {
    const uint32_t* hi32 = reinterpret_cast<const uint32_t*>(cand) + 1;  // little endian: word 1 = key
    int i = threadIdx.x;
    for (; i + 3 * NT < n; i += 4 * NT) {
      const uint32_t k0 = hi32[2 * i], k1 = hi32[2 * (i + NT)], k2 = hi32[2 * (i + 2 * NT)], k3 = hi32[2 * (i + 3 * NT)];
      f(k0);
      f(k1);
      f(k2);
      f(k3);
    }
    for (; i < n; i += NT) f(hi32[2 * i]);
  }
  template <class F4>
  __device__ __forceinline__ void for_each_uniform4(F4&& f4) const {
    const int tid = threadIdx.x;
    for (int i0 = 0; i0 < n; i0 += 4 * NT) {
      const int i = i0 + tid;
      const uint64_t c0 = (i < n) ? cand[i] : 0ull;
      const uint64_t c1 = (i + NT < n) ? cand[i + NT] : 0ull;
      const uint64_t c2 = (i + 2 * NT < n) ? cand[i + 2 * NT] : 0ull;
      const uint64_t c3 = (i + 3 * NT < n) ? cand[i + 3 * NT] : 0ull;
      f4(c0, c1, c2, c3);
    }
  }
  template <class F>
  __device__ __forceinline__ void for_each_uniform(F&& f) const {
    for_each_uniform4([&](uint64_t c0, uint64_t c1, uint64_t c2, uint64_t c3) {
      f(c0);
      f(c1);
      f(c2);
      f(c3);
    });
  }
};

// What the filter of a lone CTA leaves behind: one dense segment per warp (each warp walks its own;
// `wn`, its length, is the same in all lanes) plus the shared spill area of `sn` entries. No slot
// is empty.
template <int NT>
struct WarpSegCands {
  static constexpr bool kEmpties = false;
  const uint64_t* seg;
  int wn;
  const uint64_t* spill;
  int sn;
  template <class F>
  __device__ __forceinline__ void for_each_key(F&& f) const {
    const uint32_t* hi32 = reinterpret_cast<const uint32_t*>(seg) + 1;
    int i = lane_id();
    for (; i + 96 < wn; i += 128) {
      const uint32_t k0 = hi32[2 * i], k1 = hi32[2 * (i + 32)], k2 = hi32[2 * (i + 64)], k3 = hi32[2 * (i + 96)];
      f(k0);
      f(k1);
      f(k2);
      f(k3);
    }
    for (; i < wn; i += 32) f(hi32[2 * i]);
    const uint32_t* sp32 = reinterpret_cast<const uint32_t*>(spill) + 1;
    for (int j = threadIdx.x; j < sn; j += NT) f(sp32[2 * j]);
  }
  template <class F4>
  __device__ __forceinline__ void for_each_uniform4(F4&& f4) const {
    const int lane = lane_id();
    for (int i0 = 0; i0 < wn; i0 += 128) {
      const int i = i0 + lane;
      const uint64_t c0 = (i < wn) ? seg[i] : 0ull;
      const uint64_t c1 = (i + 32 < wn) ? seg[i + 32] : 0ull;
      const uint64_t c2 = (i + 64 < wn) ? seg[i + 64] : 0ull;
      const uint64_t c3 = (i + 96 < wn) ? seg[i + 96] : 0ull;
      f4(c0, c1, c2, c3);
    }
    const int tid = threadIdx.x;
    for (int j0 = 0; j0 < sn; j0 += 4 * NT) {
      const int j = j0 + tid;
      const uint64_t c0 = (j < sn) ? spill[j] : 0ull;
      const uint64_t c1 = (j + NT < sn) ? spill[j + NT] : 0ull;
      const uint64_t c2 = (j + 2 * NT < sn) ? spill[j + 2 * NT] : 0ull;
      const uint64_t c3 = (j + 3 * NT < sn) ? spill[j + 3 * NT] : 0ull;
      f4(c0, c1, c2, c3);
    }
  }
  template <class F>
  __device__ __forceinline__ void for_each_uniform(F&& f) const {
    for_each_uniform4([&](uint64_t c0, uint64_t c1, uint64_t c2, uint64_t c3) {
      f(c0);
      f(c1);
      f(c2);
      f(c3);
    });
  }
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
// Single-CTA finish. The source holds composites c = (key << 32) | ~idx in shared memory (0 =
// empty slot), all of them inside [lo, cap]; lo > cap means "range unknown" and costs a pass
// that finds it. Writes the `need` largest composites' indices (and keys) to
// out_idx[out_base ...], in unspecified order.
//
// Replaces the reference's refinement rounds on shared-memory survivors and its CAS insertion
// tail (topk_indexer_radix.cu:686-781, 109-141, 788-850). Because the index is part of the
// composite, equal values are resolved towards the lower index by the same rounds, and the last
// <= 256 undecided candidates are ranked by votes.
// `focus`: see FinishDigit (fftopk_decide.h). `have_hist`: the caller has already built round 0's histogram in
// `hist`, with make_finish_digit(lo, focus).
// `idx_bits`: all indices are < 2^idx_bits, so the inverted-index bits above that are all ones.
// `page`: optional per-row table; the value written is then page[idx] instead of idx + idx_offset
// (the fused page-table transform of the reference's topk_transform_* kernels, :871-958).
// ---------------------------------------------------------------------------------------------
// `known_total`: when not 0, the number of candidates in the source; if it equals `need` they all
// win and no round is run. kTrackMin: the smallest key among the winners - the key of the
// need-th largest candidate - is left in ctrl->thr_key (atomic min; the caller presets it).
template <int NT, class Src, bool kTrackMin = false>
__device__ void cta_finish(const Src& src, uint32_t need, uint64_t lo, uint64_t cap, uint64_t focus, bool have_hist,
                           int idx_bits, uint32_t* hist /* >= kFinishBins words */, Ctrl* ctrl, int32_t* out_idx,
                           uint32_t* out_key, uint32_t out_base, uint32_t out_slots /* k of the row */,
                           int32_t idx_offset, uint32_t* status,
                           const int32_t* page = nullptr /* when set: out = page[idx] */, uint32_t known_total = 0u) {
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    ctrl->fslot = 0u;  // (every path below has a block barrier before these are used)
    ctrl->small_n = 0u;
  }
  if (lo > cap) {
    // Range unknown: the smallest and the largest key present bound it.
    uint32_t kmin = ~0u, kmax = 0u;
    src.for_each_key([&](uint32_t k) {
      if (k != 0u) {
        kmin = min(kmin, k);
        kmax = max(kmax, k);
      }
    });
    kmin = __reduce_min_sync(kFull, kmin);
    kmax = __reduce_max_sync(kFull, kmax);
    if (lane == 0) {
      hist[2 * warp + 0] = kmin;
      hist[2 * warp + 1] = kmax;
    }
    __syncthreads();
    const bool in = lane < NT / 32;
    kmin = __reduce_min_sync(kFull, in ? hist[2 * lane + 0] : ~0u);
    kmax = __reduce_max_sync(kFull, in ? hist[2 * lane + 1] : 0u);
    lo = (uint64_t)kmin << 32;
    cap = ((uint64_t)kmax << 32) | 0xffffffffull;
    if (lo > cap) {  // no candidate at all
      if (tid == 0 && status) atomicOr(status, 2u);
      return;
    }
    focus = cap;
    have_hist = false;
    __syncthreads();  // the scratch words are about to be cleared as the histogram
    FFTOPK_MARK(31);
  }
  // ---- rounds: only the threshold is determined here; nothing is written yet ---------------------
  // Outcome: the threshold bin [t_lo, t_hi] of composites. Everything above t_hi wins; of the
  // bin itself either everything wins (all_bin) or, when it holds <= kSmall candidates, the best
  // `need2` of them, found by ranking.
  const uint32_t need_total = need;
  uint64_t t_lo = 0ull, t_hi = 0ull;
  uint32_t need2 = 0, cnt = 0;
  bool all_bin = false, found = false;
  if (known_total != 0u && known_total == need && lo <= cap) {
    // exactly as many candidates as are wanted: all of them win
    t_lo = lo;
    t_hi = cap;
    cnt = need2 = need;
    all_bin = found = true;
    __syncthreads();  // (the counters cleared above are used by the pass below)
  } else if (known_total != 0u && known_total <= (uint32_t)kSmall && known_total >= need && lo <= cap) {
    // so few candidates that they are ranked directly: the whole range is the "threshold bin"
    t_lo = lo;
    t_hi = cap;
    cnt = known_total;
    need2 = need;
    found = true;
    __syncthreads();
  }
  for (int round = 0; round < 24 && !found; ++round) {
    if ((uint32_t)(lo >> 32) == (uint32_t)(cap >> 32)) {
      // one key left: the inverted indices all start with the same run of ones
      const uint64_t floor_lo = single_key_floor(lo, idx_bits);
      if (lo < floor_lo && floor_lo <= cap) {
        if (focus < floor_lo) focus = cap;
        lo = floor_lo;
        have_hist = false;
      }
    }
    if (focus < lo || focus > cap) focus = cap;
    const FinishDigit dg = make_finish_digit(lo, focus);
    if (!(round == 0 && have_hist)) {
      for (int b = tid; b < kFinishBins; b += NT) hist[b] = 0u;
      __syncthreads();
      const uint64_t span = cap - lo;
      if (dg.key_only()) {
        // the digit depends on the key alone: work on the high words only (an empty slot has key 0)
        const uint32_t klo = (uint32_t)(lo >> 32), kspan = (uint32_t)(span >> 32);
        src.for_each_key([&](uint32_t k) {
          if ((!Src::kEmpties || k != 0u) && (k - klo) <= kspan) red_shared_add(&hist[dg.of_key(k)], 1u);
        });
      } else {
        src.for_each_uniform([&](uint64_t c) {
          if (c != 0ull && (c - lo) <= span) red_shared_add(&hist[dg.of(c)], 1u);
        });
      }
      __syncthreads();
    }
    FFTOPK_MARK(16);
    block_pick<NT>(hist, need, ctrl);
    FFTOPK_MARK(17);
    const int t = ctrl->t;
    if (t < 0) {
      if (tid == 0 && status) atomicOr(status, 2u);
      return;
    }
    cnt = ctrl->cnt;
    need2 = need - ctrl->above;
    finish_bin_range(dg, lo, cap, t, t_lo, t_hi);
    if (cnt == need2 || cnt <= (uint32_t)kSmall) {
      all_bin = (cnt == need2);
      found = true;
      break;
    }
    lo = t_lo;
    cap = focus = t_hi;
    need = need2;
    __syncthreads();  // every thread has read ctrl->t/cnt/above before the next round rewrites them
  }
  FFTOPK_MARK(30);
  if (!found) {
    if (tid == 0 && status) atomicOr(status, 2u);
    return;
  }
  // ---- one pass writes the certain winners (a ballot and one slot-allocating atomic per warp
  // and trip; the order of the output is unspecified) and sets the undecided candidates aside ----
  FFTOPK_MARK(32);
  const uint64_t wthr = all_bin ? (t_lo ? t_lo - 1ull : 0ull) : t_hi;  // winners: c > wthr
  const unsigned lt = (1u << lane) - 1u;
  // Slots come from one shared counter; the warps' atomics on it serialise (~30 cycles each), so
  // a warp allocates for four candidates per lane with one of them.
  uint32_t win_min = 0xffffffffu;  // (kTrackMin) smallest key among the winners this thread wrote
  auto pass = [&](auto paged) {
    src.for_each_uniform4([&](uint64_t c0, uint64_t c1, uint64_t c2, uint64_t c3) {
      const uint64_t c[4] = {c0, c1, c2, c3};
      unsigned b[4];
      uint32_t nwin = 0;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        b[u] = __ballot_sync(kFull, c[u] > wthr);
        nwin += (uint32_t)__popc(b[u]);
      }
      if (nwin) {
        uint32_t base = 0;
        if (lane == 0) base = atom_shared_add(&ctrl->fslot, nwin);
        base = out_base + __shfl_sync(kFull, base, 0);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t pos = base + (uint32_t)__popc(b[u] & lt);
          if (c[u] > wthr && FFTOPK_CHECK(3, pos, out_slots, status) && pos < out_slots) {
            const int32_t idx = (int32_t)(~(uint32_t)c[u]);
            if constexpr (decltype(paged)::value) {
              out_idx[pos] = __ldg(page + idx);
            } else {
              out_idx[pos] = idx + idx_offset;
            }
            if (out_key) out_key[pos] = (uint32_t)(c[u] >> 32);
            if constexpr (kTrackMin) win_min = min(win_min, (uint32_t)(c[u] >> 32));
          }
          base += (uint32_t)__popc(b[u]);
        }
      }
      if (!all_bin) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (c[u] <= wthr && c[u] >= t_lo && c[u] != 0ull) {
            const uint32_t s = warp_alloc(&ctrl->small_n);
            if (FFTOPK_CHECK(4, s, kSmall, status) && s < (uint32_t)kSmall) ctrl->small[s] = c[u];
          }
        }
      }
    });
  };
  if (page) {
    pass(std::true_type{});
  } else {
    pass(std::false_type{});
  }
  FFTOPK_MARK(33);
  if constexpr (kTrackMin) {
    win_min = __reduce_min_sync(kFull, win_min);
    if (lane == 0 && win_min != 0xffffffffu) atomicMin(&ctrl->thr_key, win_min);
  }
#ifdef FFTOPK_CHECKED
  {
    // every certain winner took exactly one slot, every undecided candidate was set aside
    __syncthreads();
    const uint32_t want_w = all_bin ? need_total : need_total - need2;
    if (tid == 0) {
      if (ctrl->fslot != want_w) check_fail(10, ctrl->fslot, want_w, status);
      if (!all_bin && ctrl->small_n != cnt) check_fail(11, ctrl->small_n, cnt, status);
    }
  }
#endif
  if (!all_bin) {
    __syncthreads();
    // Rank by vote: warp i takes candidate i, the lanes compare it with the candidates j (32 per
    // step); the number of larger ones is candidate i's rank, and the best need2 go behind the
    // certain winners. Up to 256 undecided candidates are cheaper to rank like this (at most 64
    // votes per warp) than to split by another round - rows of low-precision logits have
    // hundreds of exact duplicates at the threshold. (A bitonic compare-exchange network over 32
    // values is a chain of 60 dependent shuffles; this is one ballot per 32 comparisons.)
    const uint32_t certain = need_total - need2;
    const int nchunk = ((int)cnt + 31) >> 5;
    for (int i = warp; i < (int)cnt; i += NT / 32) {
      const uint64_t me = ctrl->small[i];
      uint32_t rank = 0;
      for (int ch = 0; ch < nchunk; ++ch) {
        const int j = ch * 32 + lane;
        const uint64_t other = (j < (int)cnt) ? ctrl->small[j] : 0ull;
        rank += (uint32_t)__popc(__ballot_sync(kFull, other > me));
      }
      if (lane == 0 && rank < need2) {
        const uint32_t pos = out_base + certain + rank;
        if (FFTOPK_CHECK(5, pos, out_slots, status) && pos < out_slots) {
          const int32_t idx = (int32_t)(~(uint32_t)me);
          out_idx[pos] = page ? __ldg(page + idx) : idx + idx_offset;
          if (out_key) out_key[pos] = (uint32_t)(me >> 32);
        }
        if constexpr (kTrackMin) atomicMin(&ctrl->thr_key, (uint32_t)(me >> 32));
      }
    }
  }
}

}  // namespace fftopk
