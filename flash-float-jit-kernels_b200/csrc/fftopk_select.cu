// Per-row top-2048 radix selector for B200 (sm_100a): one thread-block cluster per row.
//
// What it replaces in the reference: topk_kernel and fast_topk_split_kv_cuda_tl
// (jit_kernel/csrc/topk_indexer/topk_indexer_radix.cu:456-869) and the host launcher
// fast_topk_interface (:1051-1158).
//
// Shape of the computation for one row of `len` > 2048 valid fp32 logits, C CTAs in the cluster:
//   1. every CTA owns a contiguous shard; the TMA engine bulk-copies as much of it as fits into
//      shared memory (16 chunks, one mbarrier each), the rest is streamed with 128-bit loads;
//   2. round 0 histograms the top 12 bits of the order-preserving key (4096 bins) per CTA;
//   3. after ONE cluster barrier every CTA reads its peers' 64 super-bin sums, then the 64 fine
//      bins of the threshold super-bin, over distributed shared memory, and picks the threshold
//      bin with a warp-shuffle suffix scan (no L2 atomics, no broadcast barrier);
//   4. a second scan (from shared memory where staged, else from L2) writes the indices of
//      elements above the threshold bin straight to the output and pushes the threshold-bin
//      survivors into rank 0's shared memory; after the second cluster barrier rank 0 resolves
//      them with radix passes over (key, inverted index) composites and a warp
//      compare-exchange network for the last <= 32;
//   5. if the threshold bin holds more survivors than rank 0 can take (heavy ties, narrow value
//      ranges) the cluster keeps refining on the next 12 and 8 key bits, and exact ties that
//      remain after all 32 bits are taken in index order, shard by shard.
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fftopk.h"
#include "fftopk_device.cuh"
#include "fftopk_key.h"

namespace fftopk {

struct SelectParams {
  const float* score;
  int64_t row_stride;
  int64_t L;
  const int32_t* lengths;
  const int32_t* row_starts;
  int32_t* out_idx;
  uint32_t* out_key;
  uint32_t* status;
  int32_t B;
  int32_t idx_offset;
  int32_t stage_floats;  // shared-memory staging capacity per CTA, multiple of 128
  int32_t cand_cap;      // candidate capacity of rank 0
};

enum Mode : int { kModeNext = 0, kModeGather = 1, kModeTakeAll = 2, kModeTies = 3, kModeAbort = 4 };

// digit schedule of the distributed rounds: 12 + 12 + 8 bits
__device__ __forceinline__ int round_width(int r) { return r < 2 ? 12 : 8; }
__device__ __forceinline__ int round_shift(int r) { return r == 0 ? 20 : (r == 1 ? 8 : 0); }

// Shard of one CTA, in 16-byte granules of the aligned view of the row: granule g covers row
// elements 4g-a .. 4g-a+3, where a in 0..3 is the row's misalignment in elements.
struct Shard {
  const float* gbase;  // 16-byte aligned address of granule 0
  const float4* stage; // shared-memory copy of granules [g0, g0 + n_stage)
  uint64_t* mbar;
  int g0, g1;          // granule range of this CTA
  int n_stage;         // staged granules
  int chunk_g;         // granules per bulk-copy chunk
  int a;               // misalignment (elements)
  int len;             // valid elements in the row
};

// One granule from global memory; reads only bytes that belong to the row.
__device__ __forceinline__ float4 load_granule(const Shard& sh, int g) {
  const int i0 = 4 * g - sh.a;
  if (i0 >= 0 && i0 + 3 < sh.len) {
    return __ldg(reinterpret_cast<const float4*>(sh.gbase) + g);
  }
  float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
  const float* p = sh.gbase + 4 * (int64_t)g;
  if ((unsigned)(i0 + 0) < (unsigned)sh.len) x.x = __ldg(p + 0);
  if ((unsigned)(i0 + 1) < (unsigned)sh.len) x.y = __ldg(p + 1);
  if ((unsigned)(i0 + 2) < (unsigned)sh.len) x.z = __ldg(p + 2);
  if ((unsigned)(i0 + 3) < (unsigned)sh.len) x.w = __ldg(p + 3);
  return x;
}

__device__ __forceinline__ bool granule_full(const Shard& sh, int g) {
  const int i0 = 4 * g - sh.a;
  return i0 >= 0 && i0 + 3 < sh.len;
}

// Visit every element of the shard: op(key, idx, valid) is called by all threads of every warp
// together (valid = false for padding lanes), so op may use warp-synchronous primitives.
// WAIT: first visit, the staged chunks are consumed as their bulk copies land.
template <int NT, bool WAIT, class Op>
__device__ __forceinline__ void scan_shard(const Shard& sh, Ctrl* ctrl, Op&& op) {
  const int tid = threadIdx.x;
  auto proc = [&](const float4& x, int g, bool in) {
    const int i0 = 4 * g - sh.a;
    op(fftopk_key_from_bits(__float_as_uint(x.x)), i0 + 0, in && (unsigned)(i0 + 0) < (unsigned)sh.len);
    op(fftopk_key_from_bits(__float_as_uint(x.y)), i0 + 1, in && (unsigned)(i0 + 1) < (unsigned)sh.len);
    op(fftopk_key_from_bits(__float_as_uint(x.z)), i0 + 2, in && (unsigned)(i0 + 2) < (unsigned)sh.len);
    op(fftopk_key_from_bits(__float_as_uint(x.w)), i0 + 3, in && (unsigned)(i0 + 3) < (unsigned)sh.len);
  };
  // ---- staged part -------------------------------------------------------------------------
  if (sh.n_stage > 0) {
    const bool use_stage = WAIT ? true : (ctrl->stage_fail == 0u);
    const int nchunk = WAIT ? (sh.n_stage + sh.chunk_g - 1) / sh.chunk_g : 1;
    for (int c = 0; c < nchunk; ++c) {
      bool ok = use_stage;
      if (WAIT) {
        ok = mbar_wait_bounded(&sh.mbar[c], 0u);
        if (!ok) ctrl->stage_fail = 1u;
      }
      const int gbeg = WAIT ? c * sh.chunk_g : 0;
      const int gend = WAIT ? min(gbeg + sh.chunk_g, sh.n_stage) : sh.n_stage;
      for (int gb = gbeg; gb < gend; gb += NT) {
        const int gl = gb + tid;
        const bool in = gl < gend;
        const int g = sh.g0 + gl;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (in) x = (ok && granule_full(sh, g)) ? sh.stage[gl] : load_granule(sh, g);
        proc(x, g, in);
      }
    }
  }
  // ---- streamed part -----------------------------------------------------------------------
  constexpr int U = 4;
  for (int gb = sh.g0 + sh.n_stage; gb < sh.g1; gb += NT * U) {
    float4 x[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int g = gb + u * NT + tid;
      x[u] = (g < sh.g1) ? load_granule(sh, g) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int g = gb + u * NT + tid;
      proc(x[u], g, g < sh.g1);
    }
  }
}

// Sum each group of nb/64 consecutive bins into sup[0..63].
template <int NT>
__device__ __forceinline__ void compute_sup(const uint32_t* hist, uint32_t* sup, int nb) {
  const int tid = threadIdx.x;
  if (nb == kMaxBins) {
    constexpr int PER = kMaxBins / NT;       // bins per thread: 4 (1024 thr), 8 (512), 16 (256)
    constexpr int TPS = (kMaxBins / kSup) / PER;  // threads per super-bin: 16, 8, 4
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

template <int NT>
__global__ void __launch_bounds__(NT, 1) select2048_kernel(const SelectParams p) {
  cg::cluster_group cluster = cg::this_cluster();
  const int C = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int row = (int)(blockIdx.x / (unsigned)C);
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;

  int64_t row_start = p.row_starts ? (int64_t)p.row_starts[row] : 0;
  row_start = row_start < 0 ? 0 : (row_start > p.L ? p.L : row_start);
  int64_t len64 = (int64_t)p.lengths[row];
  len64 = len64 < 0 ? 0 : len64;
  len64 = len64 > p.L - row_start ? p.L - row_start : len64;
  const int len = (int)len64;
  const float* rowp = p.score + (int64_t)row * p.row_stride + row_start;
  int32_t* out_idx = p.out_idx + (int64_t)row * kK;
  uint32_t* out_key = p.out_key ? p.out_key + (int64_t)row * kK : nullptr;

  // Short rows: 0..len-1 then -1 (reference: naive_topk_cuda, topk_indexer_radix.cu:152-163).
  if (len <= kK) {
    if (rank == 0) {
      for (int i = tid; i < kK; i += NT) {
        out_idx[i] = i < len ? i + p.idx_offset : -1;
        if (out_key) out_key[i] = i < len ? fftopk_key_from_bits(__float_as_uint(__ldg(rowp + i))) : 0u;
      }
    }
    return;  // uniform over the cluster; no shared memory of this CTA is ever read by a peer
  }

  // ---- shared memory carve ---------------------------------------------------------------
  extern __shared__ __align__(128) unsigned char smem_raw[];
  uint32_t* hist[2] = {reinterpret_cast<uint32_t*>(smem_raw), reinterpret_cast<uint32_t*>(smem_raw) + kMaxBins};
  uint32_t* sup[2] = {hist[1] + kMaxBins, hist[1] + kMaxBins + kSup};
  uint32_t* xch = sup[1] + kSup;                                   // kMaxCluster * 64 words
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(xch + kMaxCluster * kSup);  // 8-byte aligned
  uint64_t* cand = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(ctrl) + ((sizeof(Ctrl) + 127) & ~127u));
  float* stage = reinterpret_cast<float*>(cand + p.cand_cap);     // cand_cap is a multiple of 16

  // ---- shard geometry --------------------------------------------------------------------
  Shard sh;
  sh.a = (int)((reinterpret_cast<uintptr_t>(rowp) >> 2) & 3u);
  sh.len = len;
  sh.gbase = rowp - sh.a;
  sh.stage = reinterpret_cast<const float4*>(stage);
  sh.mbar = ctrl->mbar;
  {
    const int gn = (sh.a + len + 3) >> 2;
    const int per = (((gn + C - 1) / C) + 31) & ~31;
    sh.g0 = min(rank * per, gn);
    sh.g1 = min(sh.g0 + per, gn);
    sh.n_stage = min(sh.g1 - sh.g0, p.stage_floats >> 2);
    sh.chunk_g = max(32, (((sh.n_stage + kChunks - 1) / kChunks) + 31) & ~31);
  }

  // ---- prologue: clear round-0 histogram, arm the barriers, start the bulk copies ----------
  {
    uint4* h4 = reinterpret_cast<uint4*>(hist[0]);
    for (int i = tid; i < kMaxBins / 4; i += NT) h4[i] = make_uint4(0u, 0u, 0u, 0u);
    if (tid == 0) {
      for (int c = 0; c < kChunks; ++c) mbar_init(&ctrl->mbar[c], 1u);
      ctrl->win_count = 0u;
      ctrl->cand_count = 0u;
      ctrl->wslot = 0u;
      ctrl->cslot = 0u;
      ctrl->stage_fail = 0u;
      mbar_fence_init();
    }
    __syncthreads();
    if (tid == 0 && sh.n_stage > 0) {
      // bulk copies cover only granules that lie completely inside the row
      const int gn = (sh.a + len + 3) >> 2;
      const int full_lo = sh.a > 0 ? 1 : 0;
      const int full_hi = ((sh.a + len) & 3) ? gn - 1 : gn;
      const int nchunk = (sh.n_stage + sh.chunk_g - 1) / sh.chunk_g;
      for (int c = 0; c < nchunk; ++c) {
        int lo = sh.g0 + c * sh.chunk_g;
        int hi = min(lo + sh.chunk_g, sh.g0 + sh.n_stage);
        lo = max(lo, full_lo);
        hi = min(hi, full_hi);
        const uint32_t bytes = hi > lo ? (uint32_t)(hi - lo) * 16u : 0u;
        mbar_arrive_expect_tx(&ctrl->mbar[c], bytes);
        if (bytes) bulk_g2s(stage + 4 * (lo - sh.g0), sh.gbase + 4 * (int64_t)lo, bytes, &ctrl->mbar[c]);
      }
    }
  }

  // ---- round 0: histogram of the top 12 key bits -----------------------------------------
  scan_shard<NT, true>(sh, ctrl, [&](uint32_t key, int, bool valid) { hist_add(hist[0], key >> 20, valid); });
  __syncthreads();

  Ctrl* ctrl0 = cluster.map_shared_rank(ctrl, 0);
  uint64_t* cand0 = cluster.map_shared_rank(cand, 0);

  uint32_t need = kK;
  uint32_t P = 0;  // threshold digits chosen so far (the key prefix every survivor shares)
  int mode = kModeAbort;
  int r = 0;
  for (;; ++r) {
    const int w = round_width(r);
    const int shift = round_shift(r);
    const int nb = 1 << w;
    const int fine = nb / kSup;
    uint32_t* h = hist[r & 1];
    uint32_t* s = sup[r & 1];

    compute_sup<NT>(h, s, nb);
    cluster.sync();  // every CTA's histogram and super-bin sums of this round are complete

    // (A) super-bin totals: one remote word per thread
    for (int i = tid; i < C * kSup; i += NT) {
      const uint32_t* rs = cluster.map_shared_rank(s, i / kSup);
      xch[i] = rs[i % kSup];
    }
    __syncthreads();
    if (warp == 0) {
      uint32_t lo = 0, hi = 0;
      for (int q = 0; q < C; ++q) {
        lo += xch[q * kSup + 2 * lane];
        hi += xch[q * kSup + 2 * lane + 1];
      }
      int ts = -1;
      uint32_t above = 0, cnt = 0;
      const bool ok = warp_pick64(lo, hi, need, ts, above, cnt);
      if (lane == 0) {
        ctrl->sup_sel = ok ? ts : -1;
        ctrl->sup_above = above;
      }
    }
    __syncthreads();
    const int ssel = ctrl->sup_sel;
    if (ssel < 0) {
      mode = kModeAbort;
      break;
    }
    const uint32_t sup_above = ctrl->sup_above;
    // (B) fine bins of the threshold super-bin
    for (int i = tid; i < C * kSup; i += NT) {
      const int q = i / kSup, f = i % kSup;
      uint32_t v = 0;
      if (f < fine) {
        const uint32_t* rh = cluster.map_shared_rank(h, q);
        v = rh[ssel * fine + f];
      }
      xch[i] = v;
    }
    __syncthreads();
    if (warp == 0) {
      uint32_t lo = 0, hi = 0;
      for (int q = 0; q < C; ++q) {
        lo += xch[q * kSup + 2 * lane];
        hi += xch[q * kSup + 2 * lane + 1];
      }
      int tf = -1;
      uint32_t above_f = 0, cnt_t = 0;
      const bool ok = warp_pick64(lo, hi, need - sup_above, tf, above_f, cnt_t);
      int md = kModeAbort;
      uint32_t base_w = 0, base_c = 0, tie_prefix = 0, local_c = 0, need2 = 0;
      if (ok) {
        need2 = need - sup_above - above_f;
        // this CTA's own counts above / at the threshold bin
        uint32_t lw = 0;
        lw += (2 * lane > ssel) ? s[2 * lane] : 0u;
        lw += (2 * lane + 1 > ssel) ? s[2 * lane + 1] : 0u;
        lw += (2 * lane < fine && 2 * lane > tf) ? h[ssel * fine + 2 * lane] : 0u;
        lw += (2 * lane + 1 < fine && 2 * lane + 1 > tf) ? h[ssel * fine + 2 * lane + 1] : 0u;
        lw = warp_sum(lw);
        local_c = h[ssel * fine + tf];
        if (cnt_t == need2) {
          md = kModeTakeAll;
          lw += local_c;
        } else if (cnt_t <= (uint32_t)p.cand_cap) {
          md = kModeGather;
        } else if (shift == 0) {
          md = kModeTies;
          uint32_t tp = (lane < rank) ? xch[lane * kSup + tf] : 0u;
          tie_prefix = warp_sum(tp);
        } else {
          md = kModeNext;
        }
        if (lane == 0) {
          base_w = atomicAdd(&ctrl0->win_count, lw);
          if (md == kModeGather) base_c = atomicAdd(&ctrl0->cand_count, local_c);
        }
      }
      if (lane == 0) {
        ctrl->mode = md;
        ctrl->t = ssel * fine + tf;
        ctrl->above = need2;  // remaining need after this round
        ctrl->cnt = cnt_t;
        ctrl->base_w = base_w;
        ctrl->base_c = base_c;
        ctrl->tie_prefix = tie_prefix;
        ctrl->local_c = local_c;
        ctrl->wslot = 0u;
        ctrl->cslot = 0u;
      }
    }
    // while warp 0 decides, the others clear the next round's histogram (safe: peers finished
    // reading that buffer before they arrived at this round's cluster barrier)
    {
      uint4* n4 = reinterpret_cast<uint4*>(hist[(r + 1) & 1]);
      for (int i = tid; i < kMaxBins / 4; i += NT) n4[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
    mode = ctrl->mode;
    if (mode == kModeAbort) break;
    const uint32_t Pn = (P << w) | (uint32_t)ctrl->t;
    const uint32_t Pold = P;  // digits of the rounds before this one
    const uint32_t base_w = ctrl->base_w;
    const uint32_t base_c = ctrl->base_c;
    need = ctrl->above;
    P = Pn;

    auto emit_winner = [&](uint32_t key, int idx) {
      const uint32_t pos = base_w + atomicAdd(&ctrl->wslot, 1u);
      if (pos < (uint32_t)kK) {
        out_idx[pos] = idx + p.idx_offset;
        if (out_key) out_key[pos] = key;
      }
    };

    if (mode == kModeNext) {
      const int shift2 = round_shift(r + 1);
      const uint32_t mask2 = (1u << round_width(r + 1)) - 1u;
      uint32_t* h2 = hist[(r + 1) & 1];
      scan_shard<NT, false>(sh, ctrl, [&](uint32_t key, int idx, bool valid) {
        const uint32_t hh = key >> shift;
        const bool older = valid && ((hh >> w) == Pold);
        if (older && hh > Pn) emit_winner(key, idx);
        hist_add(h2, (key >> shift2) & mask2, older && hh == Pn);
      });
      __syncthreads();
      continue;
    }
    if (mode == kModeGather) {
      scan_shard<NT, false>(sh, ctrl, [&](uint32_t key, int idx, bool valid) {
        const uint32_t hh = key >> shift;
        if (valid && ((hh >> w) == Pold)) {
          if (hh > Pn) {
            emit_winner(key, idx);
          } else if (hh == Pn) {
            const uint32_t slot = base_c + atomicAdd(&ctrl->cslot, 1u);
            if (slot < (uint32_t)p.cand_cap) cand0[slot] = ((uint64_t)key << 32) | (uint64_t)(~(uint32_t)idx);
          }
        }
      });
    } else if (mode == kModeTakeAll) {
      scan_shard<NT, false>(sh, ctrl, [&](uint32_t key, int idx, bool valid) {
        const uint32_t hh = key >> shift;
        if (valid && ((hh >> w) == Pold) && hh >= Pn) emit_winner(key, idx);
      });
    } else {  // kModeTies: all 32 key bits are fixed; P is the threshold key itself
      scan_shard<NT, false>(sh, ctrl, [&](uint32_t key, int idx, bool valid) {
        if (valid && key > Pn) emit_winner(key, idx);
      });
      // Exact duplicates of the threshold key: the first `need` of them in index order win.
      // Shards are contiguous and ordered by rank, so this CTA takes its first `quota`.
      const uint32_t tie_prefix = ctrl->tie_prefix;
      const uint32_t local_c = ctrl->local_c;
      const uint32_t quota = need > tie_prefix ? min(need - tie_prefix, local_c) : 0u;
      const uint32_t obase = (uint32_t)kK - need + tie_prefix;
      uint32_t run = 0;  // ties seen so far in this shard (uniform over the CTA)
      const bool use_stage = ctrl->stage_fail == 0u;
      for (int gb = sh.g0; gb < sh.g1 && run < quota; gb += NT) {
        const int g = gb + tid;
        const bool in = g < sh.g1;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (in) {
          const int gl = g - sh.g0;
          x = (use_stage && gl < sh.n_stage && granule_full(sh, g)) ? sh.stage[gl] : load_granule(sh, g);
        }
        const int i0 = 4 * g - sh.a;
        const float xv[4] = {x.x, x.y, x.z, x.w};
        bool m[4];
        uint32_t c = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          m[j] = in && (unsigned)(i0 + j) < (unsigned)len && fftopk_key_from_bits(__float_as_uint(xv[j])) == Pn;
          c += m[j] ? 1u : 0u;
        }
        // block exclusive scan of c in thread order
        uint32_t incl = c;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const uint32_t v = __shfl_up_sync(kFull, incl, off);
          if (lane >= off) incl += v;
        }
        if (lane == 31) ctrl->wtot[warp] = incl;
        __syncthreads();
        const uint32_t wv = (lane < NT / 32) ? ctrl->wtot[lane] : 0u;
        const uint32_t before = warp_sum(lane < warp ? wv : 0u);
        const uint32_t total = warp_sum(wv);
        uint32_t rnk = run + before + incl - c;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (m[j]) {
            if (rnk < quota && obase + rnk < (uint32_t)kK) {
              out_idx[obase + rnk] = i0 + j + p.idx_offset;
              if (out_key) out_key[obase + rnk] = Pn;
            }
            ++rnk;
          }
        }
        run += total;
        __syncthreads();
      }
    }
    break;
  }

  // No CTA may leave while a peer can still read its histograms or write into rank 0's
  // candidate buffer: one last cluster barrier for every mode.
  cluster.sync();

  if (mode == kModeGather && rank == 0) {
    const int n = (int)min(ctrl->cand_count, (uint32_t)p.cand_cap);
    const int shift = round_shift(r);
    int idx_bits = 32 - __clz(len - 1);
    cta_finish<NT>(cand, n, need, 32 + shift, (uint64_t)P, idx_bits, hist[0], ctrl, out_idx, out_key,
                   (uint32_t)kK - need, p.idx_offset, p.status);
  }
  if (tid == 0 && p.status) {
    uint32_t st = 0;
    if (ctrl->stage_fail) st |= (uint32_t)FFTOPK_ST_STAGE_TIMEOUT;
    if (mode == kModeAbort) st |= (uint32_t)FFTOPK_ST_INTERNAL;
    if (st) atomicOr(p.status, st);
  }
  if (ctrl->stage_fail && tid == 0) {
    // a copy that missed its bound may still be in flight: wait for it (bounded) before exit
    const int nchunk = (sh.n_stage + sh.chunk_g - 1) / sh.chunk_g;
    for (int c = 0; c < nchunk; ++c) (void)mbar_wait_bounded(&ctrl->mbar[c], 0u);
  }
}

// -----------------------------------------------------------------------------------------
// Merge of all-gathered shard candidates: one CTA per row, candidates held in shared memory.
// -----------------------------------------------------------------------------------------
template <int NT>
__global__ void __launch_bounds__(NT, 1) merge2048_kernel(const uint32_t* __restrict__ cand_key,
                                                         const int32_t* __restrict__ cand_idx, int G, int B,
                                                         int32_t* __restrict__ out_idx_all,
                                                         uint32_t* __restrict__ out_key_all, uint32_t* status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  uint32_t* hist = reinterpret_cast<uint32_t*>(smem_raw);
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(hist + kFinishBins);
  uint64_t* cand = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(ctrl) + ((sizeof(Ctrl) + 127) & ~127u));
  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  const int n = G * kK;
  int32_t* out_idx = out_idx_all + (int64_t)row * kK;
  uint32_t* out_key = out_key_all ? out_key_all + (int64_t)row * kK : nullptr;

  if (tid == 0) ctrl->run_total = 0u;
  __syncthreads();
  uint32_t nvalid = 0;
  for (int i = tid; i < n; i += NT) {
    const int g = i / kK, j = i % kK;
    const int64_t src = ((int64_t)g * B + row) * kK + j;
    const int32_t idx = __ldg(cand_idx + src);
    const uint32_t key = __ldg(cand_key + src);
    const bool v = idx >= 0;
    cand[i] = v ? (((uint64_t)key << 32) | (uint64_t)(~(uint32_t)idx)) : 0ull;
    nvalid += v ? 1u : 0u;
  }
  nvalid = warp_sum(nvalid);
  if ((tid & 31) == 0 && nvalid) atomicAdd(&ctrl->run_total, nvalid);
  __syncthreads();
  const uint32_t total = ctrl->run_total;
  if (total <= (uint32_t)kK) {
    // fewer candidates than k: keep them all (gather order), pad with -1
    if (tid == 0) ctrl->fslot = 0u;
    __syncthreads();
    for (int i = tid; i < n; i += NT) {
      const uint64_t c = cand[i];
      if (c != 0ull) {
        const uint32_t pos = atomicAdd(&ctrl->fslot, 1u);
        out_idx[pos] = (int32_t)(~(uint32_t)c);
        if (out_key) out_key[pos] = (uint32_t)(c >> 32);
      }
    }
    for (int i = (int)total + tid; i < kK; i += NT) {
      out_idx[i] = -1;
      if (out_key) out_key[i] = 0u;
    }
    return;
  }
  cta_finish<NT>(cand, n, (uint32_t)kK, 64, 0ull, 31, hist, ctrl, out_idx, out_key, 0u, 0, status);
}

}  // namespace fftopk

// =============================================================================================
// Host side: launch plan and C ABI
// =============================================================================================
namespace {

using namespace fftopk;

thread_local int g_last_cuda_error = 0;

struct Tuning {
  int cluster = -1, threads = -1, stage_kib = -1, cand_cap = -1;
};
Tuning g_tuning;

struct DeviceInfo {
  bool ready = false;
  int err = 0;
  int sm_count = 0;
  int smem_optin = 0;
  int cc_major = 0;
  int max_cluster_1024 = 0;  // largest cluster size that can be scheduled with the full-smem config
};
DeviceInfo g_dev[64];

constexpr size_t fixed_smem_bytes() {
  return (size_t)(2 * kMaxBins + 2 * kSup + kMaxCluster * kSup) * 4 + ((sizeof(Ctrl) + 127) & ~(size_t)127);
}

int cuda_fail(cudaError_t e) {
  g_last_cuda_error = (int)e;
  return FFTOPK_ECUDA;
}

template <int NT>
int setup_kernel(int smem_optin) {
  cudaError_t e = cudaFuncSetAttribute(select2048_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin);
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaFuncSetAttribute(select2048_kernel<NT>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
  if (e != cudaSuccess) return cuda_fail(e);
  return 0;
}

int device_info(DeviceInfo** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= 64) return FFTOPK_EDEVICE;
  DeviceInfo& d = g_dev[dev];
  if (!d.ready) {
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, dev);
    if (e != cudaSuccess) return cuda_fail(e);
    d.sm_count = prop.multiProcessorCount;
    d.smem_optin = (int)prop.sharedMemPerBlockOptin;
    d.cc_major = prop.major;
    if (prop.major < 10) return FFTOPK_EDEVICE;
    int rc = setup_kernel<1024>(d.smem_optin);
    if (rc) return rc;
    rc = setup_kernel<512>(d.smem_optin);
    if (rc) return rc;
    e = cudaFuncSetAttribute(merge2048_kernel<1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, d.smem_optin);
    if (e != cudaSuccess) return cuda_fail(e);
    // can a 16-CTA cluster with the largest shared-memory footprint be co-scheduled?
    d.max_cluster_1024 = 8;
    {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(16, 1, 1);
      cfg.blockDim = dim3(1024, 1, 1);
      cfg.dynamicSmemBytes = (size_t)d.smem_optin;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 16;
      at[0].val.clusterDim.y = 1;
      at[0].val.clusterDim.z = 1;
      cfg.attrs = at;
      cfg.numAttrs = 1;
      int nclusters = 0;
      e = cudaOccupancyMaxActiveClusters(&nclusters, select2048_kernel<1024>, &cfg);
      if (e == cudaSuccess && nclusters >= 1) d.max_cluster_1024 = 16;
      (void)cudaGetLastError();
    }
    d.ready = true;
  }
  *out = &d;
  return 0;
}

struct Plan {
  int cluster, threads, smem_bytes, stage_floats, cand_cap;
};

int floor_pow2(int64_t v) {
  int r = 1;
  while ((int64_t)r * 2 <= v) r *= 2;
  return r;
}

Plan make_plan(const DeviceInfo& d, int B, int64_t L) {
  Plan pl;
  // CTAs per row: as many as keep the whole grid on the device at once (one CTA per SM),
  // but never so many that a shard drops below ~4K elements.
  int c = floor_pow2(d.sm_count / (B > 0 ? B : 1) > 0 ? d.sm_count / (B > 0 ? B : 1) : 1);
  if (c > d.max_cluster_1024) c = d.max_cluster_1024;
  int by_len = floor_pow2(L / 4096 > 0 ? L / 4096 : 1);
  if (c > by_len) c = by_len;
  if (c < 1) c = 1;
  pl.cluster = c;
  pl.threads = 1024;
  pl.cand_cap = 4096;
  int stage_kib = -1;
  if (g_tuning.cluster > 0) pl.cluster = g_tuning.cluster;
  if (g_tuning.threads > 0) pl.threads = g_tuning.threads;
  if (g_tuning.cand_cap > 0) pl.cand_cap = (g_tuning.cand_cap + 15) & ~15;
  if (g_tuning.stage_kib >= 0) stage_kib = g_tuning.stage_kib;
  const size_t fixed = fixed_smem_bytes() + (size_t)pl.cand_cap * 8;
  size_t avail = (size_t)d.smem_optin > fixed ? (size_t)d.smem_optin - fixed : 0;
  if (stage_kib >= 0 && (size_t)stage_kib * 1024 < avail) avail = (size_t)stage_kib * 1024;
  // no point in staging more than the largest shard
  const int64_t gn = (L + 3 + 3) / 4;
  const int64_t per = ((((gn + pl.cluster - 1) / pl.cluster) + 31) & ~(int64_t)31) * 16;  // bytes
  if ((int64_t)avail > per) avail = (size_t)per;
  avail &= ~(size_t)511;
  pl.stage_floats = (int)(avail / 4);
  pl.smem_bytes = (int)(fixed + avail);
  return pl;
}

}  // namespace

extern "C" {

int fftopk_version(void) { return 100; }

const char* fftopk_strerror(int code) {
  switch (code) {
    case FFTOPK_OK: return "ok";
    case FFTOPK_EINVAL: return "invalid argument";
    case FFTOPK_ECUDA: return "CUDA runtime call failed";
    case FFTOPK_EDEVICE: return "device is not an sm_100-class GPU with cluster launch";
    case FFTOPK_ERANGE: return "size out of the supported range";
    default: return "unknown error";
  }
}

int fftopk_last_cuda_error(void) { return g_last_cuda_error; }

uint32_t fftopk_key_of(float x) {
  uint32_t bits;
  __builtin_memcpy(&bits, &x, 4);
  return fftopk_key_from_bits(bits);
}

int fftopk_set_tuning(int32_t cluster_ctas, int32_t threads, int32_t stage_kib, int32_t cand_cap) {
  if (cluster_ctas > 0 && (cluster_ctas > kMaxCluster || (cluster_ctas & (cluster_ctas - 1)))) return FFTOPK_EINVAL;
  if (threads > 0 && threads != 512 && threads != 1024) return FFTOPK_EINVAL;
  if (cand_cap > 0 && (cand_cap < kSmall || cand_cap > 16384)) return FFTOPK_EINVAL;
  g_tuning.cluster = cluster_ctas;
  g_tuning.threads = threads;
  g_tuning.stage_kib = stage_kib;
  g_tuning.cand_cap = cand_cap;
  return FFTOPK_OK;
}

int fftopk_plan(int32_t B, int64_t L, int32_t plan[6]) {
  if (!plan || B < 0 || L < 0) return FFTOPK_EINVAL;
  DeviceInfo* d = nullptr;
  int rc = device_info(&d);
  if (rc) return rc;
  const Plan pl = make_plan(*d, B, L);
  plan[0] = pl.cluster;
  plan[1] = pl.threads;
  plan[2] = pl.smem_bytes;
  plan[3] = pl.stage_floats;
  plan[4] = pl.cand_cap;
  plan[5] = d->sm_count;
  return FFTOPK_OK;
}

int fftopk_select2048(const float* score, int64_t row_stride, int32_t B, int64_t L, const int32_t* lengths,
                      const int32_t* row_starts, int32_t* out_idx, uint32_t* out_key, int32_t idx_offset,
                      uint32_t* status, void* cuda_stream) {
  if (B < 0 || L < 0 || row_stride < 0) return FFTOPK_EINVAL;
  if (B == 0) return FFTOPK_OK;
  if (!score || !lengths || !out_idx) return FFTOPK_EINVAL;
  if ((reinterpret_cast<uintptr_t>(score) & 3u) != 0) return FFTOPK_EINVAL;
  if (L > (int64_t)0x7fffffff - 8 || (int64_t)B * kMaxCluster > (int64_t)0x7fffffff) return FFTOPK_ERANGE;
  DeviceInfo* d = nullptr;
  int rc = device_info(&d);
  if (rc) return rc;
  const Plan pl = make_plan(*d, B, L);

  SelectParams p;
  p.score = score;
  p.row_stride = row_stride;
  p.L = L;
  p.lengths = lengths;
  p.row_starts = row_starts;
  p.out_idx = out_idx;
  p.out_key = out_key;
  p.status = status;
  p.B = B;
  p.idx_offset = idx_offset;
  p.stage_floats = pl.stage_floats;
  p.cand_cap = pl.cand_cap;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)B * (unsigned)pl.cluster, 1, 1);
  cfg.blockDim = dim3((unsigned)pl.threads, 1, 1);
  cfg.dynamicSmemBytes = (size_t)pl.smem_bytes;
  cfg.stream = static_cast<cudaStream_t>(cuda_stream);
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = (unsigned)pl.cluster;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  cudaError_t e;
  if (pl.threads == 1024) {
    e = cudaLaunchKernelEx(&cfg, select2048_kernel<1024>, p);
  } else {
    e = cudaLaunchKernelEx(&cfg, select2048_kernel<512>, p);
  }
  if (e != cudaSuccess) return cuda_fail(e);
  return FFTOPK_OK;
}

int fftopk_merge2048(const uint32_t* cand_key, const int32_t* cand_idx, int32_t G, int32_t B, int32_t* out_idx,
                     uint32_t* out_key, uint32_t* status, void* cuda_stream) {
  if (B < 0 || G < 1) return FFTOPK_EINVAL;
  if (G > 8) return FFTOPK_ERANGE;
  if (B == 0) return FFTOPK_OK;
  if (!cand_key || !cand_idx || !out_idx) return FFTOPK_EINVAL;
  DeviceInfo* d = nullptr;
  int rc = device_info(&d);
  if (rc) return rc;
  const size_t smem = (size_t)kFinishBins * 4 + ((sizeof(Ctrl) + 127) & ~(size_t)127) + (size_t)G * kK * 8;
  merge2048_kernel<1024><<<dim3((unsigned)B), dim3(1024), smem, static_cast<cudaStream_t>(cuda_stream)>>>(
      cand_key, cand_idx, G, B, out_idx, out_key, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  return FFTOPK_OK;
}

}  // extern "C"
