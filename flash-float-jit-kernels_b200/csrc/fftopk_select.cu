// Per-row top-2048 radix selector for B200 (sm_100a): one thread-block cluster per row.
//
// What it replaces in the reference: topk_kernel and fast_topk_split_kv_cuda_tl
// (jit_kernel/csrc/topk_indexer/topk_indexer_radix.cu:456-869) and the host launcher
// fast_topk_interface (:1051-1158).
//
// Shape of the computation for one row of `len` > 2048 valid fp32 logits, C CTAs in the cluster,
// each owning a contiguous shard of the row:
//   1. SAMPLE. Every warp reads one to four 512-byte slabs; the slabs are spread evenly over the
//      shards, so the cluster samples the row uniformly in position. The top 12 bits of the
//      order-preserving key are histogrammed per CTA (4096 bins); a cluster also histograms key
//      bits [27:16], which give a 16-bit guess when the whole sample shares its top four key bits.
//      When the whole shard fits in registers (<= 3 granules per thread) the "sample" is the
//      shard and step 2 is exact.
//   2. PICK. After ONE cluster barrier every CTA reads its peers' 64 super-bin sums, then the 64
//      fine bins of the threshold super-bin, over distributed shared memory, and finds the bin
//      with a warp-shuffle suffix scan (no L2 atomics, no reduce-then-broadcast). From a sample it
//      takes the bin whose sample rank is the expected rank of the k-th element plus five standard
//      deviations: a lower bound of the true threshold with overwhelming probability. A lone CTA
//      does all of this in one warp and also finds the mirror-image upper bound.
//   3. FILTER. One streaming pass over the shard (128-bit loads, four or eight in flight per
//      thread) with ONE float compare per element against the bin's lower edge; the few thousand
//      elements that pass are appended, by ballot, to dense per-warp segments of a list in shared
//      memory and become (key << 32 | ~index) composites. This is the only full read of the row.
//   4. GATHER + FINISH. The segments are copied into rank 0's shared memory (one remote atomic per
//      CTA reserves the range), and after the second cluster barrier rank 0 finishes: radix rounds
//      over the composites' range, one fused output pass, and the last <= 256 undecided
//      candidates ranked by votes. A lone CTA finishes over its segments where they lie. The
//      inverted index in the composite makes equal values resolve to the lower index.
//   5. If the guess admitted fewer than k elements, a list overflowed or the threshold bin is
//      larger than rank 0's buffer (heavy ties, rows of equal values), the cluster falls back to
//      full histograms over the data: 12 + 12 + 8 key bits, re-reading the shard from L2 each
//      round, and exact ties left after 32 bits are taken in index order, shard by shard.
//
// Build-time knobs (all optional, for experiments; the defaults are what was measured best):
//   FFTOPK_SAMPLE_GRANULES  granules the cluster samples per row and thread column (2048)
//   FFTOPK_EXACT_SLABS      granules per thread up to which the shard stays in registers (3)
//   FFTOPK_1B_FACTOR        second sample round when the guessed bin holds more than factor*k (2)
//   FFTOPK_U512             128-bit loads in flight per thread of the 512-thread filter (8; 16 allowed)
//   FFTOPK_CTAS_512         512-thread CTAs per SM the register budget allows (2)
//   FFTOPK_KSMALL           undecided candidates ranked by votes (256)
//   FFTOPK_TRACE            phase timestamps of block 0 (changes no result)
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/fftopk.h"
#include "fftopk_trace.cuh"
#include "fftopk_device.cuh"
#include "fftopk_host.h"
#include "fftopk_internal.h"
#include "fftopk_key.h"
#include "fftopk_merge.cuh"

namespace fftopk {


struct SelectParams {
  const void* score;  // fp32, or fp16 / bf16 for the kernels instantiated on those types
  int64_t row_stride;
  int64_t L;
  const int32_t* lengths;
  const int32_t* row_starts;
  int32_t* out_idx;
  uint32_t* out_key;
  uint32_t* status;
  int32_t B;
  int32_t k;  // elements selected per row (the reference's op: 2048); output rows have k slots
  int32_t idx_offset;
  int32_t list_cap;  // per-CTA candidate list capacity (entries), multiple of 16
  int32_t cand_cap;  // rank 0's gathered-candidate capacity (entries), multiple of 16
  int32_t force_slow;  // tests: skip the filter path and run the full-histogram path
  int32_t overlap;     // let the next launch on the stream start before this one has finished
  // fused output transforms (all optional; reference: topk_transform_decode_kernel,
  // topk_transform_prefill_kernel, topk_transform_prefill_ragged_kernel, radix.cu:871-995)
  const int32_t* src_page_table;  // [prefill_bs, src_stride]: out = table_row[idx]
  int64_t src_stride;
  const int32_t* cu_seqlens_q;    // [prefill_bs + 1] or NULL (then table row = score row)
  int32_t prefill_bs;
  const int32_t* row_offsets;     // [B]: out = idx + row_offsets[row]
  // context-parallel publication with a device-side epoch: when cp_flag is set, the output planes
  // are shifted by ((*cp_flag + 1) & 1) * cp_half_words (the half of the comm buffer that the NEXT
  // epoch writes), so that a captured CUDA graph can be replayed
  const uint32_t* cp_flag;
  int64_t cp_half_words;
  // ... and its announcement: when cp_publish is set, the last CTA of the grid to finish (arrival
  // counter at cp_publish[kCommArriveWord]) fences and releases the epoch flag cp_publish[0] at
  // system scope, so that peers that acquire the flag see every output of this launch. cp_epoch is
  // the value to store, or 0 for "the flag's current value plus one".
  uint32_t* cp_publish;
  uint32_t cp_epoch;
  // warm start (select2048_kernel<NT, false, true> only): prev_threshold[row] is a key guess of the
  // row's k-th largest element from an earlier call (0: none), from which warm_margin is
  // subtracted; next_threshold[row] receives this call's k-th largest key (or a lower bound of it)
  const uint32_t* prev_threshold;
  uint32_t* next_threshold;
  uint32_t warm_margin;
  const uint32_t* only_rows;  // (warm-start kernel only) when set: rows with only_rows[row] == 0 are left alone
};


constexpr int kRegSlabs = 4;  // granules a thread keeps in registers when the whole shard fits

// digit schedule of the full-histogram rounds: 12 + 12 + 8 bits
__device__ __forceinline__ int round_width(int r) { return r < 2 ? 12 : 8; }
__device__ __forceinline__ int round_shift(int r) { return r == 0 ? 20 : (r == 1 ? 8 : 0); }

// Element types of the score matrix. The kernel works on granules of FOUR elements of the aligned
// view of the row - 16 bytes of fp32, 8 bytes of fp16 / bf16 - and widens 16-bit elements to fp32
// (exactly, order-preserving) as it loads them, so that keys, edges and composites are the fp32
// ones everywhere and a 16-bit row is read once, in its own width.
template <class T>
struct Elem;
template <>
struct Elem<float> {
  static __device__ __forceinline__ float4 ld4(const float* gbase, int g) {
    return __ldg(reinterpret_cast<const float4*>(gbase) + g);
  }
  static __device__ __forceinline__ float ld1(const float* p) { return __ldg(p); }
};
template <>
struct Elem<__half> {
  static __device__ __forceinline__ float4 ld4(const __half* gbase, int g) {
    const uint2 r = __ldg(reinterpret_cast<const uint2*>(gbase) + g);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ float ld1(const __half* p) { return __half2float(__ldg(p)); }
};
template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float4 ld4(const __nv_bfloat16* gbase, int g) {
    const uint2 r = __ldg(reinterpret_cast<const uint2*>(gbase) + g);  // bf16 = the upper half of an fp32
    return make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u), __uint_as_float(r.y << 16),
                       __uint_as_float(r.y & 0xffff0000u));
  }
  static __device__ __forceinline__ float ld1(const __nv_bfloat16* p) {
    return __uint_as_float((uint32_t)__bfloat16_as_ushort(__ldg(p)) << 16);
  }
};

// Shard of one CTA, in granules of four elements of the aligned view of the row: granule g covers
// row elements 4g-a .. 4g-a+3, where a in 0..3 is the row's misalignment in elements.
template <class T>
struct Shard {
  const T* gbase;      // granule-aligned address of granule 0
  int g0, g1;          // granule range of this CTA
  int i0, i1;          // the part of [g0, g1) whose granules lie completely inside the row
  int a;               // misalignment (elements)
  int len;             // valid elements in the row
};

// A granule that straddles the start or the end of the row (at most two per row): scalar loads of
// the elements that belong to the row, `fill` elsewhere. Kept out of line so that the streaming
// loops stay small enough to unroll with every load in flight.
template <class T>
__device__ __noinline__ float4 load_granule_partial(const T* gbase, int a, int len, int g, float fill) {
  const int i0 = 4 * g - a;
  float4 x = make_float4(fill, fill, fill, fill);
  const T* p = gbase + 4 * (int64_t)g;
  if ((unsigned)(i0 + 0) < (unsigned)len) x.x = Elem<T>::ld1(p + 0);
  if ((unsigned)(i0 + 1) < (unsigned)len) x.y = Elem<T>::ld1(p + 1);
  if ((unsigned)(i0 + 2) < (unsigned)len) x.z = Elem<T>::ld1(p + 2);
  if ((unsigned)(i0 + 3) < (unsigned)len) x.w = Elem<T>::ld1(p + 3);
  return x;
}

// One granule from global memory; reads only bytes that belong to the row.
template <class T>
__device__ __forceinline__ float4 load_granule(const Shard<T>& sh, int g, float fill) {
  if (g >= sh.i0 && g < sh.i1) return Elem<T>::ld4(sh.gbase, g);
  return load_granule_partial(sh.gbase, sh.a, sh.len, g, fill);
}

// A kept element on its way into the list: the raw float bits and the row index. It becomes a
// (key << 32 | ~idx) composite later, in a dense pass - the hit loop is the divergent part of
// the filter and every instruction in it is paid by a whole warp for one or two lanes.
__device__ __forceinline__ uint64_t raw_to_composite(uint64_t raw, uint32_t& kmax) {
  const uint32_t key = fftopk_key_from_bits((uint32_t)(raw >> 32));
  kmax = max(kmax, key);
  return ((uint64_t)key << 32) | (uint64_t)(~(uint32_t)raw);
}

// Overflow of a thread's private candidate slots: a shared spill area, slots from one counter
// (rare, so the serialising atomic does not matter). Converts on the spot. Out of line to keep
// the filter loop small.
__device__ __noinline__ void spill_push(Ctrl* ctrl, uint64_t* spill, uint32_t spill_cap, uint64_t raw) {
  const uint32_t slot = warp_alloc(&ctrl->lcount);
  if (slot < spill_cap) {
    uint32_t k = 0;
    spill[slot] = raw_to_composite(raw, k);
    atomicMax(&ctrl->spill_kmax, k);
  } else {
    ctrl->pub_flag = 1u;
  }
}

// The one full read of the shard: every element x with !(x < edge) is kept as a
// (key << 32 | ~idx) composite. Per loop trip a thread has U 128-bit loads in flight and spends
// one compare and one predicated OR per element on a pass mask. Candidates go to a segment of the
// shared-memory list that belongs to the WARP and is filled densely: the warp walks its lanes'
// hits together, one hit per lane and loop trip, and a ballot gives each its slot - no atomic, and
// the segment's length lives in a register that is the same in all lanes. (Allocating from one
// shared counter serialised at ~20 cycles per candidate; slots private to a thread left more than
// half of the list empty, and every later pass paid for the empty slots.) A hit's value cannot be
// selected out of 4*U registers by a computed index, so it is fetched again. kStage = false does
// that inside the hit loop (the loads of the warps of a CTA overlap; best when hits are few and
// the latency of one call counts); kStage = true stores only the row index there and fetches all
// values in the dense pass that builds the composites afterwards, several loads in flight per
// lane (best when most trips have hits: a dependent load per trip of the hit loop would stall
// the warp each time). Candidates beyond the segment's capacity go to the shared spill area.
// Returns the number of candidates the warp found (those beyond seg_cap went to the spill area);
// kmax is the largest key among the entries this lane converted; post(key) is called for each of them.
template <int NT, int U, bool kStage, class T, class Post>
__device__ __forceinline__ uint32_t filter_shard(const Shard<T>& sh, float edge, uint64_t* seg, uint32_t seg_cap, Ctrl* ctrl,
                                                 uint64_t* spill, uint32_t spill_cap, uint32_t& kmax, Post&& post) {
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const unsigned lt = (1u << lane) - 1u;
  const float ninf = __uint_as_float(0xff800000u);
  const T* gbase = sh.gbase;
  const int fa = sh.a, fi1 = sh.i1, len = sh.len;
  uint32_t wcnt = 0;  // candidates of this warp so far (warp-uniform)
  uint32_t* seg32 = reinterpret_cast<uint32_t*>(seg);  // staging: candidate j's row index in word j
  auto keep = [&](bool has, int idx) {  // called by the whole warp
    const unsigned b = __ballot_sync(kFull, has);
    if (has) {
      const uint32_t pos = wcnt + (uint32_t)__popc(b & lt);
      if (kStage && pos < seg_cap) {
        seg32[pos] = (uint32_t)idx;
      } else {
        const uint64_t raw = ((uint64_t)__float_as_uint(Elem<T>::ld1(gbase + idx + fa)) << 32) | (uint64_t)(uint32_t)idx;
        if (pos < seg_cap) {
          seg[pos] = raw;
        } else {
          spill_push(ctrl, spill, spill_cap, raw);
        }
      }
    }
    wcnt += (uint32_t)__popc(b);
  };
  // one trip over granules gb + u*NT + tid, u < U; a `full` trip lies inside the shard entirely
  auto trip = [&](int gb, auto full) {
    float4 x[U];
    using Mask = std::conditional_t<(U > 8), uint64_t, uint32_t>;
    Mask vmask = ~(Mask)0;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int g = gb + u * NT + tid;
      if constexpr (decltype(full)::value) {
        x[u] = Elem<T>::ld4(gbase, g);
      } else {
        x[u] = make_float4(ninf, ninf, ninf, ninf);
        if (g < fi1) {
          x[u] = Elem<T>::ld4(gbase, g);
        } else {
          vmask &= ~((Mask)0xfu << (4 * u));  // (padding would pass an edge of -inf)
        }
      }
    }
    // pass mask of this thread's 4*U elements: bit 4u+e
    Mask mask = 0;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!(x[u].x < edge)) mask |= (Mask)1u << (4 * u);
      if (!(x[u].y < edge)) mask |= (Mask)2u << (4 * u);
      if (!(x[u].z < edge)) mask |= (Mask)4u << (4 * u);
      if (!(x[u].w < edge)) mask |= (Mask)8u << (4 * u);
    }
    if constexpr (!decltype(full)::value) mask &= vmask;
    const int el0 = 4 * (gb + tid);
    while (__any_sync(kFull, mask != 0)) {
      const bool has = mask != 0;
      const int bit = (sizeof(Mask) == 8 ? __ffsll((long long)mask) : __ffs((int)mask)) - 1;
      mask &= mask - 1;
      keep(has, el0 + (bit >> 2) * (4 * NT) + (bit & 3) - fa);
    }
  };
  int gb = sh.i0;
  for (; gb + NT * U <= fi1; gb += NT * U) trip(gb, std::true_type{});
  if (gb < fi1) trip(gb, std::false_type{});
  // edge granules [g0, i0) and [i1, g1): at most one each, visited by lane 0 of warps 0 and 1
  if (tid < 64) {  // (whole warps: keep() votes)
    const int ge = (tid == 0) ? sh.g0 : ((tid == 32) ? sh.i1 : -1);
    const int ge_end = (tid == 0) ? sh.i0 : sh.g1;
    const bool mine = ge >= 0 && ge < ge_end;
    if (__any_sync(kFull, mine)) {
      float4 x = make_float4(ninf, ninf, ninf, ninf);
      if (mine) x = load_granule_partial(sh.gbase, sh.a, len, ge, ninf);
      const int e0 = 4 * ge - fa;
      const float xv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int e = 0; e < 4; ++e)
        keep(mine && (unsigned)(e0 + e) < (unsigned)len && !(xv[e] < edge), e0 + e);
    }
  }
  // Dense conversion of the warp's segment.
  kmax = 0u;
  const uint32_t own = min(wcnt, seg_cap);
  __syncwarp();
  if constexpr (kStage) {
    // Fetch the values again (L1/L2 hits, four loads in flight per lane) and expand the staged
    // indices into composites in place, from the top down: the composites of entries
    // [j0, j0 + 128) cover words [2*j0, 2*j0 + 256), which holds no index not yet read.
    for (int j0 = (int)((own + 127u) & ~127u) - 128; j0 >= 0; j0 -= 128) {
      uint32_t idx[4], bits[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t j = (uint32_t)j0 + 32u * u + lane;
        idx[u] = j < own ? seg32[j] : 0u;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (!FFTOPK_CHECK(7, idx[u], len, ctrl_status(ctrl))) idx[u] = 0u;
        bits[u] = __float_as_uint(Elem<T>::ld1(gbase + idx[u] + fa));  // (index 0 is always readable)
      }
      __syncwarp();
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t j = (uint32_t)j0 + 32u * u + lane;
        if (j < own) {
          const uint64_t c = raw_to_composite(((uint64_t)bits[u] << 32) | idx[u], kmax);
          seg[j] = c;
          post((uint32_t)(c >> 32));
        }
      }
      __syncwarp();
    }
  } else {
    for (uint32_t j = lane; j < own; j += 32) {
      const uint64_t c = raw_to_composite(seg[j], kmax);
      seg[j] = c;
      post((uint32_t)(c >> 32));
    }
  }
  return wcnt;
}

// Visit every valid element of the shard: op(key, idx). Interior granules are read with
// unconditional 128-bit loads, four in flight per thread; the at most two granules that straddle
// the row's ends are visited by one thread each through scalar loads.
template <int NT, class T, class Op>
__device__ __forceinline__ void scan_shard(const Shard<T>& sh, Op&& op) {
  const int tid = threadIdx.x;
  const T* gbase = sh.gbase;
  const int a = sh.a, i1 = sh.i1;
  constexpr int U = 4;
  for (int gb = sh.i0; gb < i1; gb += NT * U) {
    float4 x[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int g = gb + u * NT + tid;
      x[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (g < i1) x[u] = Elem<T>::ld4(gbase, g);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int g = gb + u * NT + tid;
      if (g < i1) {
        const int e0 = 4 * g - a;
        op(fftopk_key_from_bits(__float_as_uint(x[u].x)), e0 + 0);
        op(fftopk_key_from_bits(__float_as_uint(x[u].y)), e0 + 1);
        op(fftopk_key_from_bits(__float_as_uint(x[u].z)), e0 + 2);
        op(fftopk_key_from_bits(__float_as_uint(x[u].w)), e0 + 3);
      }
    }
  }
  // edge granules of this shard: [g0, i0) and [i1, g1), at most one granule each
  const int ge = (tid == 0) ? sh.g0 : ((tid == 32) ? sh.i1 : -1);
  const int ge_end = (tid == 0) ? sh.i0 : sh.g1;
  if (ge >= 0 && ge < ge_end) {
    const float4 x = load_granule_partial(sh.gbase, sh.a, sh.len, ge, 0.f);
    const int e0 = 4 * ge - a;
    const float xv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if ((unsigned)(e0 + e) < (unsigned)sh.len) op(fftopk_key_from_bits(__float_as_uint(xv[e])), e0 + e);
    }
  }
}

// First search of the sampled path, over TWO sample histograms built in the same pass:
//   A: key bits [31:20]   (4096 bins, valid for any data, 8 bins per octave of magnitude)
//   B: key bits [27:16]   (4096 bins, 128 per octave) - meaningful only among keys that share the
//      top four bits (sign and the three high exponent bits)
// If every sampled key shares those four bits - one super-bin group of A holds the whole sample,
// which is the normal case for indexer logits (one sign, magnitudes within a factor of 2^32) - the
// pick is made on B and yields a 16-bit key prefix, fine enough that no second sample round is
// needed; otherwise on A (12 bits). Same two barriers and two rounds of remote reads as one search.
struct DualPick {
  bool ok;
  uint32_t prefix;  // the guessed key prefix ...
  int pbits;        // ... and its length in bits (12 or 16)
  uint32_t need2;   // sample rank still to go inside the guessed bin
  uint32_t cnt;     // sample elements in the guessed bin
  uint32_t total;   // sample size (cluster-wide)
  int focus_bin;    // lone CTA only: bin (same width as the guess) the threshold will not lie above; -1: unknown
};

template <int NT, class NeedFn, class NeedHiFn>
__device__ __forceinline__ DualPick cluster_pick_dual(cg::cluster_group& cluster, int C, const uint32_t* ha,
                                                      const uint32_t* sa, const uint32_t* hb, const uint32_t* sb,
                                                      bool dual, Ctrl* ctrl, int& pick_no, NeedFn&& need_of,
                                                      NeedHiFn&& need_hi_of) {
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  constexpr int fine = kMaxBins / kSup;
  if (C == 1) {
    // A lone CTA has nothing to exchange: one warp reads the super-bin sums, picks, reads the fine
    // bins of the super-bins it needs and picks again; one block barrier publishes the result.
    // (The totals buffers stay untouched, so the search counter does not advance.)
    // It also brackets the threshold from above: the bin of the mirror-image sample rank, which
    // the true threshold lies below with the same confidence. The finish then spends its first
    // digit between the two bins instead of on the whole range up to the row's maximum.
    if (warp == 0) {
      const uint32_t lo = sa[2 * lane], hi = sa[2 * lane + 1];
      const uint32_t total = warp_sum(lo + hi);
      const uint32_t need = need_of(total);
      const uint32_t need_hi = need_hi_of(total);
      int ts = -1, ts_hi = -1, tf = -1, focus_bin = -1;
      uint32_t above = 0, cnt = 0, above_hi = 0, cnt_hi = 0, above_f = 0, cnt_t = 0;
      bool ok = need > 0 && warp_pick64(lo, hi, need, ts, above, cnt);
      if (ok) {
        const uint32_t flo = ha[ts * fine + 2 * lane], fhi = ha[ts * fine + 2 * lane + 1];
        ok = warp_pick64(flo, fhi, need - above, tf, above_f, cnt_t);
        if (ok && need_hi > 0 && warp_pick64(lo, hi, need_hi, ts_hi, above_hi, cnt_hi)) {
          int tf_hi = -1;
          uint32_t a2 = 0, c2 = 0;
          const uint32_t glo = ha[ts_hi * fine + 2 * lane], ghi = ha[ts_hi * fine + 2 * lane + 1];
          if (warp_pick64(glo, ghi, need_hi - above_hi, tf_hi, a2, c2)) focus_bin = ts_hi * fine + tf_hi;
        }
      }
      if (lane == 0) {
        ctrl->t = ok ? ts * fine + tf : -1;
        ctrl->above = ok ? need - above - above_f : 0u;
        ctrl->cnt = cnt_t;
        ctrl->run_total = total;
        ctrl->focus_bin = focus_bin;
      }
    }
    __syncthreads();
    FFTOPK_MARK(43);
    DualPick d;
    d.focus_bin = ctrl->focus_bin;
    d.ok = ctrl->t >= 0;
    d.pbits = 12;
    d.prefix = (uint32_t)ctrl->t;
    d.need2 = ctrl->above;
    d.cnt = ctrl->cnt;
    d.total = ctrl->run_total;
    return d;
  }
  uint32_t* tot = ctrl->tot[pick_no & 1];
  uint32_t* tot2 = ctrl->tot2[pick_no & 1];
  for (int i = tid; i < C * kSup; i += NT) {
    const int q = i / kSup, b = i % kSup;
    const uint32_t* ra = C == 1 ? sa : cluster.map_shared_rank(sa, q);
    red_shared_add(&tot[b], ra[b]);
    if (dual) {
      const uint32_t* rb = C == 1 ? sb : cluster.map_shared_rank(sb, q);
      red_shared_add(&ctrl->totb[b], rb[b]);
    }
  }
  __syncthreads();
  FFTOPK_MARK(40);
  if (warp == 0) {
    const uint32_t lo = tot[2 * lane], hi = tot[2 * lane + 1];
    const uint32_t total = warp_sum(lo + hi);
    const uint32_t need = need_of(total);
    // four super-bins = 256 bins of A = one value of the top four key bits
    const uint32_t pair = lo + hi;
    const uint32_t grp = pair + __shfl_xor_sync(kFull, pair, 1);
    const unsigned one = __ballot_sync(kFull, fine_histogram_usable(dual, total, grp));
    const bool use_b = one != 0u;
    const uint32_t lob = ctrl->totb[2 * lane], hib = ctrl->totb[2 * lane + 1];
    uint32_t above = 0, cnt = 0;
    int ts = -1;
    const uint32_t plo = use_b ? lob : lo, phi = use_b ? hib : hi;
    const bool ok = need > 0 && warp_pick64(plo, phi, need, ts, above, cnt);
    if (lane == 0) {
      ctrl->sup_sel = ok ? ts : -1;
      ctrl->sup_above = above;
      ctrl->need = need;
      ctrl->run_total = total;
      ctrl->dual_b = use_b ? 1u : 0u;
      ctrl->dual_g = use_b ? (uint32_t)((__ffs(one) - 1) >> 1) : 0u;
    }
  }
  __syncthreads();
  FFTOPK_MARK(41);
  const int ssel = ctrl->sup_sel;
  const bool use_b = ctrl->dual_b != 0u;
  if (ssel >= 0) {
    const uint32_t* h = use_b ? hb : ha;
    for (int i = tid; i < C * kSup; i += NT) {
      const int q = i / kSup, f = i % kSup;
      const uint32_t* rh = C == 1 ? h : cluster.map_shared_rank(h, q);
      red_shared_add(&tot2[f], rh[ssel * fine + f]);
    }
  }
  __syncthreads();
  FFTOPK_MARK(42);
  if (tid < kSup) {
    ctrl->tot[(pick_no + 1) & 1][tid] = 0u;
    ctrl->tot2[(pick_no + 1) & 1][tid] = 0u;
  }
  ++pick_no;
  if (warp == 0) {
    int tf = -1;
    uint32_t above_f = 0, cnt_t = 0;
    bool ok = false;
    if (ssel >= 0) {
      const uint32_t lo = tot2[2 * lane], hi = tot2[2 * lane + 1];
      ok = warp_pick64(lo, hi, ctrl->need - ctrl->sup_above, tf, above_f, cnt_t);
    }
    if (lane == 0) {
      ctrl->t = ok ? ssel * fine + tf : -1;
      ctrl->above = ok ? ctrl->need - ctrl->sup_above - above_f : 0u;
      ctrl->cnt = cnt_t;
    }
  }
  __syncthreads();
  FFTOPK_MARK(43);
  DualPick d;
  d.focus_bin = -1;
  d.ok = ctrl->t >= 0;
  d.pbits = use_b ? 16 : 12;
  d.prefix = guess_prefix(use_b, ctrl->dual_g, (uint32_t)ctrl->t);
  d.need2 = ctrl->above;
  d.cnt = ctrl->cnt;
  d.total = ctrl->run_total;
  return d;
}

// Everything one CTA needs to know about its row and its shared memory.
template <int NT, class T>
struct RowCtx {
  int C, rank;
  Shard<T> sh;
  uint32_t* hist0;  // two histograms of kMaxBins words, back to back
  uint32_t* sup0;   // three super-bin arrays of kSup words, back to back
  // (computed addresses instead of pointer arrays: indexing an array member with the round number
  // would force the whole struct into local memory)
  __device__ __forceinline__ uint32_t* hist(int i) const { return hist0 + i * kMaxBins; }
  __device__ __forceinline__ uint32_t* sup(int i) const { return sup0 + i * kSup; }
  uint32_t* xch;
  Ctrl* ctrl;
  Ctrl* ctrl0;
  uint64_t* list;
  uint64_t* cand;
  uint64_t* cand0;
  int32_t* out_idx;
  uint32_t* out_key;
  int32_t idx_offset;
  const int32_t* page;  // fused page-table transform: out = page[idx] (NULL: out = idx + idx_offset)
  int32_t cand_cap;
  int32_t list_cap;
  uint32_t* status;
  uint32_t k;  // elements to select per row (2048 for the reference's op)
};

template <class Cx>
__device__ __forceinline__ void emit_winner(const Cx& cx, uint32_t base_w, uint32_t key, int idx) {
  const uint32_t pos = base_w + warp_alloc(&cx.ctrl->wslot);
  if (FFTOPK_CHECK(1, pos, cx.k, cx.status) && pos < cx.k) {
    cx.out_idx[pos] = cx.page ? __ldg(cx.page + idx) : idx + cx.idx_offset;
    if (cx.out_key) cx.out_key[pos] = key;
  }
}

// -----------------------------------------------------------------------------------------
// Full-histogram path: every round re-reads the shard (from L2) and histograms the next key
// digit of the elements that still match the threshold prefix. Handles anything: lists that
// would overflow, threshold bins larger than rank 0's buffer, rows of identical values.
// Returns the final mode; `need`, `P` and `r` describe where it stopped.
// -----------------------------------------------------------------------------------------
template <int NT, class T>
__device__ __forceinline__ int refine_from_data(RowCtx<NT, T>& cx, uint32_t& need, uint32_t& P, int& r, int& pick_no) {
  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int C = cx.C, rank = cx.rank;
  const Shard<T>& sh = cx.sh;
  Ctrl* ctrl = cx.ctrl;
  uint32_t* xch = cx.xch;

  // peers may still be reading this CTA's histograms from the attempt that fell back
  cluster_sync(cluster, C);
  {
    uint4* h4 = reinterpret_cast<uint4*>(cx.hist(0));
    for (int i = tid; i < kMaxBins / 4; i += NT) h4[i] = make_uint4(0u, 0u, 0u, 0u);
    if (tid == 0) {
      ctrl->pub_flag = 0u;
      ctrl->win_count = 0u;   // rank 0's copies are the cluster-wide counters; nobody touches
      ctrl->cand_count = 0u;  // them again before the cluster barrier of the first histogram pass
      ctrl->over_flag = 0u;
      ctrl->max_key = 0u;
    }
    if (tid < kSup) {
      ctrl->tot[0][tid] = ctrl->tot[1][tid] = 0u;
      ctrl->tot2[0][tid] = ctrl->tot2[1][tid] = 0u;
    }
    pick_no = 0;
  }
  __syncthreads();
  {
    uint32_t* h0 = cx.hist(0);
    scan_shard<NT, T>(sh, [&](uint32_t key, int) { hist_add(h0, key >> 20, true); });
  }
  __syncthreads();

  need = cx.k;
  P = 0;
  int mode = kModeAbort;
  for (r = 0;; ++r) {
    const int w = round_width(r);
    const int shift = round_shift(r);
    const int nb = 1 << w;
    uint32_t* h = cx.hist(r & 1);
    uint32_t* s = cx.sup(r & 1);
    compute_sup<NT>(h, s, nb);
    cluster_sync(cluster, C);  // every CTA's histogram and super-bin sums of this round are complete
    const uint32_t need_now = need;
    cluster_pick<NT>(
        cluster, C, h, s, xch, ctrl, pick_no, nb, [&](uint32_t) { return need_now; },
        [&](Picked& pk) {
          const bool last = (shift == 0);
          decide_and_allocate(cx, pk, last ? kModeTies : kModeNext, false);
          if (pk.ok && last && pk.cnt > (uint32_t)cx.cand_cap && pk.cnt != pk.need2) {
            // exact duplicates of the threshold key: ties before this shard, in rank order
            const uint32_t tp = (lane < rank) ? xch[lane * kSup + pk.tf] : 0u;
            const uint32_t tie_prefix = warp_sum(tp);
            if (lane == 0) ctrl->tie_prefix = tie_prefix;
          }
        });
    // clear the next round's histogram (peers finished reading that buffer before they arrived
    // at this round's cluster barrier)
    {
      uint4* n4 = reinterpret_cast<uint4*>(cx.hist((r + 1) & 1));
      for (int i = tid; i < kMaxBins / 4; i += NT) n4[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
    mode = ctrl->mode;
    if (mode == kModeAbort) break;
    const uint32_t Pn = (P << w) | (uint32_t)ctrl->t;
    const uint32_t Pold = P;
    const uint32_t base_w = ctrl->base_w;
    const uint32_t base_c = ctrl->base_c;
    need = ctrl->above;
    P = Pn;

    if (mode == kModeNext) {
      const int shift2 = round_shift(r + 1);
      const uint32_t mask2 = (1u << round_width(r + 1)) - 1u;
      uint32_t* h2 = cx.hist((r + 1) & 1);
      scan_shard<NT, T>(sh, [&](uint32_t key, int idx) {
        const uint32_t hh = key >> shift;
        if ((hh >> w) == Pold) {
          if (hh > Pn) emit_winner(cx, base_w, key, idx);
          hist_add(h2, (key >> shift2) & mask2, hh == Pn);
        }
      });
      __syncthreads();
      continue;
    }
    if (mode == kModeGather) {
      scan_shard<NT, T>(sh, [&](uint32_t key, int idx) {
        const uint32_t hh = key >> shift;
        if ((hh >> w) == Pold) {
          if (hh > Pn) {
            emit_winner(cx, base_w, key, idx);
          } else if (hh == Pn) {
            const uint32_t slot = base_c + warp_alloc(&ctrl->cslot);
            if (FFTOPK_CHECK(2, slot, cx.cand_cap, cx.status) && slot < (uint32_t)cx.cand_cap)
              cx.cand0[slot] = ((uint64_t)key << 32) | (uint64_t)(~(uint32_t)idx);
          }
        }
      });
    } else if (mode == kModeTakeAll) {
      scan_shard<NT, T>(sh, [&](uint32_t key, int idx) {
        const uint32_t hh = key >> shift;
        if (((hh >> w) == Pold) && hh >= Pn) emit_winner(cx, base_w, key, idx);
      });
    } else {  // kModeTies: all 32 key bits are fixed; Pn is the threshold key itself
      // (only keys under this round's prefix: larger prefixes were written by the earlier rounds,
      // and the slots reserved here are for this round's winners alone)
      scan_shard<NT, T>(sh, [&](uint32_t key, int idx) {
        if ((key >> w) == Pold && key > Pn) emit_winner(cx, base_w, key, idx);
      });
      // Exact duplicates of the threshold key: the first `need` of them in index order win.
      // Shards are contiguous and ordered by rank, so this CTA takes its first `quota`.
      const uint32_t tie_prefix = ctrl->tie_prefix;
      const uint32_t local_c = ctrl->local_c;
      const uint32_t quota = need > tie_prefix ? min(need - tie_prefix, local_c) : 0u;
      const uint32_t obase = cx.k - need + tie_prefix;
      uint32_t run = 0;  // ties seen so far in this shard (uniform over the CTA)
      for (int gb = sh.g0; gb < sh.g1 && run < quota; gb += NT) {
        const int g = gb + tid;
        const bool in = g < sh.g1;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (in) x = load_granule(sh, g, 0.f);
        const int i0 = 4 * g - sh.a;
        const float xv[4] = {x.x, x.y, x.z, x.w};
        bool m[4];
        uint32_t c = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          m[j] = in && (unsigned)(i0 + j) < (unsigned)sh.len && fftopk_key_from_bits(__float_as_uint(xv[j])) == Pn;
          c += m[j] ? 1u : 0u;
        }
        uint32_t incl = c;  // block exclusive scan of c in thread order
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
            if (rnk < quota && FFTOPK_CHECK(6, obase + rnk, cx.k, cx.status) && obase + rnk < cx.k) {
              cx.out_idx[obase + rnk] = cx.page ? __ldg(cx.page + i0 + j) : i0 + j + cx.idx_offset;
              if (cx.out_key) cx.out_key[obase + rnk] = Pn;
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
  return mode;
}

#ifndef FFTOPK_CTAS_512
#define FFTOPK_CTAS_512 2
#endif
// kAnyK = false: k is the constant 2048 of the reference's op (the compiler folds it: one register
// less in a kernel that sits at its register limit); true: k comes from the parameters.
template <int NT, bool kAnyK, bool kWarm = false, class T = float>
__device__ __forceinline__ void select_row(const SelectParams& p) {
  RowCtx<NT, T> cx;
  cg::cluster_group cluster = cg::this_cluster();
  const int C = cx.C = (int)cluster.num_blocks();
  const int rank = cx.rank = (int)cluster.block_rank();
  const int row = (int)(blockIdx.x / (unsigned)C);
  // Back-to-back kernels on one stream (every launch of this kernel is a programmatic dependent
  // launch): once every CTA of this grid has passed this point - or exited - the next kernel on
  // the stream may become resident on whatever the grid leaves free. By default this kernel then
  // waits, before its first access to global memory, until the kernel in front of it has
  // completed and its writes are visible - stream order as ever, but the launch latency of a call
  // hides behind the call before it (2 to 3 us per call in a chain of dependent calls). Only when
  // the caller has declared consecutive calls independent (fftopk_set_overlap) does it not wait:
  // the next call then fills the SMs that short rows free early.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (!p.overlap) asm volatile("griddepcontrol.wait;" ::: "memory");
  if constexpr (kWarm) {
    if (p.only_rows != nullptr && p.only_rows[row] == 0u) return;  // (uniform over the cluster)
  }
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  constexpr int NW = NT / 32;

  int64_t row_start = p.row_starts ? (int64_t)p.row_starts[row] : 0;
  row_start = row_start < 0 ? 0 : (row_start > p.L ? p.L : row_start);
  int64_t len64 = (int64_t)p.lengths[row];
  len64 = len64 < 0 ? 0 : len64;
  len64 = len64 > p.L - row_start ? p.L - row_start : len64;
  const int len = (int)len64;
  const T* rowp = static_cast<const T*>(p.score) + (int64_t)row * p.row_stride + row_start;
  const int64_t cp_shift = p.cp_flag ? (int64_t)((__ldcg(p.cp_flag) + 1u) & 1u) * p.cp_half_words : 0;
  const uint32_t K = cx.k = kAnyK ? (uint32_t)p.k : (uint32_t)kK;
  int32_t* out_idx = cx.out_idx = p.out_idx + cp_shift + (int64_t)row * K;
  uint32_t* out_key = cx.out_key = p.out_key ? p.out_key + cp_shift + (int64_t)row * K : nullptr;
  cx.idx_offset = p.idx_offset + (p.row_offsets ? __ldg(p.row_offsets + row) : 0);
  cx.page = nullptr;
  if (p.src_page_table) {
    // which table row serves this score row: the request i with cu_seqlens_q[i] <= row < cu_seqlens_q[i+1]
    // (radix.cu:925-939); without cu_seqlens_q, the row itself (decode, :880)
    int64_t req = row;
    if (p.cu_seqlens_q) {
      int lo = 0, hi = p.prefill_bs;  // invariant: cu[lo] <= row, answer in [lo, hi)
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(p.cu_seqlens_q + mid) <= row) lo = mid; else hi = mid;
      }
      req = lo;
    }
    cx.page = p.src_page_table + req * p.src_stride;
  }
  cx.cand_cap = p.cand_cap;
  cx.list_cap = p.list_cap;
  cx.status = p.status;

  // Short rows: 0..len-1 then -1 (reference: naive_topk_cuda, topk_indexer_radix.cu:152-163).
  if (len <= (int)K) {
    if (rank == 0) {
      for (int i = tid; i < (int)K; i += NT) {
        out_idx[i] = i < len ? (cx.page ? __ldg(cx.page + i) : i + cx.idx_offset) : -1;
        if (out_key) out_key[i] = i < len ? fftopk_key_from_bits(__float_as_uint(Elem<T>::ld1(rowp + i))) : 0u;
      }
      if constexpr (kWarm) {
        if (tid == 0 && p.next_threshold) p.next_threshold[row] = 0u;  // nothing to guess for such a row
      }
    }
    return;  // uniform over the cluster; no shared memory of this CTA is ever read by a peer
  }

  FFTOPK_MARK(0);
  // ---- shared memory carve ---------------------------------------------------------------
  extern __shared__ __align__(128) unsigned char smem_raw[];
  cx.hist0 = reinterpret_cast<uint32_t*>(smem_raw);
  cx.sup0 = cx.hist0 + 2 * kMaxBins;
  cx.xch = cx.sup0 + 3 * kSup;                                             // kMaxCluster * 64 words
  Ctrl* ctrl = cx.ctrl = reinterpret_cast<Ctrl*>(cx.xch + kMaxCluster * kSup);  // 8-byte aligned
  cx.list = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(ctrl) + ((sizeof(Ctrl) + 127) & ~127u));
  // a cluster of one CTA has nobody to gather from: its candidate buffer IS the list
  cx.cand = C == 1 ? cx.list : cx.list + p.list_cap;
  cx.ctrl0 = C == 1 ? ctrl : cluster.map_shared_rank(ctrl, 0);
  cx.cand0 = C == 1 ? cx.cand : cluster.map_shared_rank(cx.cand, 0);
  uint64_t* list = cx.list;

  // ---- shard geometry --------------------------------------------------------------------
  Shard<T>& sh = cx.sh;
  sh.a = (int)((reinterpret_cast<uintptr_t>(rowp) / sizeof(T)) & 3u);
  sh.len = len;
  sh.gbase = rowp - sh.a;
  const int gn = (sh.a + len + 3) >> 2;
  const int per = (((gn + C - 1) / C) + 31) & ~31;
  sh.g0 = min(rank * per, gn);
  sh.g1 = min(sh.g0 + per, gn);
  sh.i0 = max(sh.g0, sh.a > 0 ? 1 : 0);
  sh.i1 = max(sh.i0, min(sh.g1, ((sh.a + len) & 3) ? gn - 1 : gn));
  const int n_g = sh.g1 - sh.g0;
  // Whole shard in registers (same answer in every CTA of the cluster: `per` is rank-independent).
#ifndef FFTOPK_EXACT_SLABS
#define FFTOPK_EXACT_SLABS 3  // (with 4 the 256K row of the decode sweep took 16.4 us instead of 13.9 us)
#endif
  const bool exact = per <= NT * FFTOPK_EXACT_SLABS;
  // A second, finer sample histogram (see cluster_pick_dual) saves a cluster-wide sample round on
  // crowded data. A lone CTA does that round without any cluster traffic, and only when it is
  // needed, which costs it less than building the second histogram for every row.
  const bool dual = !exact && C > 1;
  // sampled mode: slabs read per warp
  #ifndef FFTOPK_SAMPLE_GRANULES
#define FFTOPK_SAMPLE_GRANULES 2048
#endif
  const int ns = min(kRegSlabs, max(1, FFTOPK_SAMPLE_GRANULES / (C * NT)));

  // ---- warm start: a key guess of the row's k-th largest element from an earlier call ----------
  // With a guess the row skips the sample, its histograms and the cluster-wide search: it is
  // filtered at once against the guess (minus the caller's margin). The checks after the filter
  // are the same as for a sampled guess - at least k admitted, no list overflowed - and a guess
  // that fails them sends the row to the full-histogram path, so the result is exact whatever the
  // guess was.
  uint32_t warm_key = 0u;
  if constexpr (kWarm) {
    if (p.prev_threshold != nullptr && !p.force_slow) {
      const uint32_t g = __ldg(p.prev_threshold + row);
      if (g != 0u) warm_key = g > p.warm_margin ? g - p.warm_margin : 1u;
    }
  }
  const bool warm = kWarm && warm_key != 0u;  // (uniform over the cluster)

  // ---- prologue: clear the search totals, both histograms and the control block --------------
  if (tid < kSup) {
    ctrl->tot[0][tid] = 0u;  // (the buffers with index 1 are cleared by the first search)
    ctrl->tot2[0][tid] = 0u;
    ctrl->totb[tid] = 0u;
  }
  {
    uint4* h4 = reinterpret_cast<uint4*>(cx.hist(0));
    if (!warm) {
      for (int i = tid; i < 2 * kMaxBins / 4; i += NT) h4[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    if (tid == 0) {
      if constexpr (kWarm) ctrl->thr_key = 0xffffffffu;
      ctrl->win_count = 0u;
      ctrl->cand_count = 0u;
      ctrl->pub_flag = 0u;
      ctrl->over_flag = 0u;
      ctrl->max_key = 0u;
      ctrl->wslot = 0u;
      ctrl->cslot = 0u;
      ctrl->lcount = 0u;
      ctrl->spill_kmax = 0u;
#ifdef FFTOPK_CHECKED
      ctrl->status_ptr = p.status;
#endif
    }
  }
  // ---- sample (or, for a shard that fits in registers, the whole shard) ------------------------
  // exact:   thread keeps granules g0 + j*NT + tid, j < kRegSlabs
  // sampled: warp w reads one 512-byte slab at g0 + w*stride; the slabs are spread evenly over the
  //          shard, so together the cluster samples the row uniformly in position
  float4 xr[kRegSlabs];
  int gr[kRegSlabs];
#pragma unroll
  for (int j = 0; j < kRegSlabs; ++j) {
    gr[j] = sh.g1;  // "none"
    xr[j] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (warm) {
    // Rank 0's counters are cleared: tell the cluster now, check just before the first remote
    // access - the barrier's latency hides behind the filter pass.
    __syncthreads();
    if (C > 1) cluster.barrier_arrive();
  } else {
  {
    if (exact) {
#pragma unroll
      for (int j = 0; j < kRegSlabs; ++j) {
        const int g = sh.g0 + j * NT + tid;
        if (g < sh.g1) gr[j] = g;
        if (g >= sh.i0 && g < sh.i1) xr[j] = Elem<T>::ld4(sh.gbase, g);
      }
    } else {
      // ns slabs per warp: small clusters of small CTAs sample more per thread, so that a row
      // is always sampled at about 8K positions or more (a thin sample needs a wide safety margin,
      // which means more candidates to carry)
#pragma unroll
      for (int j = 0; j < kRegSlabs; ++j) {
        if (j < ns) {
          int g;
          if (n_g >= NT * ns) {
            const int stride = (n_g / (NW * ns)) & ~7;
            g = sh.g0 + (warp * ns + j) * stride + lane;
          } else {
            g = sh.g0 + j * NT + tid;
          }
          if (g < sh.g1) gr[j] = g;
          if (g >= sh.i0 && g < sh.i1) xr[j] = Elem<T>::ld4(sh.gbase, g);
        }
      }
    }
    // granules straddling the row's ends (at most two per row), after every bulk load is in flight
#pragma unroll
    for (int j = 0; j < kRegSlabs; ++j) {
      if (gr[j] < sh.g1 && (gr[j] < sh.i0 || gr[j] >= sh.i1))
        xr[j] = load_granule_partial(sh.gbase, sh.a, sh.len, gr[j], 0.f);
    }
  }
  __syncthreads();  // histograms are cleared
  FFTOPK_MARK(1);
  {
    uint32_t* h0 = cx.hist(0);
#pragma unroll
    for (int j = 0; j < kRegSlabs; ++j) {
      if (j < ns || exact) {  // uniform over the CTA
        const bool in = gr[j] < sh.g1;
        const int i0 = 4 * gr[j] - sh.a;
        const float xv[4] = {xr[j].x, xr[j].y, xr[j].z, xr[j].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const uint32_t key = fftopk_key_from_bits(__float_as_uint(xv[e]));
          const bool ok = in && (unsigned)(i0 + e) < (unsigned)len;
          hist_add(h0, key >> 20, ok);
          if (dual) hist_add(h0 + kMaxBins, (key >> 16) & 0xfffu, ok);  // histogram B (see cluster_pick_dual)
        }
      }
    }
  }
  // (Asking L2 for the shard here with prefetch.global.L2, to hide HBM latency behind the
  // cluster-wide search, was measured: issuing the requests cost about as much as it saved.)
  __syncthreads();
  compute_sup<NT>(cx.hist(0), cx.sup(0), kMaxBins);
  if (dual) compute_sup<NT>(cx.hist(1), cx.sup(1), kMaxBins);
  FFTOPK_MARK(2);
  cluster_sync(cluster, C);  // #1: sample histograms complete
  }  // (!warm)
  FFTOPK_MARK(3);

  uint32_t need = K;
  uint32_t P = 0;
  int r = 0;
  int mode = kModeAbort;
  int pick_no = 0;        // number of cluster-wide searches so far (selects their total buffers)
  // what the finish starts from when the sampled path gathered (r < 0): the candidates' range,
  // the bound the first digit is focused below, and whether that digit's histogram is built
  // (as keys: the composites' bounds are (lo << 32) and (cap << 32) | 0xffffffff)
  uint32_t fin_lo = 0u, fin_cap = 0u, fin_focus = 0u;
  bool fin_hist = false;
  auto low_end = [](uint32_t key) { return (uint64_t)key << 32; };
  auto high_end = [](uint32_t key) { return ((uint64_t)key << 32) | 0xffffffffull; };
  int fin_wn = 0, fin_sn = 0;  // ... and, for a lone CTA, this warp's segment length and the spill count

  // Filter the shard against a key guess, gather what passes in rank 0 and check it: fills in what
  // the finish starts from, or sets mode to kModeFallback. `focus_bin` (lone CTA): a bin of `pbits`
  // bits the threshold will not lie above, or -1. `after_arrive`: the CTA has arrived at a cluster
  // barrier that must complete before rank 0's counters are touched.
  auto filter_gather = [&](const uint32_t gkey, const int focus_bin, const int pbits, const bool after_arrive) {
    // Lower edge of the guess as a float: key(x) >= gkey  <=>  !(x < edge), NaN included.
    // Keys outside the range real values map to (below -inf's key / above +inf's) admit
    // everything instead; that only lengthens the lists.
    const float edge = __uint_as_float(guess_edge_bits(gkey));
    // list layout: one segment per warp, then the spill area (an eighth of the list)
    const uint32_t spill_cap = (uint32_t)p.list_cap / 8u;
    const uint32_t seg_cap = ((uint32_t)p.list_cap - spill_cap) / NW;
    uint64_t* seg = list + (size_t)warp * seg_cap;
    uint64_t* spill = list + (size_t)NW * seg_cap;
    uint32_t kmax = 0u;
    // A lone CTA that knows a bin the threshold will not lie above builds the histogram of the
    // finish's first round while it converts its candidates (they pass through registers there
    // anyway): the digit rule needs only the guess and that bound.
    const uint32_t lowkey = guess_low_key(gkey);
    fin_lo = lowkey;
    if (C == 1 && focus_bin >= 0) {
      fin_focus = (((uint32_t)focus_bin + 1u) << (32 - pbits)) - 1u;
      fin_hist = fin_focus >= lowkey && make_finish_digit(low_end(lowkey), high_end(fin_focus)).key_only();
    }
    if (fin_hist) {  // (uniform over the CTA)
      uint32_t* fh = cx.hist(0);
      for (int b = tid; b < kFinishBins; b += NT) fh[b] = 0u;
      __syncthreads();
    }
    uint32_t* fh = cx.hist(0);
    auto round0 = [&](uint32_t key) {
      if (fin_hist) red_shared_add(&fh[make_finish_digit(low_end(fin_lo), high_end(fin_focus)).of_key(key)], 1u);
    };
#ifndef FFTOPK_U512
#define FFTOPK_U512 8
#endif
    constexpr int U = NT >= 1024 ? 4 : FFTOPK_U512;
    // about 1.5 k candidates per row: up to ~192K elements most trips of the hit loop have work
    const bool stage = len <= 196608;
    const uint32_t wcnt = stage ? filter_shard<NT, U, true>(sh, edge, seg, seg_cap, ctrl, spill, spill_cap, kmax, round0)
                                : filter_shard<NT, U, false>(sh, edge, seg, seg_cap, ctrl, spill, spill_cap, kmax, round0);
    FFTOPK_MARK(8);
    if (after_arrive && C > 1) cluster.barrier_wait();  // every CTA's counters are cleared (see the prologue)
    const uint32_t wown = min(wcnt, seg_cap);
    fin_wn = (int)wown;
    kmax = __reduce_max_sync(kFull, kmax);
    if (lane == 0) {
      ctrl->wtot[warp] = wown;
      ctrl->wmax[warp] = kmax;
    }
    __syncthreads();
    FFTOPK_MARK(44);
    // hand the candidates to rank 0: one remote atomic per CTA allocates the range
    if (warp == 0) {
      const uint32_t wmine = lane < NW ? ctrl->wtot[lane] : 0u;
      uint32_t incl = wmine;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const uint32_t v = __shfl_up_sync(kFull, incl, off);
        if (lane >= off) incl += v;
      }
      const uint32_t cmax = max(__reduce_max_sync(kFull, lane < NW ? ctrl->wmax[lane] : 0u), ctrl->spill_kmax);
      uint32_t base = 0;
      if (lane == 31) {
        const uint32_t spill_n = min(ctrl->lcount, spill_cap);
        base = atomicAdd(&cx.ctrl0->cand_count, incl + spill_n);
        atomicMax(&cx.ctrl0->max_key, cmax);
        if (ctrl->pub_flag) atomicOr(&cx.ctrl0->over_flag, 1u);
        ctrl->base_c = base + incl;  // where the spill entries go
      }
      base = __shfl_sync(kFull, base, 31);
      if (lane < NW) ctrl->wtot[lane] = base + incl - wmine;
    }
    __syncthreads();
    FFTOPK_MARK(45);
    fin_sn = (int)min(ctrl->lcount, spill_cap);
    if (fin_hist) {  // the entries that went to the spill area
      const uint32_t* sp32 = reinterpret_cast<const uint32_t*>(spill) + 1;
      const FinishDigit dg = make_finish_digit(low_end(fin_lo), high_end(fin_focus));
      for (int j = tid; j < fin_sn; j += NT) red_shared_add(&fh[dg.of_key(sp32[2 * j])], 1u);
    }
    if (C > 1) {
      const uint32_t dst = ctrl->wtot[warp];
      for (uint32_t j = lane; j < wown; j += 32) {
        if (dst + j < (uint32_t)p.cand_cap) cx.cand0[dst + j] = seg[j];
      }
      const uint32_t sbase = ctrl->base_c;
      for (uint32_t j = tid; j < (uint32_t)fin_sn; j += NT) {
        if (sbase + j < (uint32_t)p.cand_cap) cx.cand0[sbase + j] = spill[j];
      }
    }
    FFTOPK_MARK(46);
    cluster_sync(cluster, C);  // #2: every candidate has landed in rank 0
    FFTOPK_MARK(9);
    {
      // every thread reads rank 0's totals itself (no broadcast barrier; for rank 0, whose finish
      // is the critical path, these are local reads)
      const Ctrl* c0 = rank == 0 ? ctrl : cx.ctrl0;
      const uint32_t total = c0->cand_count;
      const uint32_t over = c0->over_flag;
      const uint32_t maxkey = c0->max_key;
      // fewer than k admitted (the guess was too high), a list overflowed, or more than rank 0
      // can hold: start over with full histograms
      const uint32_t room = C == 1 ? 0xffffffffu : (uint32_t)p.cand_cap;  // (a lone CTA keeps them in the list)
      mode = sampled_attempt_ok(over, total, K, room) ? kModeGather : kModeFallback;
      // every candidate's key lies in [lowkey, maxkey]
      fin_cap = maxkey;
      if (fin_hist) {
        if (fin_cap < fin_focus) fin_cap = fin_focus;  // (a looser bound keeps the digit rule of the histogram)
      } else {
        fin_focus = fin_cap;
      }
    }
    need = K;
    P = 0;
    r = -1;  // finish first, final barrier afterwards
    FFTOPK_MARK(10);
  };

  if (p.force_slow) {
    mode = kModeFallback;
  } else if (warm) {
    filter_gather(warm_key, -1, 12, true);
    FFTOPK_MARK(4);
    // (a miss is worth knowing about: the row is then selected by the full-histogram path)
    if (mode == kModeFallback && rank == 0 && tid == 0 && p.status) atomicOr(p.status, (uint32_t)FFTOPK_ST_GUESS_MISSED);
  } else if (exact) {
    // ---- the sample is the row: its histogram gives the threshold bin directly -----------------
    cluster_pick<NT>(
        cluster, C, cx.hist(0), cx.sup(0), cx.xch, ctrl, pick_no, kMaxBins, [&](uint32_t) { return K; },
        [&](Picked& pk) { decide_and_allocate(cx, pk, kModeFallback, false); });
    mode = ctrl->mode;
    FFTOPK_MARK(4);
    if (mode == kModeGather || mode == kModeTakeAll) {
      const uint32_t t = (uint32_t)ctrl->t;
      const uint32_t base_w = ctrl->base_w, base_c = ctrl->base_c;
      const bool take_eq = (mode == kModeTakeAll);
      need = ctrl->above;
      P = t;
#pragma unroll
      for (int j = 0; j < kRegSlabs; ++j) {
        const int i0 = 4 * gr[j] - sh.a;
        const float xv[4] = {xr[j].x, xr[j].y, xr[j].z, xr[j].w};
        if (gr[j] < sh.g1) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if ((unsigned)(i0 + e) < (unsigned)len) {
              const uint32_t key = fftopk_key_from_bits(__float_as_uint(xv[e]));
              const uint32_t bin = key >> 20;
              if (bin > t || (take_eq && bin == t)) {
                emit_winner(cx, base_w, key, i0 + e);
              } else if (bin == t) {
                const uint32_t slot = base_c + warp_alloc(&ctrl->cslot);
                if (FFTOPK_CHECK(2, slot, p.cand_cap, p.status) && slot < (uint32_t)p.cand_cap)
                  cx.cand0[slot] = ((uint64_t)key << 32) | (uint64_t)(~(uint32_t)(i0 + e));
              }
            }
          }
        }
      }
    }
  } else {
    // ---- sampled: pick a conservative lower bound from the sample, filter the shard once ------
    // need_of: sample rank whose true rank is >= k with overwhelming probability
    // (m expected sample elements among the true top k, plus five standard deviations).
    const float flen = (float)len;
    const DualPick dp = cluster_pick_dual<NT>(cluster, C, cx.hist(0), cx.sup(0), cx.hist(1), cx.sup(1), dual, ctrl, pick_no,
                                              [&](uint32_t n_s) { return sample_lower_rank(K, n_s, flen); },
                                              [&](uint32_t n_s) { return sample_upper_rank(K, n_s, flen); });
    FFTOPK_MARK(4);
    // If the sample says the guessed bin alone holds more than ~2k row elements (values crowded
    // into a sliver of the key space), a second sample round on the next 12 key bits sharpens it.
    // (Below that, carrying the extra candidates is cheaper than the round: measured 1.0-1.5 us
    // per call on N(0,1) rows of 384K..2M elements.)
#ifndef FFTOPK_1B_FACTOR
#define FFTOPK_1B_FACTOR 2.0f
#endif
    int smode = !dp.ok ? kModeFallback
                       : (sample_bin_too_coarse(dp.cnt, dp.total, flen, K, FFTOPK_1B_FACTOR) ? kModeNext : kModeGather);
    uint32_t gkey = guess_key(dp.prefix, dp.pbits);
    if (smode == kModeNext) {
      const int sb = 32 - dp.pbits - 12;  // position of the next 12 bits
      const uint32_t rem = dp.need2;
      // Peers may still be reading, from this CTA, the histogram the guess was made on and both
      // super-bin arrays; the other histogram buffer and the third super-bin array are free.
      uint32_t* h1 = cx.hist(dp.pbits == 16 ? 0 : 1);
      uint32_t* s1 = cx.sup(2);
      {
        uint4* h4 = reinterpret_cast<uint4*>(h1);
        for (int i = tid; i < kMaxBins / 4; i += NT) h4[i] = make_uint4(0u, 0u, 0u, 0u);
      }
      __syncthreads();
#pragma unroll
      for (int j = 0; j < kRegSlabs; ++j) {
        if (j < ns && gr[j] < sh.g1) {
          const int e0 = 4 * gr[j] - sh.a;
          const float xv[4] = {xr[j].x, xr[j].y, xr[j].z, xr[j].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t key = fftopk_key_from_bits(__float_as_uint(xv[e]));
            hist_add(h1, (key >> sb) & 0xfffu,
                     (unsigned)(e0 + e) < (unsigned)len && (key >> (32 - dp.pbits)) == dp.prefix);
          }
        }
      }
      __syncthreads();
      compute_sup<NT>(h1, s1, kMaxBins);
      cluster_sync(cluster, C);  // #1b
      cluster_pick<NT>(
          cluster, C, h1, s1, cx.xch, ctrl, pick_no, kMaxBins, [&](uint32_t) { return rem; },
          [&](Picked& pk) {
            if (lane == 0) {
              ctrl->mode = pk.ok ? kModeGather : kModeFallback;
              ctrl->t = pk.t;
            }
          });
      smode = ctrl->mode;
      gkey |= (uint32_t)ctrl->t << sb;
      FFTOPK_MARK(11);
    }
    if (smode == kModeGather) {
      filter_gather(gkey, dp.focus_bin, dp.pbits, false);
    } else {
      mode = kModeFallback;
    }
  }

  if (mode == kModeFallback) mode = refine_from_data<NT, T>(cx, need, P, r, pick_no);

  // Candidates that peers pushed into rank 0 are complete after a cluster barrier. The sampled
  // path has had that barrier already (#2) and only needs one more so that rank 0 outlives the
  // peers' reads of its counters: it goes after the finish, off the critical path. Every other
  // path pushes right up to here, so the barrier comes first.
  const bool finish_first = (r < 0);  // uniform over the cluster
  FFTOPK_MARK(5);
  if (!finish_first) cluster_sync(cluster, C);
  FFTOPK_MARK(6);
  if (mode == kModeGather && rank == 0) {
    const int idx_bits = 32 - __clz(len - 1);
    if (r < 0 && C == 1) {
      // sampled path of a lone CTA: the warps' segments where the filter left them
      const uint32_t spill_cap1 = (uint32_t)p.list_cap / 8u;
      const uint32_t seg_cap1 = ((uint32_t)p.list_cap - spill_cap1) / NW;
      const WarpSegCands<NT> src{list + (size_t)warp * seg_cap1, fin_wn, list + (size_t)NW * seg_cap1, fin_sn};
      cta_finish<NT, WarpSegCands<NT>, kWarm>(src, need, low_end(fin_lo), high_end(fin_cap), high_end(fin_focus), fin_hist,
                                              idx_bits, cx.hist(0), ctrl, out_idx, out_key, K - need, K, cx.idx_offset,
                                              p.status, cx.page, ctrl->cand_count);
    } else {
      // every candidate shares the key prefix P above bit `sh` of the key (sampled path: range known)
      const int sh = r < 0 ? 0 : round_shift(r);
      const uint64_t lo = r < 0 ? low_end(fin_lo) : ((uint64_t)P << (32 + sh));
      const uint64_t cap = r < 0 ? high_end(fin_cap) : (lo | ((1ull << (32 + sh)) - 1ull));
      const DenseCands<NT> src{cx.cand, (int)min(ctrl->cand_count, (uint32_t)p.cand_cap)};
      cta_finish<NT, DenseCands<NT>, kWarm>(src, need, lo, cap, cap, false, idx_bits, cx.hist(0), ctrl, out_idx, out_key,
                                            K - need, K, cx.idx_offset, p.status, cx.page, (uint32_t)src.n);
    }
  }
  if constexpr (kWarm) {
    // This call's threshold for the next one: the smallest key the finish let win (the row's k-th
    // largest key), or, where no finish ran, the lower edge of the bin the threshold was found in
    // (a lower bound: the next call then admits a few more candidates and tightens it again).
    if (rank == 0 && p.next_threshold != nullptr) {
      __syncthreads();
      if (tid == 0) {
        uint32_t thr = 0u;
        if (mode == kModeGather) {
          thr = ctrl->thr_key != 0xffffffffu ? ctrl->thr_key : 0u;
        } else if ((mode == kModeTakeAll || mode == kModeTies) && r >= 0) {
          thr = P << round_shift(r);
        }
        p.next_threshold[row] = thr;
      }
    }
  }
  FFTOPK_MARK(34);
  if (finish_first) cluster_sync(cluster, C);
  FFTOPK_MARK(7);
  if (tid == 0 && p.status && mode == kModeAbort) atomicOr(p.status, (uint32_t)FFTOPK_ST_INTERNAL);
}

template <int NT, bool kAnyK = false, bool kWarm = false, class T = float>
__global__ void __launch_bounds__(NT, (NT == 512 ? FFTOPK_CTAS_512 : 1024 / NT)) select2048_kernel(const SelectParams p) {
  select_row<NT, kAnyK, kWarm, T>(p);
  if (p.cp_publish) {
    // Context-parallel publication folded into the selection: the CTA's barrier orders every
    // thread's output writes before thread 0's arrival, a release at device scope (one operation
    // by the arriving thread, as in a grid-wide barrier, instead of a fence per thread); the last
    // CTA of the grid, which has acquired all the others' arrivals, releases the epoch flag
    // system-wide (peers acquire it in their merge kernel). The counter goes back to zero for the
    // next launch, which stream order keeps behind this one.
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t* arrive = p.cp_publish + kCommArriveWord;
      uint32_t old;
      asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(arrive) : "memory");
      if (old == gridDim.x - 1u) {
        *arrive = 0u;
        const uint32_t epoch = p.cp_epoch ? p.cp_epoch : __ldcg(p.cp_publish) + 1u;
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.cp_publish), "r"(epoch) : "memory");
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Context-parallel top-2048 in ONE launch per GPU: local selection, exchange and merge. Every GPU
// holds a contiguous slice of each row. The row's cluster first selects the local top 2048 of its
// slice (keys and global indices) exactly as select2048_kernel does; its first CTA then PUSHES the
// 2048 candidates as self-validating packets {index, epoch, key, epoch} into the inbox of every
// GPU, its own included, with plain 16-byte stores over NVLink - no flag, no fence (a system-scope
// fence was measured at 4.5 us per publication), no round trip. After that CTA g of the cluster
// (g < G) polls, in its own GPU's memory and with a time limit, the packets shard g sent for the
// row, and the cluster merges the G lists (merge_row). No second launch, no collective call, no
// launch-wide synchronisation: a row is merged as soon as its own G slices have been selected.
// The inbox has two halves that alternate by epoch parity: a GPU can only start call e+2 after
// its own call e+1 has seen every peer's packets of e+1, which the peer sent after it had finished
// call e and with it every read of its inbox half e.
// ---------------------------------------------------------------------------------------------
struct CpFused {
  uint4* inbox[kMaxShards];   // inbox (half 0, source shard 0, row 0) of every GPU, own included
  uint32_t* row_epoch;        // this GPU's epoch counter of row 0; row r's is kCommRowFlagWords * r further
  int64_t inbox_half_packets; // packets between the two halves of an inbox
  unsigned long long wait_ns;
  int32_t* out_idx;           // [B, 2048] merged result
  uint32_t epoch;             // epoch of this call, or 0: each row counter's value plus one
  int32_t G, own, b_cap;
};

template <int NT>
__global__ void __launch_bounds__(NT, (NT == 512 ? FFTOPK_CTAS_512 : 1024 / NT)) select_merge2048_kernel(const SelectParams p,
                                                                                                      const CpFused f) {
  cg::cluster_group cluster = cg::this_cluster();
  const int C = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int row = (int)(blockIdx.x / (unsigned)C);
  const int tid = threadIdx.x;
  uint32_t* my_epoch = f.row_epoch + (int64_t)row * kCommRowFlagWords;
  // launched as a programmatic dependent, like the selection kernel (see select_row): the call in
  // front of this one has to have completed before the row's epoch counter is read
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // (the previous call's update of the counter is complete - stream order - and this call's comes
  // at the very end: every CTA of the cluster reads the same value)
  const uint32_t epoch = f.epoch ? f.epoch : __ldcg(my_epoch) + 1u;
  select_row<NT, false>(p);
  // Every output of the row is written: by this CTA, or by its peers before a cluster barrier
  // this CTA has passed.
  FFTOPK_MARK(60);
  // packets of (half, source shard, row): ((half * 8 + shard) * b_cap + row) * 2048
  const int64_t half_off = (int64_t)(epoch & 1u) * f.inbox_half_packets;
  if (rank == 0) {
    __syncthreads();
    constexpr int PER = kK / NT;
    const int32_t* lidx = p.out_idx + (int64_t)row * kK;
    const uint32_t* lkey = p.out_key + (int64_t)row * kK;
    const int64_t dst_off = half_off + ((int64_t)f.own * f.b_cap + row) * kK;
    int32_t ci[PER];
    uint32_t ck[PER];
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      ci[u] = __ldcg(lidx + u * NT + tid);
      ck[u] = __ldcg(lkey + u * NT + tid);
    }
    for (int d = 0; d < f.G; ++d) {
      uint4* dst = f.inbox[d] + dst_off;
#pragma unroll
      for (int u = 0; u < PER; ++u) st_packet(dst + u * NT + tid, ci[u], ck[u], epoch);
    }
  }
  FFTOPK_MARK(61);
  // ---- merge: same carve of the dynamic shared memory as the selection --------------------------
  extern __shared__ __align__(128) unsigned char smem_raw[];
  MergeSmem sm;
  sm.hist = reinterpret_cast<uint32_t*>(smem_raw);
  sm.sup = sm.hist + 2 * kMaxBins;
  sm.xch = sm.sup + 3 * kSup;
  sm.ctrl = reinterpret_cast<Ctrl*>(sm.xch + kMaxCluster * kSup);
  sm.cand = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(sm.ctrl) + ((sizeof(Ctrl) + 127) & ~127u));
  sm.cand_cap = C == 1 ? p.list_cap : p.list_cap + p.cand_cap;
  const uint4* mine = rank < f.G ? f.inbox[f.own] + half_off + ((int64_t)rank * f.b_cap + row) * kK : nullptr;
  merge_row<NT>(cluster, C, f.G, rank, sm, nullptr, nullptr, nullptr, mine, epoch, f.wait_ns,
                f.out_idx + (int64_t)row * kK, nullptr, p.status);
  // the row's epoch counter moves on only now: every CTA of the cluster read it before the first
  // cluster barrier of the merge
  if (rank == 0 && tid == 0 && f.epoch == 0u) *my_epoch = epoch;
  FFTOPK_MARK(69);
}

}  // namespace fftopk

// =============================================================================================
// Host side: launch plan and C ABI
// =============================================================================================
namespace {

using namespace fftopk;

// Process-wide overrides (fftopk_set_tuning, fftopk_set_overlap). Writers and readers go through
// the mutex; every launch works on its own snapshot.
struct Tuning {
  int cluster = -1, threads = -1, list_cap = -1, cand_cap = -1, force_slow = 0, overlap = 0;
};
std::mutex g_tuning_mu;
Tuning g_tuning;

Tuning tuning_snapshot() {
  std::lock_guard<std::mutex> lock(g_tuning_mu);
  return g_tuning;
}

struct DeviceInfo {
  DeviceOnce once;
  int sm_count = 0;
  int smem_optin = 0;
  int cc_major = 0;
  int max_cluster = 0;  // largest cluster size that can be scheduled with the latency-mode footprint
  int active16 = 0, active8 = 0;  // clusters of that size the device holds at once (same footprint)
};
DeviceInfo g_dev[kMaxDevices];

constexpr size_t fixed_smem_bytes() {
  return (size_t)(2 * kMaxBins + 3 * kSup + kMaxCluster * kSup) * 4 + ((sizeof(Ctrl) + 127) & ~(size_t)127);
}

constexpr int kLatencyListCap = 6144, kLatencyCandCap = 16384;  // one CTA per SM: use the shared memory
constexpr int kBatchListCap = 4096, kBatchCandCap = 4096;       // several CTAs per SM
// One CTA per row (list = candidates), two CTAs per SM. Rows of up to ~192K elements leave about
// 3600 candidates; with the small list two CTAs take 2 x 90 KB of the SM's 256 KB and the rest
// stays L1, which the value re-reads of the filter hit (measured on B=64 ragged rows <= 128K:
// 5.3 us per call with lists of 4608..7168 entries, 6.2 us with 8192 or more).
constexpr int kOverlapListCap1 = 6144, kOverlapListCap1Long = 9216;
constexpr int64_t kOverlapShortRow = 196608;
constexpr int kOverlapListCap = 3072, kOverlapCandCap = 6144;   // two CTAs per SM


template <int NT>
int setup_kernel(int smem_optin) {
  cudaError_t e = cudaFuncSetAttribute(select2048_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin);
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaFuncSetAttribute(select2048_kernel<NT>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaFuncSetAttribute(select2048_kernel<NT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin);
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaFuncSetAttribute(select2048_kernel<NT, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
  if (e != cudaSuccess) return cuda_fail(e);
  if constexpr (NT >= 512) {
    e = cudaFuncSetAttribute(select2048_kernel<NT, true, false, __half>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin);
    if (e != cudaSuccess) return cuda_fail(e);
    e = cudaFuncSetAttribute(select2048_kernel<NT, true, false, __half>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return cuda_fail(e);
    e = cudaFuncSetAttribute(select2048_kernel<NT, true, false, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             smem_optin);
    if (e != cudaSuccess) return cuda_fail(e);
    e = cudaFuncSetAttribute(select2048_kernel<NT, true, false, __nv_bfloat16>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return cuda_fail(e);
    e = cudaFuncSetAttribute(select2048_kernel<NT, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin);
    if (e != cudaSuccess) return cuda_fail(e);
    e = cudaFuncSetAttribute(select2048_kernel<NT, false, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return cuda_fail(e);
    e = cudaFuncSetAttribute(select_merge2048_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin);
    if (e != cudaSuccess) return cuda_fail(e);
    e = cudaFuncSetAttribute(select_merge2048_kernel<NT>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  return 0;
}

int init_device(DeviceInfo& d, int dev) {
  cudaDeviceProp prop;
  cudaError_t e = cudaGetDeviceProperties(&prop, dev);
  if (e != cudaSuccess) return cuda_fail(e);
  d.sm_count = prop.multiProcessorCount;
  d.smem_optin = (int)prop.sharedMemPerBlockOptin;
  d.cc_major = prop.major;
  if (prop.major < 10) return FFTOPK_EDEVICE;
  int rc = setup_kernel<1024>(d.smem_optin);
  if (rc) return rc;
  rc = setup_kernel<512>(d.smem_optin);
  if (rc) return rc;
  rc = setup_kernel<256>(d.smem_optin);
  if (rc) return rc;
  // can a 16-CTA cluster with the latency-mode shared-memory footprint be co-scheduled, and how
  // many clusters of 16 / of 8 CTAs does the device hold at once? (A cluster lives inside one
  // GPC, so fewer 16-CTA clusters fit than SM count / 16: a batch with more rows than that would
  // run in two waves.)
  d.max_cluster = 8;
  d.active16 = 0;
  d.active8 = d.sm_count / 8;
  for (int cs = 16; cs >= 8; cs /= 2) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cs * 32, 1, 1);
    cfg.blockDim = dim3(1024, 1, 1);
    cfg.dynamicSmemBytes = fixed_smem_bytes() + (size_t)(kLatencyListCap + kLatencyCandCap) * 8;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = cs;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    int nclusters = 0;
    e = cudaOccupancyMaxActiveClusters(&nclusters, select2048_kernel<1024>, &cfg);
    if (e == cudaSuccess && nclusters >= 1) {
      if (cs == 16) {
        d.max_cluster = 16;
        d.active16 = nclusters;
      } else {
        d.active8 = nclusters;
      }
    }
    (void)cudaGetLastError();
  }
  return 0;
}

// Properties of the current device; the first call on a device (any thread) sets the kernels'
// function attributes.
int device_info(DeviceInfo** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= kMaxDevices) return FFTOPK_EDEVICE;
  DeviceInfo& d = g_dev[dev];
  const int rc = d.once.run([&] { return init_device(d, dev); });
  if (rc) return rc;
  *out = &d;
  return 0;
}

struct Plan {
  int cluster, threads, smem_bytes, list_cap, cand_cap;
};

int floor_pow2(int64_t v) {
  int r = 1;
  while ((int64_t)r * 2 <= v) r *= 2;
  return r;
}

// Replaces the reference's split heuristic (topk_indexer_radix.cu:1081-1111: at most 8 CTAs per
// row, a hard-coded SM count of 132). `overlap`: the launch may overlap its neighbours on the
// stream (throughput plan).
Plan make_plan(const DeviceInfo& d, const Tuning& tn, bool overlap, int B, int64_t L) {
  Plan pl;
  const int rows = B > 0 ? B : 1;
  // CTAs per row: as many as keep the whole grid resident at once with one CTA per SM, but never
  // so many that a shard drops below ~2K elements.
  int c = floor_pow2(d.sm_count / rows > 0 ? d.sm_count / rows : 1);
  if (c > d.max_cluster) c = d.max_cluster;
  if (c == 16 && rows > d.active16) c = 8;  // all rows in one wave
  if (c == 8 && rows > d.active8) c = 4;
  const int by_len = floor_pow2(L / 2048 > 0 ? L / 2048 : 1);
  if (c > by_len) c = by_len;
  pl.cluster = c < 1 ? 1 : c;
  // Short rows spread over many CTAs leave a thread one or two granules: 512 threads do the same
  // with cheaper block barriers (measured at B=1 and B=4: 10.2-11.0 us against 11.4-12.3 us for
  // L = 16K and 32K; from 64K on 1024 threads win).
  pl.threads = (L <= 32768 && pl.cluster >= 8) ? 512 : 1024;
  const bool one_per_sm = (int64_t)rows * pl.cluster <= d.sm_count;
  pl.list_cap = one_per_sm ? kLatencyListCap : kBatchListCap;
  pl.cand_cap = one_per_sm ? kLatencyCandCap : kBatchCandCap;
  if (rows > d.sm_count) {
    // More rows than SMs: the batch fills the device by itself. One 512-thread CTA per row with
    // the list of the throughput plan, two CTAs per SM (measured on ragged rows of up to 128K
    // elements: 29.7 us per call at B=256 and 52.6 us at B=512, against 38.5 / 68.1 us with 1024
    // threads; a list of 4096 entries split over 32 warps overflowed its segments and sent rows
    // to the full-histogram path: 78 / 113 us).
    pl.cluster = 1;
    pl.threads = 512;
    pl.list_cap = L <= kOverlapShortRow ? kOverlapListCap1 : kOverlapListCap1Long;
  }
  if (overlap) {
    // Back-to-back calls may overlap: what counts is work per row, not the latency of one call.
    // Few CTAs per row (less cluster traffic per row), 512 threads and about 110 KB of shared
    // memory so that two CTAs - of different calls - share an SM, and about four calls in flight.
    int ct = floor_pow2(d.sm_count / (4 * rows) > 0 ? d.sm_count / (4 * rows) : 1);
    if (ct < pl.cluster) pl.cluster = ct;
    pl.threads = 512;
    if (pl.cluster == 1) {
      pl.list_cap = L <= kOverlapShortRow ? kOverlapListCap1 : kOverlapListCap1Long;
    } else {
      pl.list_cap = kOverlapListCap;
      pl.cand_cap = kOverlapCandCap;
    }
  }
  if (tn.cluster > 0) pl.cluster = tn.cluster;
  if (tn.threads > 0) pl.threads = tn.threads;
  if (tn.list_cap > 0) pl.list_cap = (tn.list_cap + 15) & ~15;
  if (tn.cand_cap > 0) pl.cand_cap = (tn.cand_cap + 15) & ~15;
  if (pl.cluster == 1) pl.cand_cap = pl.list_cap;  // one CTA per row: the two buffers are the same memory
  pl.smem_bytes = (int)(fixed_smem_bytes() + (size_t)(pl.cluster == 1 ? pl.list_cap : pl.list_cap + pl.cand_cap) * 8);
  return pl;
}

SelectCall basic_call(const float* score, int64_t row_stride, int32_t B, int64_t L, const int32_t* lengths,
                      const int32_t* row_starts, int32_t* out_idx, uint32_t* out_key, int32_t idx_offset,
                      uint32_t* status, void* cuda_stream) {
  SelectCall c;
  c.score = score;
  c.row_stride = row_stride;
  c.B = B;
  c.L = L;
  c.lengths = lengths;
  c.row_starts = row_starts;
  c.out_idx = out_idx;
  c.out_key = out_key;
  c.idx_offset = idx_offset;
  c.status = status;
  c.cuda_stream = cuda_stream;
  return c;
}

}  // namespace

namespace fftopk {

int launch_select(const SelectCall& c) {
  if (c.B < 0 || c.L < 0 || c.row_stride < 0 || c.k < 1 || c.k > kMaxK) return FFTOPK_EINVAL;
  if (c.B == 0) return FFTOPK_OK;
  if (!c.score || !c.lengths || !c.out_idx) return FFTOPK_EINVAL;
  const bool half_width = c.dtype != kDtypeF32;
  if ((reinterpret_cast<uintptr_t>(c.score) & (half_width ? 1u : 3u)) != 0) return FFTOPK_EINVAL;
  if (c.L > (int64_t)0x7fffffff - 8 || (int64_t)c.B * kMaxCluster > (int64_t)0x7fffffff) return FFTOPK_ERANGE;
  DeviceInfo* d = nullptr;
  int rc = device_info(&d);
  if (rc) return rc;
  const Tuning tn = tuning_snapshot();
  const bool overlap = tn.overlap != 0 && c.may_overlap;
  Plan pl = make_plan(*d, tn, overlap, c.B, c.L);
  if (half_width && pl.threads < 512) pl.threads = 512;  // (the 16-bit kernels exist for 512 and 1024 threads)
  if (c.k > kK && pl.cluster == 1 && tn.list_cap <= 0) {
    // more winners than the lone-CTA list was sized for: the long-row list
    pl.list_cap = pl.cand_cap = kOverlapListCap1Long;
    pl.smem_bytes = (int)(fixed_smem_bytes() + (size_t)pl.list_cap * 8);
  }

  SelectParams p;
  p.score = c.score;
  p.row_stride = c.row_stride;
  p.L = c.L;
  p.lengths = c.lengths;
  p.row_starts = c.row_starts;
  p.out_idx = c.out_idx;
  p.out_key = c.out_key;
  p.status = c.status;
  p.B = c.B;
  p.k = c.k;
  p.idx_offset = c.idx_offset;
  p.list_cap = pl.list_cap;
  p.cand_cap = pl.cand_cap;
  p.force_slow = tn.force_slow;
  p.overlap = overlap ? 1 : 0;
  p.src_page_table = c.src_page_table;
  p.src_stride = c.src_stride;
  p.cu_seqlens_q = c.cu_seqlens_q;
  p.prefill_bs = c.prefill_bs;
  p.row_offsets = c.row_offsets;
  p.cp_flag = c.cp_flag;
  p.cp_half_words = c.cp_half_words;
  p.cp_publish = c.cp_publish;
  p.cp_epoch = c.cp_epoch;
  p.prev_threshold = c.prev_threshold;
  p.next_threshold = c.next_threshold;
  p.warm_margin = c.warm_margin;
  p.only_rows = c.only_rows;
  const bool warm = c.prev_threshold != nullptr || c.next_threshold != nullptr;
  if (warm && (c.k != kK || pl.threads < 512)) return FFTOPK_EINVAL;
  if ((size_t)pl.smem_bytes > (size_t)d->smem_optin) return FFTOPK_ERANGE;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)c.B * (unsigned)pl.cluster, 1, 1);
  cfg.blockDim = dim3((unsigned)pl.threads, 1, 1);
  cfg.dynamicSmemBytes = (size_t)pl.smem_bytes;
  cfg.stream = static_cast<cudaStream_t>(c.cuda_stream);
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = (unsigned)pl.cluster;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  // (every launch: see the top of select_row for what the kernel does with it)
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.numAttrs = 2;
  cudaError_t e;
  const bool any_k = c.k != kK;
  if (half_width) {
    if (warm || c.src_page_table || c.cp_flag || c.cp_publish) return FFTOPK_EINVAL;
    if (c.dtype == kDtypeF16) {
      e = pl.threads == 1024 ? cudaLaunchKernelEx(&cfg, select2048_kernel<1024, true, false, __half>, p)
                             : cudaLaunchKernelEx(&cfg, select2048_kernel<512, true, false, __half>, p);
    } else {
      e = pl.threads == 1024 ? cudaLaunchKernelEx(&cfg, select2048_kernel<1024, true, false, __nv_bfloat16>, p)
                             : cudaLaunchKernelEx(&cfg, select2048_kernel<512, true, false, __nv_bfloat16>, p);
    }
  } else if (warm) {
    e = pl.threads == 1024 ? cudaLaunchKernelEx(&cfg, select2048_kernel<1024, false, true>, p)
                           : cudaLaunchKernelEx(&cfg, select2048_kernel<512, false, true>, p);
  } else if (pl.threads == 1024) {
    e = any_k ? cudaLaunchKernelEx(&cfg, select2048_kernel<1024, true>, p) : cudaLaunchKernelEx(&cfg, select2048_kernel<1024>, p);
  } else if (pl.threads == 512) {
    e = any_k ? cudaLaunchKernelEx(&cfg, select2048_kernel<512, true>, p) : cudaLaunchKernelEx(&cfg, select2048_kernel<512>, p);
  } else {
    e = any_k ? cudaLaunchKernelEx(&cfg, select2048_kernel<256, true>, p) : cudaLaunchKernelEx(&cfg, select2048_kernel<256>, p);
  }
  if (e != cudaSuccess) return cuda_fail(e);
  return FFTOPK_OK;
}

// Single-launch context-parallel call (see select_merge2048_kernel). FFTOPK_ERANGE when the
// launch plan for (B, L) gives a row fewer CTAs than there are shards or too little shared memory
// for the merge: the caller then uses the two-launch sequence.
int launch_select_merge(const SelectCall& c, void* const* comms, int32_t G, int32_t own, int32_t b_cap, uint32_t epoch,
                        int32_t wait_ms, int32_t* out_idx) {
  if (c.B < 0 || c.L < 0 || c.row_stride < 0) return FFTOPK_EINVAL;
  if (!comms || G < 1 || own < 0 || own >= G || b_cap < 1 || c.B > b_cap || wait_ms < 0) return FFTOPK_EINVAL;
  if (G > kMaxShards) return FFTOPK_ERANGE;
  if (c.B == 0) return FFTOPK_OK;
  if (!c.score || !c.lengths || !out_idx) return FFTOPK_EINVAL;
  if ((reinterpret_cast<uintptr_t>(c.score) & 3u) != 0) return FFTOPK_EINVAL;
  if (c.L > (int64_t)0x7fffffff - 8) return FFTOPK_ERANGE;
  DeviceInfo* d = nullptr;
  int rc = device_info(&d);
  if (rc) return rc;
  const Tuning tn = tuning_snapshot();
  const Plan pl = make_plan(*d, tn, false, c.B, c.L);
  const int room = pl.cluster == 1 ? pl.list_cap : pl.list_cap + pl.cand_cap;
  if (pl.cluster < G || room < G * kK || pl.threads < 512 || (size_t)pl.smem_bytes > (size_t)d->smem_optin) return FFTOPK_ERANGE;

  SelectParams p;
  memset(&p, 0, sizeof(p));
  CpFused f;
  memset(&f, 0, sizeof(f));
  for (int g = 0; g < G; ++g) {
    if (!comms[g]) return FFTOPK_EINVAL;
    f.inbox[g] = reinterpret_cast<uint4*>(static_cast<int32_t*>(comms[g]) + comm_inbox_offset(b_cap));
  }
  int32_t* own_words = static_cast<int32_t*>(comms[own]);
  f.row_epoch = reinterpret_cast<uint32_t*>(own_words + comm_rowflag_offset(b_cap));
  f.inbox_half_packets = (int64_t)(comm_inbox_half_words(b_cap) / 4);
  f.wait_ns = (unsigned long long)wait_ms * 1000000ull;
  f.out_idx = out_idx;
  f.epoch = epoch;
  f.G = G;
  f.own = own;
  f.b_cap = b_cap;
  p.score = c.score;
  p.row_stride = c.row_stride;
  p.L = c.L;
  p.lengths = c.lengths;
  p.out_idx = own_words + comm_stage_offset(b_cap);  // local selection output, pushed from there
  p.out_key = reinterpret_cast<uint32_t*>(p.out_idx + (size_t)b_cap * kK);
  p.status = c.status;
  p.B = c.B;
  p.k = kK;
  p.idx_offset = c.idx_offset;
  p.list_cap = pl.list_cap;
  p.cand_cap = pl.cand_cap;
  p.force_slow = tn.force_slow;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)c.B * (unsigned)pl.cluster, 1, 1);
  cfg.blockDim = dim3((unsigned)pl.threads, 1, 1);
  cfg.dynamicSmemBytes = (size_t)pl.smem_bytes;
  cfg.stream = static_cast<cudaStream_t>(c.cuda_stream);
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = (unsigned)pl.cluster;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 2;
  const cudaError_t e = pl.threads == 1024 ? cudaLaunchKernelEx(&cfg, select_merge2048_kernel<1024>, p, f)
                                           : cudaLaunchKernelEx(&cfg, select_merge2048_kernel<512>, p, f);
  if (e != cudaSuccess) return cuda_fail(e);
  return FFTOPK_OK;
}

}  // namespace fftopk

extern "C" {

int fftopk_version(void) { return 200; }

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

int fftopk_last_cuda_error(void) { return fftopk::g_last_cuda_error; }

#ifdef FFTOPK_CHECKED
// Checked builds only: the first violation recorded by the selection kernels (rec[0..3]) and by the
// merge kernel (rec[4..7]) as (site, index, limit, block); site 0 = none. Clears both records.
int fftopk_checked_read(uint32_t rec[8]) {
  const uint32_t zero[4] = {0u, 0u, 0u, 0u};
  cudaError_t e = cudaMemcpyFromSymbol(rec, fftopk::g_check_rec, sizeof(zero));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(fftopk::g_check_rec, zero, sizeof(zero));
  if (e != cudaSuccess) return fftopk::cuda_fail(e);
  return fftopk::checked_read_merge(rec + 4);
}
#endif

#ifdef FFTOPK_TRACE
int fftopk_trace_read(unsigned long long* times, int* ids, int* n) {
  cudaError_t e = cudaMemcpyFromSymbol(n, fftopk::g_trace_n, sizeof(int));
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(times, fftopk::g_trace_t, sizeof(unsigned long long) * fftopk::kTraceCap);
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(ids, fftopk::g_trace_id, sizeof(int) * fftopk::kTraceCap);
  return (int)e;
}
int fftopk_trace_clear(void) {
  const int z = 0;
  return (int)cudaMemcpyToSymbol(fftopk::g_trace_n, &z, sizeof(int));
}
#endif

uint32_t fftopk_key_of(float x) {
  uint32_t bits;
  __builtin_memcpy(&bits, &x, 4);
  return fftopk_key_from_bits(bits);
}

int fftopk_set_tuning(int32_t cluster_ctas, int32_t threads, int32_t list_cap, int32_t cand_cap,
                      int32_t force_full_histogram) {
  if (cluster_ctas > 0 && (cluster_ctas > kMaxCluster || (cluster_ctas & (cluster_ctas - 1)))) return FFTOPK_EINVAL;
  if (threads > 0 && threads != 256 && threads != 512 && threads != 1024) return FFTOPK_EINVAL;
  if (cand_cap > 0 && (cand_cap < 32 || cand_cap > 16384)) return FFTOPK_EINVAL;
  if (list_cap > 0 && (list_cap < 32 || list_cap > 16384)) return FFTOPK_EINVAL;
  std::lock_guard<std::mutex> lock(g_tuning_mu);
  g_tuning.cluster = cluster_ctas;
  g_tuning.threads = threads;
  g_tuning.list_cap = list_cap;
  g_tuning.cand_cap = cand_cap;
  g_tuning.force_slow = force_full_histogram > 0 ? 1 : 0;
  return FFTOPK_OK;
}

int fftopk_set_overlap(int32_t enable) {
  std::lock_guard<std::mutex> lock(g_tuning_mu);
  g_tuning.overlap = enable ? 1 : 0;
  return FFTOPK_OK;
}

int fftopk_plan(int32_t B, int64_t L, int32_t plan[6]) {
  if (!plan || B < 0 || L < 0) return FFTOPK_EINVAL;
  DeviceInfo* d = nullptr;
  int rc = device_info(&d);
  if (rc) return rc;
  const Tuning tn = tuning_snapshot();
  const Plan pl = make_plan(*d, tn, tn.overlap != 0, B, L);
  plan[0] = pl.cluster;
  plan[1] = pl.threads;
  plan[2] = pl.smem_bytes;
  plan[3] = pl.list_cap;
  plan[4] = pl.cand_cap;
  plan[5] = d->sm_count;
  return FFTOPK_OK;
}

int fftopk_select2048(const float* score, int64_t row_stride, int32_t B, int64_t L, const int32_t* lengths,
                      const int32_t* row_starts, int32_t* out_idx, uint32_t* out_key, int32_t idx_offset,
                      uint32_t* status, void* cuda_stream) {
  return launch_select(basic_call(score, row_stride, B, L, lengths, row_starts, out_idx, out_key, idx_offset, status,
                                  cuda_stream));
}

int fftopk_select_topk(const float* score, int64_t row_stride, int32_t B, int64_t L, const int32_t* lengths,
                       const int32_t* row_starts, int32_t k, int32_t* out_idx, uint32_t* out_key, int32_t idx_offset,
                       uint32_t* status, void* cuda_stream) {
  SelectCall c = basic_call(score, row_stride, B, L, lengths, row_starts, out_idx, out_key, idx_offset, status, cuda_stream);
  c.k = k;
  return launch_select(c);
}

int fftopk_select2048_warm(const float* score, int64_t row_stride, int32_t B, int64_t L, const int32_t* lengths,
                           const int32_t* row_starts, const uint32_t* prev_threshold, uint32_t margin,
                           uint32_t* next_threshold, int32_t* out_idx, uint32_t* status, void* cuda_stream) {
  if (B > 0 && !prev_threshold && !next_threshold) return FFTOPK_EINVAL;
  SelectCall c = basic_call(score, row_stride, B, L, lengths, row_starts, out_idx, nullptr, 0, status, cuda_stream);
  c.prev_threshold = prev_threshold;
  c.next_threshold = next_threshold;
  c.warm_margin = margin;
  return launch_select(c);
}

int fftopk_select2048_page_table(const float* score, int64_t row_stride, int32_t B, int64_t L,
                                 const int32_t* lengths, const int32_t* row_starts, int32_t* dst_page_table,
                                 const int32_t* src_page_table, int64_t src_stride, const int32_t* cu_seqlens_q,
                                 int32_t prefill_bs, uint32_t* status, void* cuda_stream) {
  if (B > 0 && (!src_page_table || src_stride < 0 || prefill_bs < 1 || prefill_bs > B)) return FFTOPK_EINVAL;
  SelectCall c = basic_call(score, row_stride, B, L, lengths, row_starts, dst_page_table, nullptr, 0, status, cuda_stream);
  c.src_page_table = src_page_table;
  c.src_stride = src_stride;
  c.cu_seqlens_q = cu_seqlens_q;
  c.prefill_bs = prefill_bs;
  return launch_select(c);
}

int fftopk_select2048_ragged(const float* score, int64_t row_stride, int32_t B, int64_t L, const int32_t* lengths,
                             const int32_t* row_starts, int32_t* topk_indices_ragged,
                             const int32_t* topk_indices_offset, uint32_t* status, void* cuda_stream) {
  if (B > 0 && !topk_indices_offset) return FFTOPK_EINVAL;
  SelectCall c = basic_call(score, row_stride, B, L, lengths, row_starts, topk_indices_ragged, nullptr, 0, status, cuda_stream);
  c.row_offsets = topk_indices_offset;
  return launch_select(c);
}

}  // extern "C"
