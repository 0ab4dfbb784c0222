// Indexer logits fused with the top-2048 selection (sm_100a: TMA + tcgen05 + TMEM).
//
// The logit of key t of a row is  sum over 64 heads h of  w[h] * relu(q[h] . k[t])  (q[h], k[t] of
// dimension 128; bf16, or fp8 e4m3 with an optional scale per key). The reference contains no producer of these logits - its selector starts
// from a finished fp32 [B, L] matrix (jit_kernel/topk_indexer.py:42-75) and its README only names
// the step (README.md:24) - so there is no reference counterpart; this is the step in front of the
// hot path, fused with it.
//
// Producer kernel, one CTA per (row, slice of key tiles), two CTAs per SM, 320 threads in three roles:
//   warp 0      one thread issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle, no multicast):
//               the row's q once (64 heads x 128), then key tiles of 128 keys x 128 through a ring
//               of shared-memory stages guarded by full / empty mbarriers;
//   warp 1      allocates 256 TMEM columns; one thread issues, per tile, eight tcgen05.mma of
//               K=16 (bf16; four of K=32 for fp8), M=128 keys, N=64 heads, that accumulate
//               D[key][head] in fp32 in one of four
//               64-column TMEM buffers, and commits to the stage's empty barrier and the buffer's
//               full barrier;
//   warps 2-9   epilogue, two groups of four warps, one group per TMEM buffer (every second
//               tile): tcgen05.ld hands every thread the 64 head values of ONE key; relu,
//               weights and the sum are in-thread - one logit per thread and tile. With a threshold
//               guess for the row (the previous decode step's, see fftopk_select2048_warm) the
//               logit is compared with the guess's edge and the few that pass are appended, by
//               ballot and one atomic per warp, to the row's candidate list. The logit is also
//               written (4 bytes per key beside the 256 or 132 read), but read again only by a row
//               whose guess fails.
// Every wait on an mbarrier has a time limit; when one runs out the CTA raises
// FFTOPK_ST_STAGE_TIMEOUT, lets its copies in flight land, frees its TMEM and returns.
//
// Finish, inside the producer: the CTAs of a row count themselves off as they run out of tiles, and
// the last one decides. If the row's guess held - at least 2048 candidates, no more than the list
// holds - it pulls the list into the shared memory its stages no longer need and selects the exact
// top 2048 (cta_finish: ties to the lower index) and the new threshold; otherwise it marks the row
// and the selector of fftopk_select.cu runs on the row's logits. That launch follows as a
// programmatic dependent: it is resident, waiting, by the time the producer ends, and rows that are
// not marked cost it an empty CTA. The last CTA also zeroes the row's counters, so a call leaves the
// workspace ready for the next one and a call is two launches, none of them a memset.
#include <cooperative_groups.h>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/fftopk.h"
#include "fftopk_trace.cuh"
#include "fftopk_device.cuh"
#include "fftopk_host.h"
#include "fftopk_internal.h"
#include "fftopk_key.h"

namespace fftopk {

// Build-time knobs (optional, for experiments; the defaults are what was measured best):
//   FFTOPK_IDX_CTAS_PER_SM  producer CTAs per SM (2: two independent TMA -> MMA -> epilogue pipelines
//                           per SM hide each other's per-tile latencies; measured at B=1, L=1M, fp8:
//                           40.0 us per call against 45.1 with one CTA per SM, bf16: 56.2 / 56.6)
//   FFTOPK_IDX_STAGES_FP8   key tiles in flight per CTA for fp8 operands (4 x 16 KiB; 12 stages on
//                           one CTA per SM: 46.7 us, no gain over 8)
#ifndef FFTOPK_IDX_CTAS_PER_SM
#define FFTOPK_IDX_CTAS_PER_SM 2
#endif
#ifndef FFTOPK_IDX_STAGES_FP8
#define FFTOPK_IDX_STAGES_FP8 (8 / FFTOPK_IDX_CTAS_PER_SM)
#endif
constexpr int kIdxHeads = 64;
constexpr int kIdxDim = 128;
constexpr int kIdxTile = 128;      // keys per tile = rows of the MMA
constexpr int kIdxThreads = 320;    // TMA warp, MMA warp, two groups of four epilogue warps
// Operand formats: bf16 (two 128-byte swizzle rows per key, MMA K = 16) or fp8 e4m3 (one row per
// key, MMA K = 32, an optional fp32 scale per key applied in the epilogue).
template <bool kFp8>
struct IdxFmt {
  static constexpr int kElemBytes = kFp8 ? 1 : 2;
  static constexpr int kChunk = 128 / kElemBytes;                 // elements per 128-byte swizzle row
  static constexpr int kBoxes = kIdxDim / kChunk;                 // TMA boxes per tile: 2 (bf16), 1 (fp8)
  static constexpr uint32_t kTileBytes = kIdxTile * kIdxDim * kElemBytes;   // 32 / 16 KiB
  static constexpr uint32_t kQBytes = kIdxHeads * kIdxDim * kElemBytes;     // 16 / 8 KiB
  static constexpr int kMmaPerBox = 4;                            // 128 bytes of K per box / 32 bytes per MMA
  static constexpr int kStages = kFp8 ? FFTOPK_IDX_STAGES_FP8 : 4 / FFTOPK_IDX_CTAS_PER_SM;  // key tiles in flight: 128 KiB either way
  // instruction descriptor: D fp32; A and B bf16 (format 1) or e4m3 (format 0), both K-major; M = 128, N = 64
  static constexpr uint32_t kInstrDesc = (1u << 4) | ((kFp8 ? 0u : 1u) << 7) | ((kFp8 ? 0u : 1u) << 10) |
                                         ((uint32_t)(kIdxHeads >> 3) << 17) | ((uint32_t)(kIdxTile >> 4) << 24);
};
constexpr int kIdxBufs = 4;         // TMEM accumulators of 64 columns: the MMAs run up to four tiles ahead of the epilogue
// fp8: the per-key scales of a tile ride along with it as one 512-byte bulk copy onto the same
// barrier. Their shared-memory slots form a ring of stages + accumulators entries: the copy for
// tile i reuses the slot of tile i - ring, whose epilogue read its scales before it released its
// accumulator, which the MMAs of tile i - stages - whose completion frees the stage this copy waits
// for - had to wait for. (As loads in the epilogue the same 4 MB cost 2 us per call at 1M keys.)
template <bool kFp8>
struct IdxScaleRing {
  static constexpr int kSlots = kFp8 ? IdxFmt<true>::kStages + kIdxBufs : 0;
};
constexpr uint32_t kIdxScaleBytes = kIdxTile * 4;
constexpr int kIdxCandCap = 8192;  // slots of a row's candidate list: what the freed stages of a CTA hold (64 KiB of composites)
constexpr unsigned long long kIdxWaitNs = 200ull * 1000 * 1000;

struct IndexerParams {
  const float* w;            // [B, 64] head weights
  const float* k_scale;      // fp8 only: [B, k_scale_stride] one scale per key, or nullptr
  int64_t k_scale_stride;
  int32_t scale_bulk;        // k_scale and its stride are 16-byte aligned: the scales of a tile travel as one bulk copy
  const int32_t* lengths;    // [B]
  int64_t k_rows_per_seq;    // rows of the key tensor map per batch row
  int32_t B;
  int64_t L;
  float* logits;             // [B, logits_stride]: every valid key's logit
  int64_t logits_stride;
  const uint32_t* guess;     // [B] threshold key guesses (0: none) or nullptr
  uint32_t margin;
  uint64_t* cand;            // [B, kIdxCandCap] candidates as (key << 32 | ~index) composites
  uint32_t* cand_count;      // [B] candidates appended so far (may exceed the capacity: the row then falls back)
  uint32_t* done_count;      // [B] CTAs of the row that have run out of tiles
  uint32_t* select_rows;     // [B] out: 1 = the selector has to run on the row's logits
  int32_t* out_idx;          // [B, 2048]
  uint32_t* thr_out;         // [B] the row's new threshold key (rows finished here)
  uint32_t* status;
};

// ---- mbarrier / TMA / tcgen05 wrappers -----------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
  return ok != 0u;
}
// Bounded wait: false when the time ran out or another thread of the CTA has given up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (t - t0 > kIdxWaitNs) {
      *abort_flag = 1u;
      return false;
    }
  }
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// 1-D bulk copy global -> shared (16-byte aligned addresses, size a multiple of 16 bytes)
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// Shared-memory matrix descriptor of a K-major operand in the 128-byte-swizzle layout a TMA box of
// 128 bytes (64 bf16 or 128 fp8) x rows produces: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);  // start address, 16-byte units
  d |= (uint64_t)1u << 16;                       // leading byte offset (unused with swizzle): 1
  d |= (uint64_t)(1024u >> 4) << 32;             // stride byte offset: 8 rows x 128 B
  d |= (uint64_t)1u << 46;                       // descriptor version of sm_100
  d |= (uint64_t)2u << 61;                       // layout type: 128-byte swizzle
  return d;
}
template <bool kFp8>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
  if constexpr (kFp8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(IdxFmt<true>::kInstrDesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(IdxFmt<false>::kInstrDesc), "r"(accumulate)
        : "memory");
  }
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

// ---- finish of one row, by the last of its CTAs to run out of tiles ----------------------------------
// `gkey`: the key guess the row was filtered with (margin already subtracted); `count`: how many
// candidates were appended. `cand_smem` holds kIdxCandCap composites, `hist` kFinishBins words.
template <int NT>
__device__ __noinline__ void indexer_finish_row(const IndexerParams& p, int row, int len, uint32_t gkey, uint32_t count,
                                                   uint64_t* cand_smem, uint32_t* hist, Ctrl* ctrl) {
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const bool held = len > kK && count >= (uint32_t)kK && count <= (uint32_t)kIdxCandCap;
  if (!held) {  // (uniform over the CTA)
    if (tid == 0) {
      p.select_rows[row] = 1u;
      if (p.status) atomicOr(p.status, (uint32_t)FFTOPK_ST_GUESS_MISSED);
    }
    return;
  }
  // the list, out of L2 (other SMs wrote it), eight loads in flight per thread
  const uint64_t* src = p.cand + (size_t)row * kIdxCandCap;
  uint32_t kmax = 0u;
  for (uint32_t i0 = 0; i0 < count; i0 += 8u * NT) {
    uint64_t c[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const uint32_t i = i0 + (uint32_t)u * NT + tid;
      c[u] = i < count ? __ldcg(src + i) : 0ull;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const uint32_t i = i0 + (uint32_t)u * NT + tid;
      if (i < count) {
        cand_smem[i] = c[u];
        kmax = max(kmax, (uint32_t)(c[u] >> 32));
      }
    }
  }
  kmax = __reduce_max_sync(kFull, kmax);
  if (lane == 0) ctrl->wmax[warp] = kmax;
  if (tid == 0) ctrl->thr_key = 0xffffffffu;
  __syncthreads();
  kmax = 0u;
#pragma unroll
  for (int w = 0; w < NT / 32; ++w) kmax = max(kmax, ctrl->wmax[w]);
  // every candidate's key lies in [the guess's lowest admitted key, kmax]
  const uint64_t lo = (uint64_t)guess_low_key(gkey) << 32;
  const uint64_t cap = ((uint64_t)kmax << 32) | 0xffffffffull;
  const int idx_bits = 32 - __clz(len - 1);
  const DenseCands<NT> list{cand_smem, (int)count};
  cta_finish<NT, DenseCands<NT>, true>(list, (uint32_t)kK, lo, cap, cap, false, idx_bits, hist, ctrl,
                                       p.out_idx + (int64_t)row * kK, nullptr, 0u, (uint32_t)kK, 0, p.status, nullptr, count);
  __syncthreads();
  if (tid == 0) {
    p.thr_out[row] = ctrl->thr_key != 0xffffffffu ? ctrl->thr_key : 0u;
    p.select_rows[row] = 0u;
  }
}

__device__ __forceinline__ int indexer_row_tiles(const IndexerParams& p, int row, int& len) {
  int64_t len64 = p.lengths[row];
  len64 = len64 < 0 ? 0 : (len64 > p.L ? p.L : len64);
  len = (int)len64;
  return (len + kIdxTile - 1) / kIdxTile;
}

// whether the scales of a row's tile t travel with the tile (a bulk copy of 128 floats): the copy
// must stay inside the row's scale array
template <bool kFp8>
__device__ __forceinline__ bool idx_scales_by_copy(const IndexerParams& p, int t) {
  if constexpr (kFp8) {
    return p.k_scale != nullptr && p.scale_bulk != 0 && (int64_t)(t + 1) * kIdxTile <= p.k_scale_stride;
  } else {
    return false;
  }
}
// the key guess a row is filtered with: the caller's, less the margin (0: none)
__device__ __forceinline__ uint32_t indexer_row_guess(const IndexerParams& p, int row) {
  const uint32_t raw = p.guess != nullptr ? p.guess[row] : 0u;
  return raw == 0u ? 0u : (raw > p.margin ? raw - p.margin : 1u);
}

// ---- epilogue of one segment (warps 2-9): one key per thread; group g of four warps serves every
// second tile. (With two accumulators and one group the loop MMA -> full barrier -> TMEM loads ->
// empty barrier -> next MMA into the same accumulator took ~1.1 us per pair of tiles: as long as
// the key tiles' copies take in bf16, twice as long as they take in fp8.) Out of line: the 64
// accumulator values of a key want the registers the kernel's segment bookkeeping would hold.
template <bool kFp8>
__device__ __noinline__ void indexer_epilogue_segment(const IndexerParams& p, int row, int t_lo, int t_step, int n, int it_base,
                                                      uint32_t tmem_base, uint64_t* tfull, uint64_t* tempty,
                                                      volatile uint32_t* abort_flag, float* w_smem, const float* ks_smem) {
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int group = (warp - 2) >> 2;
  const int quarter = warp & 3;                 // the TMEM lanes this warp may read: 32 * (warp % 4)
  const int key_in_tile = quarter * 32 + lane;
  const unsigned lt = (1u << lane) - 1u;
  const float4* w4 = reinterpret_cast<const float4*>(w_smem);
  // the row's weights, among the epilogue warps only
  if (tid >= 64 && tid < 64 + kIdxHeads) w_smem[tid - 64] = __ldg(p.w + (int64_t)row * kIdxHeads + (tid - 64));
  int len;
  indexer_row_tiles(p, row, len);
  const uint32_t guess = indexer_row_guess(p, row);
  const bool filter_mode = guess != 0u;
  const float edge = __uint_as_float(guess_edge_bits(guess));
  if (tid == kIdxThreads - 1 && t_lo == 0 && !filter_mode) p.select_rows[row] = 1u;  // no guess to test: the selector takes the row
  asm volatile("bar.sync 1, 256;" ::: "memory");
  for (int i = ((it_base & 1) == group) ? 0 : 1; i < n; i += 2) {
    const int it = it_base + i;
    const int buf = it % kIdxBufs;
    const uint32_t bph = (uint32_t)(it / kIdxBufs) & 1u;
    const int t = t_lo + i * t_step;
    const int key = t * kIdxTile + key_in_tile;
    const bool valid = key < len;
    // The key's scale: out of the ring in shared memory where the tile's copy brought it (read below,
    // before the accumulator is released: see IdxScaleRing), else loaded here, before the wait,
    // so that its latency hides behind the tile's copy and MMAs.
    float scale = 1.f;
    const bool scales = idx_scales_by_copy<kFp8>(p, t);
    if constexpr (kFp8) {
      if (p.k_scale != nullptr && !scales && valid) scale = __ldg(p.k_scale + (int64_t)row * p.k_scale_stride + key);
    }
    if (!mbar_wait(&tfull[buf], bph, abort_flag)) break;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * kIdxHeads;
    uint32_t v0[32], v1[32];
    tmem_ld32(taddr, v0);
    tmem_ld32(taddr + 32u, v1);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    if constexpr (kFp8) {
      if (scales) scale = ks_smem[(it % IdxScaleRing<kFp8>::kSlots) * kIdxTile + key_in_tile];
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    mbar_arrive(&tempty[buf]);  // the values are in registers: the accumulator buffer may be overwritten
    float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 wa = w4[j], wb = w4[8 + j];
      acc0 = fmaf(wa.x, fmaxf(__uint_as_float(v0[4 * j + 0]), 0.f), acc0);
      acc1 = fmaf(wb.x, fmaxf(__uint_as_float(v1[4 * j + 0]), 0.f), acc1);
      acc0 = fmaf(wa.y, fmaxf(__uint_as_float(v0[4 * j + 1]), 0.f), acc0);
      acc1 = fmaf(wb.y, fmaxf(__uint_as_float(v1[4 * j + 1]), 0.f), acc1);
      acc0 = fmaf(wa.z, fmaxf(__uint_as_float(v0[4 * j + 2]), 0.f), acc0);
      acc1 = fmaf(wb.z, fmaxf(__uint_as_float(v1[4 * j + 2]), 0.f), acc1);
      acc0 = fmaf(wa.w, fmaxf(__uint_as_float(v0[4 * j + 3]), 0.f), acc0);
      acc1 = fmaf(wb.w, fmaxf(__uint_as_float(v1[4 * j + 3]), 0.f), acc1);
    }
    // relu(s * x) = s * relu(x) for a positive scale: the key's scale multiplies the finished sum
    const float logit = (acc0 + acc1) * scale;
    if (valid) p.logits[(int64_t)row * p.logits_stride + key] = logit;
    if (filter_mode) {
      const bool hit = valid && !(logit < edge);
      const unsigned b = __ballot_sync(kFull, hit);
      if (b) {
        uint32_t slot = 0;
        if (lane == 0) slot = atomicAdd(p.cand_count + row, (uint32_t)__popc(b));
        slot = __shfl_sync(kFull, slot, 0) + (uint32_t)__popc(b & lt);
        if (hit && slot < (uint32_t)kIdxCandCap)
          p.cand[(size_t)row * kIdxCandCap + slot] =
              ((uint64_t)fftopk_key_from_bits(__float_as_uint(logit)) << 32) | (uint64_t)(~(uint32_t)key);
      }
    }
  }
}

// ---- producer --------------------------------------------------------------------------------------
// Work split. The tiles of all rows, row after row, form one sequence; CTA c takes the c-th run of
// `quota` consecutive tiles of it (quota = tiles / CTAs, rounded up), so every CTA streams the same
// number of bytes whatever the rows' lengths are, and a run may cover the end of one row, several
// whole rows and the start of another. The part of a run inside one row is a segment: the CTA
// loads that row's q and weights, runs its pipeline over the segment's tiles, lets it drain and
// counts the tiles off at the row's arrival counter. The row -> first-tile table is computed by
// every CTA for itself (a block scan over the lengths) and kept in shared memory, for batches of up
// to kIdxBalancedRows rows; larger batches give every row one CTA.
constexpr int kIdxBalancedRows = 1024;

template <bool kFp8>
__global__ void __launch_bounds__(kIdxThreads, FFTOPK_IDX_CTAS_PER_SM)
    indexer_logits_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                          const __grid_constant__ IndexerParams p) {
  using F = IdxFmt<kFp8>;
  static_assert((size_t)F::kStages * F::kTileBytes >= (size_t)kIdxCandCap * 8, "the stages hold a row's candidate list");
  static_assert(F::kQBytes >= (uint32_t)kFinishBins * 4u, "q's place holds the finish's histogram");
  constexpr uint32_t kIdxTileBytes = F::kTileBytes;
  constexpr uint32_t kIdxQBytes = F::kQBytes;
  constexpr int kIdxStages = F::kStages;
  extern __shared__ unsigned char idx_smem_raw[];
  // 1024-byte alignment for the swizzled tiles
  unsigned char* base = idx_smem_raw + ((1024u - (smem_u32(idx_smem_raw) & 1023u)) & 1023u);
  unsigned char* a_smem = base;                                   // kIdxStages x 32 KiB
  unsigned char* q_smem = a_smem + (size_t)kIdxStages * kIdxTileBytes;  // 16 / 8 KiB
  float* w_smem = reinterpret_cast<float*>(q_smem + kIdxQBytes);  // 64 floats
  float* ks_smem = w_smem + kIdxHeads;                            // fp8: ring of per-tile key scales
  uint64_t* bars = reinterpret_cast<uint64_t*>(ks_smem + IdxScaleRing<kFp8>::kSlots * kIdxTile);
  uint64_t* full = bars;                     // [kIdxStages]
  uint64_t* empty = bars + kIdxStages;       // [kIdxStages]
  uint64_t* tfull = bars + 2 * kIdxStages;   // [kIdxBufs]
  uint64_t* tempty = tfull + kIdxBufs;       // [kIdxBufs]
  uint64_t* qfull = tempty + kIdxBufs;       // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 32);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  uint32_t* last_flag = tmem_slot + 2;       // [2]: this CTA finishes the row; the row's candidate count
  uint32_t* scan_part = tmem_slot + 4;       // [12]: warp totals of the block scan
  Ctrl* fin_ctrl = reinterpret_cast<Ctrl*>(tmem_slot + 16);
  uint32_t* first_tile = reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(fin_ctrl) + ((sizeof(Ctrl) + 15) & ~15u));
  // first_tile[r], r <= B: tiles of the rows before r (balanced mode only)

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  // the selector follows as a programmatic dependent (see the host side): let it become resident
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (tid == 0) {
    // the copies' descriptors, on their way while the tile table is built
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_q)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_k)) : "memory");
    for (int s = 0; s < kIdxStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < kIdxBufs; ++b) {
      mbar_init(&tfull[b], 1);
      mbar_init(&tempty[b], 128);
    }
    mbar_init(qfull, 1);
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)(kIdxBufs * kIdxHeads))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  // Everything above touched shared and tensor memory only. From here on the kernel in front of this
  // one on the stream (the selector of the call before, in a decode loop) has to have completed:
  // the producer is launched as its programmatic dependent, so its launch and this prologue hide
  // behind that kernel.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- this CTA's run of tiles [g0, g1) and the row it starts in (the barriers in here also
  // publish the mbarriers and the TMEM address) ------------------------------------------------------
  const bool balanced = p.B <= kIdxBalancedRows;
  uint32_t g0 = 0u, g1 = 0u;
  int row = 0;
  if (p.B == 1) {
    // one row: no table to build (and see below: its tiles go to the CTAs interleaved, not in runs)
    int len_r;
    const uint32_t total = (uint32_t)indexer_row_tiles(p, 0, len_r);
    if (tid == 0) {
      first_tile[0] = 0u;
      first_tile[1] = total;
      if (total == 0u && blockIdx.x == 0) p.select_rows[0] = 1u;
    }
    __syncthreads();
    const TileRun run = tile_run(total, gridDim.x, blockIdx.x);
    g0 = run.g0;
    g1 = run.g1;
  } else if (balanced) {
    constexpr int PER = (kIdxBalancedRows + kIdxThreads - 1) / kIdxThreads;
    uint32_t mine[PER];
    uint32_t sum = 0u;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int r = tid * PER + j;
      int len_r;
      mine[j] = r < p.B ? (uint32_t)indexer_row_tiles(p, r, len_r) : 0u;
      if (r < p.B && mine[j] == 0u && blockIdx.x == 0) p.select_rows[r] = 1u;  // no key at all: the selector pads the row
      sum += mine[j];
    }
    uint32_t incl = sum;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t v = __shfl_up_sync(kFull, incl, off);
      if (lane >= off) incl += v;
    }
    if (lane == 31) scan_part[warp] = incl;
    __syncthreads();
    uint32_t before = 0u;
    for (int wv = 0; wv < warp; ++wv) before += scan_part[wv];
    uint32_t run = before + incl - sum;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int r = tid * PER + j;
      if (r < p.B) first_tile[r] = run;
      run += mine[j];
      if (r == p.B - 1) first_tile[p.B] = run;
    }
    __syncthreads();
    const TileRun own = tile_run(first_tile[p.B], gridDim.x, blockIdx.x);
    g0 = own.g0;
    g1 = own.g1;
    row = tile_row_at(first_tile, p.B, g0);
  } else {
    row = (int)blockIdx.x;
    int len_r;
    g1 = (uint32_t)indexer_row_tiles(p, row, len_r);
    if (g1 == 0u && tid == 0) p.select_rows[row] = 1u;
    __syncthreads();
  }
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  if (g0 >= g1) {  // (uniform) nothing to do
    if (warp == 1) {
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(kIdxBufs * kIdxHeads))
                   : "memory");
    }
    return;
  }

  int it_base = 0;   // tiles this CTA has been through: selects stages, accumulators and barrier phases
  int seg_no = 0;
  for (uint32_t g = g0; g < g1; ++row) {
    // ---- the segment of this row -----------------------------------------------------------------
    // (tile counts out of shared memory: the thread that issues the copies waits for no global load)
    const uint32_t row_g0 = balanced ? first_tile[row] : 0u;
    const int ntiles = balanced ? (int)(first_tile[row + 1] - row_g0) : (int)g1;
    int t_lo, n;
    if (!tile_segment(row_g0, (uint32_t)ntiles, g, g1, t_lo, n)) continue;  // (a row without tiles)
    g += (uint32_t)n;
    int t_step = 1;
    if (p.B == 1) {
      // One row: CTA x takes tiles x, x + CTAs, ... - as many as its run would hold (the first `rest`
      // CTAs one more) - so that at any moment the CTAs read one dense window of the key cache
      // (measured 0.2 us per call faster at 128K keys, 0.7 us at 1M, than a run per CTA).
      t_lo = (int)blockIdx.x;
      t_step = (int)gridDim.x;
    }
    // (No barrier of the whole CTA here: the barriers at the end of the segment before have ordered
    // everything this one overwrites. And nothing in front of the role branches that waits for
    // global memory: the threads that issue the copies and the MMAs start at once; the row's
    // length and guess are read by the epilogue warps, and by everybody at the segment's end.)

    if (warp == 0) {
      // ---- TMA producer ---------------------------------------------------------------------------
      if (lane == 0) {
        mbar_expect_tx(qfull, kIdxQBytes);
#pragma unroll
        for (int bx = 0; bx < F::kBoxes; ++bx)
          tma_load_2d(q_smem + (size_t)bx * (kIdxQBytes / F::kBoxes), &map_q, bx * F::kChunk, row * kIdxHeads, qfull);
        for (int i = 0; i < n; ++i) {
          const int it = it_base + i;
          const int s = it % kIdxStages;
          const uint32_t ph = (uint32_t)(it / kIdxStages) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) break;
          const int t = t_lo + i * t_step;
          const bool scales = idx_scales_by_copy<kFp8>(p, t);
          mbar_expect_tx(&full[s], kIdxTileBytes + (scales ? kIdxScaleBytes : 0u));
          const int y = (int)((int64_t)row * p.k_rows_per_seq + (int64_t)t * kIdxTile);
          unsigned char* dst = a_smem + (size_t)s * kIdxTileBytes;
#pragma unroll
          for (int bx = 0; bx < F::kBoxes; ++bx)
            tma_load_2d(dst + (size_t)bx * (kIdxTileBytes / F::kBoxes), &map_k, bx * F::kChunk, y, &full[s]);
          if constexpr (kFp8) {
            if (scales)
              bulk_load(ks_smem + (it % IdxScaleRing<kFp8>::kSlots) * kIdxTile,
                        p.k_scale + (int64_t)row * p.k_scale_stride + (int64_t)t * kIdxTile, kIdxScaleBytes, &full[s]);
          }
        }
      }
    } else if (warp == 1) {
      // ---- MMA issuer -----------------------------------------------------------------------------
      if (lane == 0) {
        bool ok = mbar_wait(qfull, (uint32_t)seg_no & 1u, abort_flag);
        for (int i = 0; ok && i < n; ++i) {
          const int it = it_base + i;
          const int s = it % kIdxStages;
          const uint32_t ph = (uint32_t)(it / kIdxStages) & 1u;
          const int buf = it % kIdxBufs;
          const uint32_t bph = (uint32_t)(it / kIdxBufs) & 1u;
          if (!mbar_wait(&tempty[buf], bph ^ 1u, abort_flag)) break;
          if (!mbar_wait(&full[s], ph, abort_flag)) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_u32(a_smem + (size_t)s * kIdxTileBytes);
          const uint32_t b_addr = smem_u32(q_smem);
          const uint32_t d_tmem = tmem_base + (uint32_t)buf * kIdxHeads;
#pragma unroll
          for (int kc = 0; kc < F::kBoxes; ++kc) {
#pragma unroll
            for (int kk = 0; kk < F::kMmaPerBox; ++kk) {
              // one MMA consumes 32 bytes of K (16 bf16 or 32 fp8): 32 bytes further inside the swizzle row
              const uint64_t ad = umma_desc_sw128(a_addr + (uint32_t)kc * (kIdxTileBytes / F::kBoxes) + (uint32_t)kk * 32u);
              const uint64_t bd = umma_desc_sw128(b_addr + (uint32_t)kc * (kIdxQBytes / F::kBoxes) + (uint32_t)kk * 32u);
              umma<kFp8>(d_tmem, ad, bd, (kc | kk) != 0 ? 1u : 0u);
            }
          }
          umma_commit(&empty[s]);     // the stage may be refilled once these MMAs have read it
          umma_commit(&tfull[buf]);   // ... and the accumulator is complete
        }
      }
    } else {
      // ---- epilogue ---------------------------------------------------------------------------------
      indexer_epilogue_segment<kFp8>(p, row, t_lo, t_step, n, it_base, tmem_base, tfull, tempty, abort_flag, w_smem, ks_smem);
    }
    // The idle lanes of the two single-thread warps wait here for their working lane: what follows
    // (global loads, a fence) would otherwise run ahead on them and hold the warp's issue slot while
    // the working lane has copies or MMAs to issue (measured: the first tile's MMAs 1.7 us late).
    if (warp < 2) __syncwarp();
    it_base += n;
    ++seg_no;
    int len;
    indexer_row_tiles(p, row, len);
    const uint32_t guess = indexer_row_guess(p, row);
    const bool filter_mode = guess != 0u;
    // ---- end of the segment: every tile has been through the epilogue, so every copy and MMA of
    // the segment has completed; the CTA counts its tiles off and the row's last CTA finishes it ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    if (__syncthreads_or((int)*abort_flag)) break;  // (uniform)
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (!filter_mode) continue;  // (uniform)
    if (tid == 0) {
      // Release: the barrier has ordered every thread's candidate stores before this fence, the
      // fence orders them before the arrival (the pattern of a grid-wide barrier: one fence by
      // the arriving thread instead of one per thread - 320 of them took 1.4 us).
      __threadfence();
      const bool last = atomicAdd(p.done_count + row, (uint32_t)n) + (uint32_t)n == (uint32_t)ntiles;
      uint32_t count = 0u;
      if (last) {
        // every tile of the row has been counted off: nobody appends any more (each CTA's appends
        // were performed before its arrival). Take the count and leave both counters at zero for
        // the next call.
        count = atomicExch(p.cand_count + row, 0u);
        p.done_count[row] = 0u;
        __threadfence();  // acquire: the other CTAs' candidates, before this CTA reads them (behind the barrier below)
      }
      last_flag[0] = last ? 1u : 0u;
      last_flag[1] = count;
    }
    __syncthreads();
    if (last_flag[0] != 0u) {  // (uniform)
      // the stages hold the list, q's place the histogram
      indexer_finish_row<kIdxThreads>(p, row, len, guess, last_flag[1], reinterpret_cast<uint64_t*>(a_smem),
                                      reinterpret_cast<uint32_t*>(q_smem), fin_ctrl);
      // the next segment's copies overwrite what the threads wrote there
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncthreads();
    }
  }
  // ---- wind down ---------------------------------------------------------------------------------
  if (*abort_flag) {
    // a wait ran out: give copies that may still be in flight a moment to land before the shared
    // memory goes away. The rows of this call are not all finished and their counters not all back
    // at zero: the caller sees the status bit and zero-fills the workspace again.
    unsigned long long t0, t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    do {
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    } while (t - t0 < 100000ull);
    if (tid == 0 && p.status) atomicOr(p.status, (uint32_t)FFTOPK_ST_STAGE_TIMEOUT);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(kIdxBufs * kIdxHeads))
                 : "memory");
  }
}

}  // namespace fftopk

// ==============================================================================================
// Host side
// ==============================================================================================
namespace {
using namespace fftopk;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

DeviceOnce g_indexer_once[kMaxDevices];
EncodeTiledFn g_encode = nullptr;
std::mutex g_encode_mu;

constexpr size_t indexer_smem_bytes(bool fp8) {
  return 1024 +
         (fp8 ? (size_t)IdxFmt<true>::kStages * IdxFmt<true>::kTileBytes : (size_t)IdxFmt<false>::kStages * IdxFmt<false>::kTileBytes) +
         (fp8 ? IdxFmt<true>::kQBytes : IdxFmt<false>::kQBytes) + kIdxHeads * 4 + (fp8 ? IdxScaleRing<true>::kSlots * kIdxScaleBytes : 0) +
         32 * 8 + 64 + ((sizeof(Ctrl) + 15) & ~(size_t)15) +
         (size_t)(kIdxBalancedRows + 1) * 4 + 16;
}

int indexer_setup() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= kMaxDevices) return FFTOPK_EDEVICE;
  {
    std::lock_guard<std::mutex> lock(g_encode_mu);
    if (g_encode == nullptr) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
      if (e != cudaSuccess) return cuda_fail(e);
      if (fn == nullptr || qres != cudaDriverEntryPointSuccess) return FFTOPK_EDEVICE;
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
  }
  return g_indexer_once[dev].run([&] {
    cudaError_t e2 = cudaFuncSetAttribute(indexer_logits_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)indexer_smem_bytes(false));
    if (e2 != cudaSuccess) return cuda_fail(e2);
    e2 = cudaFuncSetAttribute(indexer_logits_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              (int)indexer_smem_bytes(true));
    if (e2 != cudaSuccess) return cuda_fail(e2);
    return 0;
  });
}

// [rows, 128] bf16 or fp8 (one byte), row pitch `pitch_elems`, boxes of 128 bytes x box_rows rows,
// 128-byte swizzle
int make_map(CUtensorMap* map, const void* ptr, bool fp8, uint64_t rows, uint64_t pitch_elems, uint32_t box_rows) {
  const cuuint64_t gdim[2] = {(cuuint64_t)kIdxDim, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)pitch_elems * (fp8 ? 1 : 2)};
  const cuuint32_t box[2] = {(cuuint32_t)(fp8 ? 128 : 64), box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = g_encode(map, fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                              const_cast<void*>(ptr), gdim, gstride, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : FFTOPK_EINVAL;
}

// Workspace: [candidate lists: B x kIdxCandCap composites][candidate counts: B words][arrival
// counts: B words][rows the selector takes: B words]
struct IndexerLayout {
  size_t cand_off, count_off, done_off, select_off, total;
};
IndexerLayout indexer_layout(int32_t B) {
  IndexerLayout l;
  const size_t words = ((size_t)B * 4 + 255) & ~(size_t)255;
  l.cand_off = 0;
  l.count_off = (size_t)B * kIdxCandCap * 8;
  l.done_off = l.count_off + words;
  l.select_off = l.done_off + words;
  l.total = l.select_off + words;
  return l;
}

template <bool kFp8>
cudaError_t launch_producer(dim3 grid, cudaStream_t stream, const CUtensorMap& map_q, const CUtensorMap& map_k,
                            const IndexerParams& p) {
  // a programmatic dependent of whatever kernel the stream holds in front of it: the kernel waits
  // for that one (griddepcontrol.wait) before it touches global memory
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kIdxThreads, 1, 1);
  cfg.dynamicSmemBytes = indexer_smem_bytes(kFp8);
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, indexer_logits_kernel<kFp8>, map_q, map_k, p);
}

}  // namespace

extern "C" {

size_t fftopk_indexer_workspace_bytes(int32_t B) {
  if (B <= 0) return 0;
  return indexer_layout(B).total;
}

static int indexer_topk_impl(bool fp8, const void* q, const void* k_cache, int64_t k_rows_per_seq, const float* k_scale,
                             int64_t k_scale_stride, const float* w, int32_t B, int64_t L, const int32_t* lengths,
                             uint32_t* thresholds, uint32_t margin, float* logits, int64_t logits_stride, int32_t* out_idx,
                             void* d_workspace, size_t workspace_bytes, uint32_t* status, void* cuda_stream) {
  if (B < 0 || L < 0 || k_rows_per_seq < L || logits_stride < L) return FFTOPK_EINVAL;
  if (k_scale != nullptr && k_scale_stride < L) return FFTOPK_EINVAL;
  if (B == 0) return FFTOPK_OK;
  if (!q || !k_cache || !w || !lengths || !thresholds || !logits || !out_idx || !d_workspace) return FFTOPK_EINVAL;
  if (((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache)) & 15u) != 0) return FFTOPK_EINVAL;
  if ((reinterpret_cast<uintptr_t>(d_workspace) & 255u) != 0) return FFTOPK_EINVAL;
  if (L > (int64_t)0x7fffffff - 256 || B > 65535 || (int64_t)B * k_rows_per_seq > (int64_t)0x7fffffff - 256) return FFTOPK_ERANGE;
  const IndexerLayout lay = indexer_layout(B);
  if (workspace_bytes < lay.total) return FFTOPK_EINVAL;
  int rc = indexer_setup();
  if (rc) return rc;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return cuda_fail(e);
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  char* ws = static_cast<char*>(d_workspace);

  CUtensorMap map_q, map_k;
  rc = make_map(&map_q, q, fp8, (uint64_t)B * kIdxHeads, kIdxDim, kIdxHeads);
  if (rc) return rc;
  rc = make_map(&map_k, k_cache, fp8, (uint64_t)B * (uint64_t)k_rows_per_seq, kIdxDim, kIdxTile);
  if (rc) return rc;

  IndexerParams p;
  memset(&p, 0, sizeof(p));
  p.w = w;
  p.k_scale = k_scale;
  p.k_scale_stride = k_scale_stride;
  p.scale_bulk = (k_scale != nullptr && (reinterpret_cast<uintptr_t>(k_scale) & 15u) == 0 && (k_scale_stride & 3) == 0) ? 1 : 0;
  p.lengths = lengths;
  p.k_rows_per_seq = k_rows_per_seq;
  p.B = B;
  p.L = L;
  p.logits = logits;
  p.logits_stride = logits_stride;
  p.guess = thresholds;
  p.margin = margin;
  p.cand = reinterpret_cast<uint64_t*>(ws + lay.cand_off);
  p.cand_count = reinterpret_cast<uint32_t*>(ws + lay.count_off);
  p.done_count = reinterpret_cast<uint32_t*>(ws + lay.done_off);
  p.select_rows = reinterpret_cast<uint32_t*>(ws + lay.select_off);
  p.out_idx = out_idx;
  p.thr_out = thresholds;
  p.status = status;

  // batches of up to kIdxBalancedRows rows: as many CTAs as are resident at once, each with an equal
  // share of all rows' tiles (found on the device); larger batches: one CTA per row
  const int64_t ntiles = (L + kIdxTile - 1) / kIdxTile;
  int64_t ctas = B;
  if (B <= kIdxBalancedRows) {
    ctas = (int64_t)sms * FFTOPK_IDX_CTAS_PER_SM;
    if (ctas > (int64_t)B * ntiles) ctas = (int64_t)B * ntiles;
    if (ctas < 1) ctas = 1;
  }
  const dim3 grid((unsigned)ctas, 1u, 1u);
  // the producer: logits; rows with a guess are filtered as the logits are produced and finished
  // by their last CTA
  e = fp8 ? launch_producer<true>(grid, stream, map_q, map_k, p) : launch_producer<false>(grid, stream, map_q, map_k, p);
  if (e != cudaSuccess) return cuda_fail(e);
  // the selector on the logits of the rows without a usable guess; it hands back their thresholds
  SelectCall c;
  c.score = logits;
  c.row_stride = logits_stride;
  c.B = B;
  c.L = L;
  c.lengths = lengths;
  c.out_idx = out_idx;
  c.status = status;
  c.cuda_stream = cuda_stream;
  c.next_threshold = thresholds;
  c.only_rows = p.select_rows;
  c.may_overlap = false;  // (a programmatic dependent of the producer that waits for it, like every default launch)
  return launch_select(c);
}

int fftopk_indexer_topk2048(const void* q, const void* k_cache, int64_t k_rows_per_seq, const float* w, int32_t B, int64_t L,
                            const int32_t* lengths, uint32_t* thresholds, uint32_t margin, float* logits,
                            int64_t logits_stride, int32_t* out_idx, void* d_workspace, size_t workspace_bytes,
                            uint32_t* status, void* cuda_stream) {
  return indexer_topk_impl(false, q, k_cache, k_rows_per_seq, nullptr, 0, w, B, L, lengths, thresholds, margin, logits,
                           logits_stride, out_idx, d_workspace, workspace_bytes, status, cuda_stream);
}

int fftopk_indexer_topk2048_fp8(const void* q, const void* k_cache, int64_t k_rows_per_seq, const float* k_scale,
                                int64_t k_scale_stride, const float* w, int32_t B, int64_t L, const int32_t* lengths,
                                uint32_t* thresholds, uint32_t margin, float* logits, int64_t logits_stride,
                                int32_t* out_idx, void* d_workspace, size_t workspace_bytes, uint32_t* status,
                                void* cuda_stream) {
  return indexer_topk_impl(true, q, k_cache, k_rows_per_seq, k_scale, k_scale_stride, w, B, L, lengths, thresholds, margin,
                           logits, logits_stride, out_idx, d_workspace, workspace_bytes, status, cuda_stream);
}

}  // extern "C"
