// Indexer logits fused with the top-2048 selection (sm_100a: TMA + tcgen05 + TMEM).
//
// The logit of key t of a row is  sum over 64 heads h of  w[h] * relu(q[h] . k[t])  (q[h], k[t] of
// dimension 128, bf16). The reference contains no producer of these logits - its selector starts
// from a finished fp32 [B, L] matrix (jit_kernel/topk_indexer.py:42-75) and its README only names
// the step (README.md:24) - so there is no reference counterpart; this is the step in front of the
// hot path, fused with it.
//
// Producer kernel, one CTA per (row, slice of key tiles), 192 threads in three roles:
//   warp 0      one thread issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle, no multicast):
//               the row's q once (64 heads x 128), then key tiles of 128 keys x 128 through a ring
//               of shared-memory stages guarded by full / empty mbarriers;
//   warp 1      allocates 128 TMEM columns; one thread issues, per tile, eight tcgen05.mma
//               (M=128 keys, N=64 heads, K=16) that accumulate D[key][head] in fp32 in one of two
//               64-column TMEM buffers, and commits to the stage's empty barrier and the buffer's
//               full barrier;
//   warps 2-5   epilogue: tcgen05.ld hands every thread the 64 head values of ONE key; relu,
//               weights and the sum are in-thread - one logit per thread and tile. With a threshold
//               guess for the row (the previous decode step's, see fftopk_select2048_warm) the
//               logit is compared with the guess's edge and the few that pass are appended, by
//               ballot and one atomic per warp, to the row's candidate list; the logit itself is
//               not written. Without a guess the logits are written for the selector.
// Every wait on an mbarrier has a time limit; when one runs out the CTA raises
// FFTOPK_ST_STAGE_TIMEOUT, lets its copies in flight land, frees its TMEM and returns.
//
// Finish kernel (one 8-CTA cluster per row): if the row's guess held - at least 2048 candidates, no
// more than the list holds - merge_row selects the exact top 2048 of the list (ties to the lower
// index) and hands back the new threshold; otherwise the row is marked, a second pass of the
// producer writes its logits and the selector of fftopk_select.cu runs on them (rows that are not
// marked cost those two launches nothing but an empty CTA).
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
#include "fftopk_merge.cuh"

namespace fftopk {

constexpr int kIdxHeads = 64;
constexpr int kIdxDim = 128;
constexpr int kIdxTile = 128;      // keys per tile = rows of the MMA
constexpr int kIdxStages = 4;      // key tiles in flight
constexpr int kIdxThreads = 192;
constexpr int kIdxChunk = 64;      // bf16 elements per 128-byte swizzle row
constexpr uint32_t kIdxTileBytes = kIdxTile * kIdxDim * 2;   // 32 KiB: two boxes of 128 rows x 128 B
constexpr uint32_t kIdxQBytes = kIdxHeads * kIdxDim * 2;     // 16 KiB: two boxes of 64 rows x 128 B
constexpr int kIdxCandShards = 8;  // the candidate list of a row: 8 x 2048 slots, the merge's layout
constexpr unsigned long long kIdxWaitNs = 200ull * 1000 * 1000;

struct IndexerParams {
  const float* w;            // [B, 64] head weights
  const int32_t* lengths;    // [B]
  int64_t k_rows_per_seq;    // rows of the key tensor map per batch row
  int32_t B;
  int64_t L;
  float* logits;             // [B, logits_stride]: written for rows without a guess / marked rows
  int64_t logits_stride;
  const uint32_t* guess;     // [B] threshold key guesses (0: none) or nullptr
  uint32_t margin;
  int32_t* cand_idx;         // [8, B, 2048] candidate indices (-1: empty), cand_key the same shape
  uint32_t* cand_key;
  uint32_t* cand_count;      // [B]
  const uint32_t* only_rows; // second pass: rows with only_rows[b] != 0 get their logits written,
                             // the others are skipped; nullptr in the first pass
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
// Shared-memory matrix descriptor of a K-major operand in the 128-byte-swizzle layout a TMA box of
// 64 bf16 x rows produces: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);  // start address, 16-byte units
  d |= (uint64_t)1u << 16;                       // leading byte offset (unused with swizzle): 1
  d |= (uint64_t)(1024u >> 4) << 32;             // stride byte offset: 8 rows x 128 B
  d |= (uint64_t)1u << 46;                       // descriptor version of sm_100
  d |= (uint64_t)2u << 61;                       // layout type: 128-byte swizzle
  return d;
}
// Instruction descriptor: D fp32, A and B bf16, both K-major, M = 128, N = 64.
constexpr uint32_t kIdxInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kIdxHeads >> 3) << 17) |
                                   ((uint32_t)(kIdxTile >> 4) << 24);
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(kIdxInstrDesc), "r"(accumulate)
      : "memory");
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

// ---- producer --------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kIdxThreads, 1)
    indexer_logits_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                          const IndexerParams p) {
  extern __shared__ unsigned char idx_smem_raw[];
  // 1024-byte alignment for the swizzled tiles
  unsigned char* base = idx_smem_raw + ((1024u - (smem_u32(idx_smem_raw) & 1023u)) & 1023u);
  unsigned char* a_smem = base;                                   // kIdxStages x 32 KiB
  unsigned char* q_smem = a_smem + (size_t)kIdxStages * kIdxTileBytes;  // 16 KiB
  float* w_smem = reinterpret_cast<float*>(q_smem + kIdxQBytes);  // 64 floats
  uint64_t* bars = reinterpret_cast<uint64_t*>(w_smem + kIdxHeads);
  uint64_t* full = bars;                     // [kIdxStages]
  uint64_t* empty = bars + kIdxStages;       // [kIdxStages]
  uint64_t* tfull = bars + 2 * kIdxStages;   // [2]
  uint64_t* tempty = tfull + 2;              // [2]
  uint64_t* qfull = tempty + 2;              // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(qfull + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int row = blockIdx.y;
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  if (p.only_rows != nullptr && p.only_rows[row] == 0u) return;  // (uniform over the CTA; nothing allocated yet)
  int64_t len64 = p.lengths[row];
  len64 = len64 < 0 ? 0 : (len64 > p.L ? p.L : len64);
  const int len = (int)len64;
  const int ntiles = (len + kIdxTile - 1) / kIdxTile;
  uint32_t guess = (p.only_rows == nullptr && p.guess != nullptr) ? p.guess[row] : 0u;
  if (guess != 0u) guess = guess > p.margin ? guess - p.margin : 1u;
  const bool filter_mode = guess != 0u;
  const float edge = __uint_as_float(guess_edge_bits(guess));
  if ((int)blockIdx.x >= ntiles) return;  // (uniform)

  if (tid == 0) {
    for (int s = 0; s < kIdxStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&tfull[0], 1);
    mbar_init(&tfull[1], 1);
    mbar_init(&tempty[0], 128);
    mbar_init(&tempty[1], 128);
    mbar_init(qfull, 1);
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid < kIdxHeads) w_smem[tid] = __ldg(p.w + (int64_t)row * kIdxHeads + tid);
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(128u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- TMA producer -----------------------------------------------------------------------
    if (lane == 0) {
      mbar_expect_tx(qfull, kIdxQBytes);
      tma_load_2d(q_smem, &map_q, 0, row * kIdxHeads, qfull);
      tma_load_2d(q_smem + kIdxQBytes / 2, &map_q, kIdxChunk, row * kIdxHeads, qfull);
      int it = 0;
      for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++it) {
        const int s = it % kIdxStages;
        const uint32_t ph = (uint32_t)(it / kIdxStages) & 1u;
        if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) break;
        mbar_expect_tx(&full[s], kIdxTileBytes);
        const int y = (int)((int64_t)row * p.k_rows_per_seq + (int64_t)t * kIdxTile);
        unsigned char* dst = a_smem + (size_t)s * kIdxTileBytes;
        tma_load_2d(dst, &map_k, 0, y, &full[s]);
        tma_load_2d(dst + kIdxTileBytes / 2, &map_k, kIdxChunk, y, &full[s]);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ---------------------------------------------------------------------------
    if (lane == 0) {
      bool ok = mbar_wait(qfull, 0u, abort_flag);
      int it = 0;
      for (int t = blockIdx.x; ok && t < ntiles; t += gridDim.x, ++it) {
        const int s = it % kIdxStages;
        const uint32_t ph = (uint32_t)(it / kIdxStages) & 1u;
        const int buf = it & 1;
        const uint32_t bph = (uint32_t)(it >> 1) & 1u;
        if (!mbar_wait(&tempty[buf], bph ^ 1u, abort_flag)) break;
        if (!mbar_wait(&full[s], ph, abort_flag)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = smem_u32(a_smem + (size_t)s * kIdxTileBytes);
        const uint32_t b_addr = smem_u32(q_smem);
        const uint32_t d_tmem = tmem_base + (uint32_t)buf * kIdxHeads;
#pragma unroll
        for (int kc = 0; kc < 2; ++kc) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            // 16 bf16 = 32 bytes further along K inside the 128-byte swizzle row
            const uint64_t ad = umma_desc_sw128(a_addr + (uint32_t)kc * (kIdxTileBytes / 2) + (uint32_t)kk * 32u);
            const uint64_t bd = umma_desc_sw128(b_addr + (uint32_t)kc * (kIdxQBytes / 2) + (uint32_t)kk * 32u);
            umma_bf16(d_tmem, ad, bd, (kc | kk) != 0 ? 1u : 0u);
          }
        }
        umma_commit(&empty[s]);     // the stage may be refilled once these MMAs have read it
        umma_commit(&tfull[buf]);   // ... and the accumulator is complete
      }
    }
  } else {
    // ---- epilogue: one key per thread -------------------------------------------------------------
    const int quarter = warp & 3;                 // the TMEM lanes this warp may read: 32 * (warp % 4)
    const int key_in_tile = quarter * 32 + lane;
    const unsigned lt = (1u << lane) - 1u;
    int it = 0;
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++it) {
      const int buf = it & 1;
      const uint32_t bph = (uint32_t)(it >> 1) & 1u;
      if (!mbar_wait(&tfull[buf], bph, abort_flag)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * kIdxHeads;
      float logit = 0.f;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t v[32];
        tmem_ld32(taddr + (uint32_t)half * 32u, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 32; ++j) logit = fmaf(w_smem[half * 32 + j], fmaxf(__uint_as_float(v[j]), 0.f), logit);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(&tempty[buf]);  // the accumulator buffer may be overwritten
      const int key = t * kIdxTile + key_in_tile;
      const bool valid = key < len;
      if (filter_mode) {
        const bool hit = valid && !(logit < edge);
        const unsigned b = __ballot_sync(kFull, hit);
        if (b) {
          uint32_t slot = 0;
          if (lane == 0) slot = atomicAdd(p.cand_count + row, (uint32_t)__popc(b));
          slot = __shfl_sync(kFull, slot, 0) + (uint32_t)__popc(b & lt);
          if (hit && slot < (uint32_t)(kIdxCandShards * kK)) {
            const size_t at = ((size_t)(slot / kK) * p.B + row) * kK + (slot % kK);
            p.cand_idx[at] = key;
            p.cand_key[at] = fftopk_key_from_bits(__float_as_uint(logit));
          }
        }
      } else if (valid) {
        p.logits[(int64_t)row * p.logits_stride + key] = logit;
      }
    }
  }
  // ---- wind down ---------------------------------------------------------------------------------
  if (*abort_flag) {
    // a wait ran out: give copies that may still be in flight a moment to land before the shared
    // memory goes away
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
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(128u) : "memory");
  }
}

// ---- finish: decide whether the guess held; if so, the exact top 2048 of the candidate list ------
template <int NT>
__global__ void __launch_bounds__(NT, 1)
    indexer_finish_kernel(const int32_t* __restrict__ cand_idx, const uint32_t* __restrict__ cand_key,
                          const uint32_t* __restrict__ cand_count, const uint32_t* __restrict__ guess,
                          const int32_t* __restrict__ lengths, int B, int32_t* __restrict__ out_idx_all,
                          uint32_t* __restrict__ thr_out, uint32_t* __restrict__ rewrite_rows,
                          uint32_t* __restrict__ select_rows, uint32_t* status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int G = kIdxCandShards;
  cg::cluster_group cluster = cg::this_cluster();
  const int g = (int)cluster.block_rank();
  const int row = (int)(blockIdx.x / (unsigned)G);
  const uint32_t count = cand_count[row];
  const uint32_t had_guess = guess != nullptr ? guess[row] : 0u;
  const bool short_row = lengths[row] <= kK;
  const bool held = had_guess != 0u && !short_row && count >= (uint32_t)kK && count <= (uint32_t)(G * kK);
  if (!held) {  // (uniform over the cluster)
    if (g == 0 && threadIdx.x == 0) {
      rewrite_rows[row] = had_guess != 0u ? 1u : 0u;  // its logits were not written in the first pass
      select_rows[row] = 1u;
      if (had_guess != 0u && status) atomicOr(status, (uint32_t)FFTOPK_ST_GUESS_MISSED);
    }
    return;
  }
  MergeSmem sm;
  sm.hist = reinterpret_cast<uint32_t*>(smem_raw);
  sm.sup = sm.hist + kMaxBins;
  sm.xch = sm.sup + kSup;
  sm.ctrl = reinterpret_cast<Ctrl*>(sm.xch + kMaxCluster * kSup);
  sm.cand = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(sm.ctrl) + ((sizeof(Ctrl) + 127) & ~127u));
  sm.cand_cap = G * kK;
  const int64_t off = ((int64_t)g * B + row) * kK;
  merge_row<NT, true>(cluster, G, G, g, sm, cand_idx + off, cand_key + off, nullptr, nullptr, 0u, 0ull,
                      out_idx_all + (int64_t)row * kK, nullptr, status, thr_out + row);
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

constexpr size_t indexer_smem_bytes() {
  return 1024 + (size_t)kIdxStages * kIdxTileBytes + kIdxQBytes + kIdxHeads * 4 + 16 * 8 + 64;
}
size_t finish_smem_bytes() {
  return (size_t)(kMaxBins + kSup + kMaxCluster * kSup) * 4 + ((sizeof(Ctrl) + 127) & ~(size_t)127) +
         (size_t)kIdxCandShards * kK * 8;
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
    cudaError_t e2 = cudaFuncSetAttribute(indexer_logits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)indexer_smem_bytes());
    if (e2 != cudaSuccess) return cuda_fail(e2);
    e2 = cudaFuncSetAttribute(indexer_finish_kernel<512>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)finish_smem_bytes());
    if (e2 != cudaSuccess) return cuda_fail(e2);
    return 0;
  });
}

// [rows, 128] bf16, row pitch `pitch_elems`, boxes of 64 elements x box_rows rows, 128-byte swizzle
int make_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t pitch_elems, uint32_t box_rows) {
  const cuuint64_t gdim[2] = {(cuuint64_t)kIdxDim, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)pitch_elems * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kIdxChunk, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : FFTOPK_EINVAL;
}

struct IndexerLayout {
  size_t idx_off, key_off, count_off, rewrite_off, select_off, total;
};
IndexerLayout indexer_layout(int32_t B) {
  IndexerLayout l;
  const size_t plane = (size_t)kIdxCandShards * B * kK * 4;
  l.idx_off = 0;
  l.key_off = plane;
  l.count_off = 2 * plane;
  l.rewrite_off = l.count_off + (((size_t)B * 4 + 255) & ~(size_t)255);
  l.select_off = l.rewrite_off + (((size_t)B * 4 + 255) & ~(size_t)255);
  l.total = l.select_off + (((size_t)B * 4 + 255) & ~(size_t)255);
  return l;
}

}  // namespace

extern "C" {

size_t fftopk_indexer_workspace_bytes(int32_t B) {
  if (B <= 0) return 0;
  return indexer_layout(B).total;
}

int fftopk_indexer_topk2048(const void* q, const void* k_cache, int64_t k_rows_per_seq, const float* w, int32_t B, int64_t L,
                            const int32_t* lengths, uint32_t* thresholds, uint32_t margin, float* logits,
                            int64_t logits_stride, int32_t* out_idx, void* d_workspace, size_t workspace_bytes,
                            uint32_t* status, void* cuda_stream) {
  if (B < 0 || L < 0 || k_rows_per_seq < L || logits_stride < L) return FFTOPK_EINVAL;
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
  rc = make_map(&map_q, q, (uint64_t)B * kIdxHeads, kIdxDim, kIdxHeads);
  if (rc) return rc;
  rc = make_map(&map_k, k_cache, (uint64_t)B * (uint64_t)k_rows_per_seq, kIdxDim, kIdxTile);
  if (rc) return rc;

  IndexerParams p;
  memset(&p, 0, sizeof(p));
  p.w = w;
  p.lengths = lengths;
  p.k_rows_per_seq = k_rows_per_seq;
  p.B = B;
  p.L = L;
  p.logits = logits;
  p.logits_stride = logits_stride;
  p.guess = thresholds;
  p.margin = margin;
  p.cand_idx = reinterpret_cast<int32_t*>(ws + lay.idx_off);
  p.cand_key = reinterpret_cast<uint32_t*>(ws + lay.key_off);
  p.cand_count = reinterpret_cast<uint32_t*>(ws + lay.count_off);
  p.status = status;
  uint32_t* rewrite_rows = reinterpret_cast<uint32_t*>(ws + lay.rewrite_off);
  uint32_t* select_rows = reinterpret_cast<uint32_t*>(ws + lay.select_off);

  // empty candidate lists (index -1), counts and marks zero
  e = cudaMemsetAsync(ws + lay.idx_off, 0xff, lay.key_off, stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(ws + lay.count_off, 0, lay.total - lay.count_off, stream);
  if (e != cudaSuccess) return cuda_fail(e);

  const int64_t ntiles = (L + kIdxTile - 1) / kIdxTile;
  int per_row = sms / B > 0 ? sms / B : 1;
  if (per_row > ntiles) per_row = (int)ntiles;
  const dim3 grid((unsigned)per_row, (unsigned)B);
  // pass 1: rows with a guess are filtered as their logits are produced; the others get logits
  indexer_logits_kernel<<<grid, kIdxThreads, indexer_smem_bytes(), stream>>>(map_q, map_k, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  // decide per row; rows whose guess held are finished here
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)B * kIdxCandShards, 1, 1);
    cfg.blockDim = dim3(512, 1, 1);
    cfg.dynamicSmemBytes = finish_smem_bytes();
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = kIdxCandShards;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, indexer_finish_kernel<512>, (const int32_t*)p.cand_idx, (const uint32_t*)p.cand_key,
                           (const uint32_t*)p.cand_count, (const uint32_t*)thresholds, lengths, (int)B, out_idx, thresholds,
                           rewrite_rows, select_rows, status);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  // pass 2 (marked rows only): write the logits the first pass did not
  IndexerParams p2 = p;
  p2.only_rows = rewrite_rows;
  indexer_logits_kernel<<<grid, kIdxThreads, indexer_smem_bytes(), stream>>>(map_q, map_k, p2);
  e = cudaGetLastError();
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
  c.only_rows = select_rows;
  c.may_overlap = false;
  return launch_select(c);
}

}  // extern "C"
