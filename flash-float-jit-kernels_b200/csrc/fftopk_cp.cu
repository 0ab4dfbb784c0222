// Context-parallel side of the top-2048 selector: the candidate merge, and a fused
// gather-and-merge over peer memory that needs no collective library call.
//
// Every GPU selects a local top-2048 over its slice of the sequence (fftopk_select2048 with keys
// and a global index offset). The global top-2048 is contained in the union of the local ones, so
// one cluster per row - one CTA per shard - pulls the G*2048 (key, global index) candidates,
// drops those below the largest of the shards' own 2048-th keys, and its first CTA runs the same
// single-CTA finish the selector uses on what is left.
//
//  * fftopk_merge2048: candidates already gathered into local memory (NCCL all-gather).
//  * fftopk_merge2048_cp: every rank published its candidates in a buffer its peers have mapped
//    (CUDA IPC over NVLink) - the selection kernel's last CTA releases the buffer's epoch flag -
//    and the merge kernel itself waits - bounded - for each shard's flag and pulls the shard's
//    candidates with plain loads. Gather and merge are one kernel; there is no multicast load and
//    no library kernel that touches peer memory.
//
// No reference counterpart: the reference has no multi-GPU path.
#include <cooperative_groups.h>
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

constexpr int kMergeThreads = 512;

// Publishes an epoch without a selection in front of it (a call with no rows): fences and
// releases the flag. Selections publish by themselves (last CTA of select2048_kernel).
__global__ void publish_kernel(uint32_t* flag, uint32_t epoch) {
  if (epoch == 0u) epoch = __ldcg(flag) + 1u;  // device-side epochs: the next one
  __threadfence_system();
  st_release_sys(flag, epoch);
}

// One cluster per row, one CTA per shard (see merge_row).
template <int NT>
__global__ void __launch_bounds__(NT, 1) merge2048_kernel(const MergeSrc src, int G, int B,
                                                         int32_t* __restrict__ out_idx_all,
                                                         uint32_t* __restrict__ out_key_all, uint32_t* status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  MergeSmem sm;
  sm.hist = reinterpret_cast<uint32_t*>(smem_raw);
  sm.sup = sm.hist + 2 * kMaxBins;
  sm.xch = sm.sup + 2 * kSup;
  sm.ctrl = reinterpret_cast<Ctrl*>(sm.xch + kMaxCluster * kSup);
  sm.cand = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(sm.ctrl) + ((sizeof(Ctrl) + 127) & ~127u));
  sm.cand_cap = G * kK;
  cg::cluster_group cluster = cg::this_cluster();
  const int g = G == 1 ? 0 : (int)cluster.block_rank();
  const int row = (int)(blockIdx.x / (unsigned)G);
  // device-side epochs: this rank's own flag already holds the epoch of this call (its selection
  // published earlier on the same stream)
  const uint32_t epoch = (src.epoch == 0u && src.own_flag != nullptr) ? __ldcg(src.own_flag) : src.epoch;
  const int64_t half_shift = src.own_flag != nullptr && src.epoch == 0u ? (int64_t)(epoch & 1u) * src.half_words : 0;
  merge_row<NT>(cluster, G, G, g, sm, src.idx[g] + half_shift + (int64_t)row * kK, src.key[g] + half_shift + (int64_t)row * kK,
                src.flag[g], nullptr, epoch, src.wait_ns, out_idx_all + (int64_t)row * kK,
                out_key_all ? out_key_all + (int64_t)row * kK : nullptr, status);
}

// ---------------------------------------------------------------------------------------------
// Scratch for the allocation-free entry point (fftopk_topk2048_sliced_noalloc): the per-slice
// candidates and the per-slice lengths live in this file-scope array instead of a buffer from
// cudaMalloc. Every GPU that loads the library holds these bytes until the process exits.
// In HOST code the name below is only a stand-in for the symbol, never a device address: the
// address is fetched once per device with cudaGetSymbolAddress (static_scratch_ptr).
// ---------------------------------------------------------------------------------------------
constexpr int kStaticMaxRows = 8;
constexpr int kStaticMaxSlices = 8;
constexpr size_t kStaticCandWords = (size_t)kStaticMaxSlices * 2 * kStaticMaxRows * kK;  // 262,144 words = 1 MiB
constexpr size_t kStaticLenWords = (size_t)kStaticMaxSlices * kStaticMaxRows;            // 64 words
constexpr size_t kStaticBytes = (kStaticCandWords + kStaticLenWords) * 4;                // 1 MiB + 256 B
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

// Valid length of every (slice, row): how much of row b falls into columns [g*ls, g*ls + lg).
__global__ void slice_lengths_kernel(const int32_t* __restrict__ lengths, int B, int slices, int64_t L, int64_t ls,
                                     int32_t* __restrict__ out /* [slices][kStaticMaxRows] */) {
  const int i = threadIdx.x;
  if (i < slices * kStaticMaxRows) {
    const int g = i / kStaticMaxRows, b = i % kStaticMaxRows;
    int64_t v = 0;
    if (b < B) {
      int64_t lg = L - g * ls < ls ? L - g * ls : ls;  // columns of slice g (0 when the slice starts beyond L)
      lg = lg < 0 ? 0 : lg;
      int64_t len = lengths[b];
      len = len < 0 ? 0 : (len > L ? L : len);
      v = len - g * ls;
      v = v < 0 ? 0 : (v > lg ? lg : v);
    }
    out[i] = (int32_t)v;
  }
}

}  // namespace fftopk

#ifdef FFTOPK_CHECKED
namespace fftopk {
int checked_read_merge(uint32_t rec[4]) {
  const uint32_t zero[4] = {0u, 0u, 0u, 0u};
  cudaError_t e = cudaMemcpyFromSymbol(rec, g_check_rec, sizeof(zero));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_check_rec, zero, sizeof(zero));
  return e == cudaSuccess ? 0 : cuda_fail(e);
}
}  // namespace fftopk
#endif

namespace {
using namespace fftopk;

DeviceOnce g_merge_once[kMaxDevices];

// First call on a device (any thread): the merge kernel's shared-memory attribute.
int merge_setup() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= kMaxDevices) return FFTOPK_EDEVICE;
  return g_merge_once[dev].run([&] {
    int optin = 0;
    cudaError_t e2 = cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    if (e2 != cudaSuccess) return cuda_fail(e2);
    e2 = cudaFuncSetAttribute(merge2048_kernel<kMergeThreads>, cudaFuncAttributeMaxDynamicSharedMemorySize, optin);
    if (e2 != cudaSuccess) return cuda_fail(e2);
    return 0;
  });
}

size_t merge_smem(int G) {
  return (size_t)(2 * kMaxBins + 2 * kSup + kMaxCluster * kSup) * 4 + ((sizeof(Ctrl) + 127) & ~(size_t)127) +
         (size_t)G * kK * 8;
}

// One cluster of G CTAs per row.
int launch_merge(const MergeSrc& src, int G, int B, int32_t* out_idx, uint32_t* out_key, uint32_t* status,
                 cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)B * (unsigned)G, 1, 1);
  cfg.blockDim = dim3(kMergeThreads, 1, 1);
  cfg.dynamicSmemBytes = merge_smem(G);
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = (unsigned)G;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, merge2048_kernel<kMergeThreads>, src, G, B, out_idx, out_key, status);
  if (e != cudaSuccess) return cuda_fail(e);
  return FFTOPK_OK;
}

// comm buffer layout, in 32-bit words, for a row capacity of b_cap:
// see CommLayout (fftopk_internal.h)
size_t comm_words(int32_t b_cap) { return comm_total_words(b_cap); }

// Device address of g_static_scratch on the current device, looked up once per device.
void* g_static_ptr[kMaxDevices];
DeviceOnce g_static_once[kMaxDevices];

int static_scratch_ptr(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= kMaxDevices) return FFTOPK_EDEVICE;
  const int rc = g_static_once[dev].run([&] {
    void* p = nullptr;
    cudaError_t e2 = cudaGetSymbolAddress(&p, g_static_scratch);  // with device `dev` current
    if (e2 != cudaSuccess) return cuda_fail(e2);
    if (p == nullptr) return (int)FFTOPK_EDEVICE;
    g_static_ptr[dev] = p;
    return 0;
  });
  if (rc) return rc;
  *out = g_static_ptr[dev];
  return 0;
}

}  // namespace

extern "C" {

int fftopk_merge2048(const uint32_t* cand_key, const int32_t* cand_idx, int64_t shard_stride, int32_t G, int32_t B,
                     int32_t* out_idx, uint32_t* out_key, uint32_t* status, void* cuda_stream) {
  if (B < 0 || G < 1 || shard_stride < 0) return FFTOPK_EINVAL;
  if (G > kMaxShards) return FFTOPK_ERANGE;
  if (B == 0) return FFTOPK_OK;
  if (!cand_key || !cand_idx || !out_idx) return FFTOPK_EINVAL;
  if (shard_stride == 0) shard_stride = (int64_t)B * kK;
  int rc = merge_setup();
  if (rc) return rc;
  MergeSrc src;
  memset(&src, 0, sizeof(src));
  for (int g = 0; g < G; ++g) {
    src.idx[g] = cand_idx + (int64_t)g * shard_stride;
    src.key[g] = cand_key + (int64_t)g * shard_stride;
  }
  return launch_merge(src, G, B, out_idx, out_key, status, static_cast<cudaStream_t>(cuda_stream));
}

int fftopk_comm_bytes(int32_t b_cap, size_t* bytes) {
  if (b_cap < 1 || !bytes) return FFTOPK_EINVAL;
  *bytes = comm_words(b_cap) * 4;
  return FFTOPK_OK;
}

int fftopk_comm_create(int32_t b_cap, void** comm, unsigned char handle[64]) {
  if (b_cap < 1 || !comm || !handle) return FFTOPK_EINVAL;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, comm_words(b_cap) * 4);
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaMemset(p, 0, comm_words(b_cap) * 4);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return cuda_fail(e);
  }
  memcpy(handle, &h, 64);
  *comm = p;
  return FFTOPK_OK;
}

int fftopk_comm_open(const unsigned char handle[64], void** peer_comm) {
  if (!handle || !peer_comm) return FFTOPK_EINVAL;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  cudaError_t e = cudaIpcOpenMemHandle(peer_comm, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return cuda_fail(e);
  return FFTOPK_OK;
}

int fftopk_comm_close(void* peer_comm) {
  if (!peer_comm) return FFTOPK_EINVAL;
  cudaError_t e = cudaIpcCloseMemHandle(peer_comm);
  if (e != cudaSuccess) return cuda_fail(e);
  return FFTOPK_OK;
}

int fftopk_comm_destroy(void* comm) {
  if (!comm) return FFTOPK_EINVAL;
  cudaError_t e = cudaFree(comm);
  if (e != cudaSuccess) return cuda_fail(e);
  return FFTOPK_OK;
}

int fftopk_select2048_cp(const float* score, int64_t row_stride, int32_t B, int64_t L, const int32_t* lengths,
                         int32_t idx_offset, void* comm, int32_t b_cap, uint32_t epoch, uint32_t* status,
                         void* cuda_stream) {
  if (!comm || b_cap < 1 || B < 0 || B > b_cap) return FFTOPK_EINVAL;
  uint32_t* flag = reinterpret_cast<uint32_t*>(static_cast<int32_t*>(comm) + (size_t)4 * b_cap * kK);
  const int64_t half = (int64_t)2 * b_cap * kK;
  if (B > 0) {
    SelectCall c;
    c.score = score;
    c.row_stride = row_stride;
    c.B = B;
    c.L = L;
    c.lengths = lengths;
    c.idx_offset = idx_offset;
    c.status = status;
    c.cuda_stream = cuda_stream;
    c.may_overlap = false;  // the publish kernel and the peers' merges consume this launch's output
    // host-side epoch: the half is known here; device-side epoch (0): the kernel picks the half
    // from the flag it finds
    int32_t* base = static_cast<int32_t*>(comm) + (epoch != 0u ? (size_t)(epoch & 1u) * half : 0);
    c.out_idx = base;
    c.out_key = reinterpret_cast<uint32_t*>(base + (size_t)b_cap * kK);
    if (epoch == 0u) {
      c.cp_flag = flag;
      c.cp_half_words = half;
    }
    c.cp_publish = flag;  // the selection's last CTA fences and releases the epoch flag
    c.cp_epoch = epoch;
    return launch_select(c);
  }
  // no rows: the epoch still has to advance
  publish_kernel<<<1, 1, 0, static_cast<cudaStream_t>(cuda_stream)>>>(flag, epoch);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  return FFTOPK_OK;
}

int fftopk_merge2048_cp(void* const* comms, int32_t G, int32_t own, int32_t B, int32_t b_cap, uint32_t epoch,
                        int32_t wait_ms, int32_t* out_idx, uint32_t* out_key, uint32_t* status, void* cuda_stream) {
  if (!comms || G < 1 || B < 0 || b_cap < 1 || B > b_cap || wait_ms < 0 || own < 0 || own >= G) return FFTOPK_EINVAL;
  if (G > kMaxShards) return FFTOPK_ERANGE;
  if (B == 0) return FFTOPK_OK;
  if (!out_idx) return FFTOPK_EINVAL;
  int rc = merge_setup();
  if (rc) return rc;
  MergeSrc src;
  memset(&src, 0, sizeof(src));
  for (int g = 0; g < G; ++g) {
    if (!comms[g]) return FFTOPK_EINVAL;
    const int32_t* words = static_cast<const int32_t*>(comms[g]);
    const int32_t* base = words + (epoch != 0u ? (size_t)(epoch & 1u) * 2 * b_cap * kK : 0);
    src.idx[g] = base;
    src.key[g] = reinterpret_cast<const uint32_t*>(base + (size_t)b_cap * kK);
    src.flag[g] = reinterpret_cast<const uint32_t*>(words + (size_t)4 * b_cap * kK);
  }
  src.epoch = epoch;
  src.own_flag = src.flag[own];
  src.half_words = (int64_t)2 * b_cap * kK;
  src.wait_ns = (unsigned long long)wait_ms * 1000000ull;
  return launch_merge(src, G, B, out_idx, out_key, status, static_cast<cudaStream_t>(cuda_stream));
}

int fftopk_topk2048_cp(const float* score, int64_t row_stride, int32_t B, int64_t L, const int32_t* lengths,
                       int32_t idx_offset, void* const* comms, int32_t G, int32_t own, int32_t b_cap, uint32_t epoch,
                       int32_t wait_ms, int32_t* out_idx, uint32_t* status, void* cuda_stream) {
  SelectCall c;
  c.score = score;
  c.row_stride = row_stride;
  c.B = B;
  c.L = L;
  c.lengths = lengths;
  c.idx_offset = idx_offset;
  c.status = status;
  c.cuda_stream = cuda_stream;
  return launch_select_merge(c, comms, G, own, b_cap, epoch, wait_ms, out_idx);
}

int fftopk_topk2048_sliced_noalloc(const float* score, int64_t row_stride, int32_t B, int64_t L,
                                   const int32_t* lengths, int32_t slices, int32_t* out_idx, uint32_t* status,
                                   void* cuda_stream) {
  if (B < 0 || L < 0 || row_stride < 0 || slices < 1) return FFTOPK_EINVAL;
  if (B > kStaticMaxRows || slices > kStaticMaxSlices) return FFTOPK_ERANGE;  // beyond the built-in scratch
  if (B == 0) return FFTOPK_OK;
  if (!score || !lengths || !out_idx) return FFTOPK_EINVAL;
  if (L > (int64_t)0x7fffffff - 8) return FFTOPK_ERANGE;
  void* scratch = nullptr;
  int rc = static_scratch_ptr(&scratch);  // first call on a device: cudaGetSymbolAddress
  if (rc) return rc;
  rc = merge_setup();
  if (rc) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  int32_t* cand = static_cast<int32_t*>(scratch);
  int32_t* slice_len = cand + kStaticCandWords;
  const int64_t ls = (L + slices - 1) / slices;  // columns per slice (the last one may be shorter)
  slice_lengths_kernel<<<1, kStaticMaxSlices * kStaticMaxRows, 0, stream>>>(lengths, B, slices, L, ls, slice_len);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  MergeSrc src;
  memset(&src, 0, sizeof(src));
  for (int g = 0; g < slices; ++g) {
    int32_t* idx_plane = cand + (size_t)g * 2 * kStaticMaxRows * kK;
    uint32_t* key_plane = reinterpret_cast<uint32_t*>(idx_plane + (size_t)kStaticMaxRows * kK);
    const int64_t first = (int64_t)g * ls;
    const int64_t lg = L - first < ls ? (L - first > 0 ? L - first : 0) : ls;
    // every slot of the slice's planes is rewritten by this call: nothing has to start at zero
    SelectCall c;
    c.score = score + (lg > 0 ? first : 0);
    c.row_stride = row_stride;
    c.B = B;
    c.L = lg;
    c.lengths = slice_len + (size_t)g * kStaticMaxRows;
    c.out_idx = idx_plane;
    c.out_key = key_plane;
    c.idx_offset = (int32_t)first;
    c.status = status;
    c.cuda_stream = cuda_stream;
    c.may_overlap = false;  // reads the slice lengths written by the kernel enqueued just above
    rc = launch_select(c);
    if (rc) return rc;
    src.idx[g] = idx_plane;
    src.key[g] = key_plane;
  }
  return launch_merge(src, slices, B, out_idx, nullptr, status, stream);
}

}  // extern "C"
