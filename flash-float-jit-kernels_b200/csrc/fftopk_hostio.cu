// Host-buffer entry point of the top-2048 selector: the caller's logits, lengths and result live
// in host memory (the situation of a CPU-side caller of the reference's op that keeps its score
// matrix in pinned memory, benchmark/bench_topk.py style). Everything is enqueued on one stream:
//   1. the VALID prefix of every row, and nothing else, comes to the device - the kernel never
//      reads beyond the lengths, so the padding of a ragged batch (half of the bytes of a padded
//      [B, L] matrix on average) never crosses PCIe. From pinned memory one gather kernel reads
//      the prefixes straight out of host memory (the device can address pinned memory) with
//      megabytes of loads in flight: one launch, where one cudaMemcpyAsync per row was measured
//      at ~13 us per copy (0.86 ms for 64 rows, slower than copying the padded matrix whole).
//      Pageable memory takes the copy-per-row path.
//   2. the selection kernel (fftopk_select2048),
//   3. the device -> host copy of the indices.
// The device staging area is the caller's: no allocation here.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fftopk.h"
#include "fftopk_host.h"
#include "fftopk_internal.h"

namespace {

constexpr size_t kAlign = 256;
inline size_t align_up(size_t v) { return (v + kAlign - 1) & ~(kAlign - 1); }

struct HostLayout {
  size_t score_off, len_off, out_off, status_off, total;
  int64_t row_stride;  // floats
};

HostLayout host_layout(int32_t B, int64_t L) {
  HostLayout h;
  h.row_stride = (L + 3) & ~(int64_t)3;  // rows start 16-byte aligned
  h.score_off = 0;
  h.len_off = align_up((size_t)B * (size_t)h.row_stride * 4);
  h.out_off = h.len_off + align_up((size_t)B * 4);
  h.status_off = h.out_off + align_up((size_t)B * 2048 * 4);
  h.total = h.status_off + kAlign;
  return h;
}

// Row b's valid prefix from host memory into the staging matrix. grid = (chunks, B).
__global__ void __launch_bounds__(256) gather_rows_kernel(const float* __restrict__ h, int64_t h_stride,
                                                         float* __restrict__ d, int64_t d_stride,
                                                         const int32_t* __restrict__ lengths, int64_t L) {
  const int b = blockIdx.y;
  int64_t len = lengths[b];
  len = len < 0 ? 0 : (len > L ? L : len);
  const float* src = h + (int64_t)b * h_stride;
  float* dst = d + (int64_t)b * d_stride;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) {  // (dst rows are 16-byte aligned by layout)
    const int64_t n4 = len >> 2;
    const float4* s4 = reinterpret_cast<const float4*>(src);
    float4* d4 = reinterpret_cast<float4*>(dst);
    int64_t i = t;
    for (; i + 3 * step < n4; i += 4 * step) {  // four loads in flight per thread
      const float4 a = s4[i], b4 = s4[i + step], c = s4[i + 2 * step], e = s4[i + 3 * step];
      d4[i] = a;
      d4[i + step] = b4;
      d4[i + 2 * step] = c;
      d4[i + 3 * step] = e;
    }
    for (; i < n4; i += step) d4[i] = s4[i];
    for (int64_t j = (n4 << 2) + t; j < len; j += step) dst[j] = src[j];
  } else {
    for (int64_t j = t; j < len; j += step) dst[j] = src[j];
  }
}

// Read-only bandwidth probe: all threads of the grid walk the buffer together, 128 bits per load,
// eight independent loads in flight per thread, wrapping around until `rounds` rounds are done.
// Loads bypass L1 (ld.global.cg), so a buffer that fits in L2 measures L2 read bandwidth and a
// buffer much larger than L2 measures HBM read bandwidth. The XOR of everything read goes to
// `sink` so that no load can be dropped.
__global__ void __launch_bounds__(1024) read_probe_kernel(const uint4* __restrict__ buf, uint32_t n16, uint32_t rounds,
                                                         uint32_t* __restrict__ sink) {
  constexpr int U = 8;
  const uint32_t nthreads = gridDim.x * blockDim.x;
  uint32_t idx = (blockIdx.x * blockDim.x + threadIdx.x) % n16;
  const uint32_t step = nthreads % n16;
  uint32_t acc = 0u;
  for (uint32_t r = 0; r < rounds; ++r) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                   : "l"(buf + idx));
      idx += step;
      if (idx >= n16) idx -= n16;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) acc ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
  }
  if (acc == 0x9e3779b9u) *sink = acc;  // (practically never true; keeps the loads alive)
}

// The address under which the device sees a host buffer, or nullptr if it cannot (pageable memory).
const float* device_view_of_host(const float* h) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, h) != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  if (attr.type != cudaMemoryTypeHost || attr.devicePointer == nullptr) return nullptr;
  return static_cast<const float*>(attr.devicePointer);
}

}  // namespace

extern "C" {

size_t fftopk_host_workspace_bytes(int32_t B, int64_t L) {
  if (B <= 0 || L < 0) return 0;
  return host_layout(B, L).total;
}

int fftopk_select2048_host(const float* h_score, int64_t h_row_stride, int32_t B, int64_t L, const int32_t* h_lengths,
                           int32_t* h_out_idx, void* d_workspace, size_t workspace_bytes, uint32_t* d_status,
                           void* cuda_stream) {
  if (B < 0 || L < 0 || h_row_stride < 0) return FFTOPK_EINVAL;
  if (B == 0) return FFTOPK_OK;
  if (!h_score || !h_lengths || !h_out_idx || !d_workspace) return FFTOPK_EINVAL;
  if (L > (int64_t)0x7fffffff - 8) return FFTOPK_ERANGE;
  const HostLayout h = host_layout(B, L);
  if (workspace_bytes < h.total || (reinterpret_cast<uintptr_t>(d_workspace) & (kAlign - 1)) != 0) return FFTOPK_EINVAL;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  char* ws = static_cast<char*>(d_workspace);
  float* d_score = reinterpret_cast<float*>(ws + h.score_off);
  int32_t* d_len = reinterpret_cast<int32_t*>(ws + h.len_off);
  int32_t* d_out = reinterpret_cast<int32_t*>(ws + h.out_off);

  cudaError_t err = cudaMemcpyAsync(d_len, h_lengths, (size_t)B * 4, cudaMemcpyHostToDevice, stream);
  if (err != cudaSuccess) return fftopk::cuda_fail(err);
  const float* hv = B <= 65535 ? device_view_of_host(h_score) : nullptr;  // (grid.y limit)
  if (hv) {
    const int chunks = (int)((L + 32767) / 32768 < 1 ? 1 : ((L + 32767) / 32768 > 64 ? 64 : (L + 32767) / 32768));
    gather_rows_kernel<<<dim3((unsigned)chunks, (unsigned)B), 256, 0, stream>>>(hv, h_row_stride, d_score, h.row_stride,
                                                                               d_len, L);
    err = cudaGetLastError();
    if (err != cudaSuccess) return fftopk::cuda_fail(err);
  } else {
    // pageable memory: one copy per row; neighbouring whole rows of an unpadded matrix merge
    int32_t b = 0;
    while (b < B) {
      int64_t len = h_lengths[b];
      len = len < 0 ? 0 : (len > L ? L : len);
      if (len == 0) {
        ++b;
        continue;
      }
      int32_t e = b + 1;
      if (len == L && h_row_stride == L && h.row_stride == L) {
        while (e < B && h_lengths[e] >= L) ++e;
      }
      const size_t bytes = (e - b == 1) ? (size_t)len * 4 : (size_t)(e - b) * (size_t)L * 4;
      err = cudaMemcpyAsync(d_score + (int64_t)b * h.row_stride, h_score + (int64_t)b * h_row_stride, bytes,
                            cudaMemcpyHostToDevice, stream);
      if (err != cudaSuccess) return fftopk::cuda_fail(err);
      b = e;
    }
  }
  fftopk::SelectCall c;
  c.score = d_score;
  c.row_stride = h.row_stride;
  c.B = B;
  c.L = L;
  c.lengths = d_len;
  c.out_idx = d_out;
  c.status = d_status;
  c.cuda_stream = cuda_stream;
  c.may_overlap = false;  // reads what the gather kernel / the copies enqueued above have staged
  const int rc = fftopk::launch_select(c);
  if (rc) return rc;
  err = cudaMemcpyAsync(h_out_idx, d_out, (size_t)B * 2048 * 4, cudaMemcpyDeviceToHost, stream);
  if (err != cudaSuccess) return fftopk::cuda_fail(err);
  return FFTOPK_OK;
}

int fftopk_probe_read_bandwidth(const void* d_buf, size_t bytes, size_t bytes_to_read, uint32_t* d_sink,
                                size_t* bytes_read, void* cuda_stream) {
  if (!d_buf || !d_sink || !bytes_read || bytes < 16 || (reinterpret_cast<uintptr_t>(d_buf) & 15u) != 0) return FFTOPK_EINVAL;
  if (bytes / 16 > 0x7fffffffull) return FFTOPK_ERANGE;
  int dev = 0, sms = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err == cudaSuccess) err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (err != cudaSuccess) return fftopk::cuda_fail(err);
  const uint32_t n16 = (uint32_t)(bytes / 16);
  const size_t per_round = (size_t)sms * 2 * 1024 * 8 * 16;  // two CTAs of 1024 threads per SM
  size_t rounds = (bytes_to_read + per_round - 1) / per_round;
  rounds = rounds < 1 ? 1 : (rounds > 0x7fffffffull ? 0x7fffffffull : rounds);
  read_probe_kernel<<<dim3((unsigned)sms * 2), 1024, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint4*>(d_buf), n16, (uint32_t)rounds, d_sink);
  err = cudaGetLastError();
  if (err != cudaSuccess) return fftopk::cuda_fail(err);
  *bytes_read = rounds * per_round;
  return FFTOPK_OK;
}

size_t fftopk_widen_workspace_bytes(int32_t B, int64_t L) {
  (void)B;
  (void)L;
  return 0;  // kept for callers of the first form of fftopk_select_topk_16bit, which staged fp32 copies
}

int fftopk_select_topk_16bit(const void* score16, int32_t dtype, int64_t row_stride, int32_t B, int64_t L,
                             const int32_t* lengths, const int32_t* row_starts, int32_t k, int32_t* out_idx,
                             void* d_workspace, size_t workspace_bytes, uint32_t* status, void* cuda_stream) {
  (void)d_workspace;  // not needed any more: the rows are read in their own width
  (void)workspace_bytes;
  if (dtype != FFTOPK_DTYPE_FP16 && dtype != FFTOPK_DTYPE_BF16) return FFTOPK_EINVAL;
  fftopk::SelectCall call;
  call.score = score16;
  call.dtype = dtype == FFTOPK_DTYPE_FP16 ? fftopk::kDtypeF16 : fftopk::kDtypeBF16;
  call.row_stride = row_stride;
  call.B = B;
  call.L = L;
  call.lengths = lengths;
  call.row_starts = row_starts;
  call.k = k;
  call.out_idx = out_idx;
  call.status = status;
  call.cuda_stream = cuda_stream;
  return fftopk::launch_select(call);
}

}  // extern "C"
