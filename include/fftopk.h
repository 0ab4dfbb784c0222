/*
 * fftopk.h — C ABI of the B200 (sm_100a) per-row top-2048 radix selector.
 *
 * This is the native boundary a host binds instead of the reference's pybind11
 * module `topk_indexer_radix` (jit_kernel/csrc/topk_indexer/topk_indexer_radix.cu:1252-1257),
 * whose `fast_topk(score, indices, lengths, row_starts)` takes at::Tensor objects.
 * Here every argument is a plain pointer or integer; no torch / ATen type crosses
 * the boundary.
 *
 * Conventions shared by every entry point that takes a stream:
 *   - returns 0 (FFTOPK_OK) or a negative FFTOPK_E* code; never throws;
 *   - enqueues work on `cuda_stream` (a cudaStream_t passed as void*; NULL = the
 *     legacy default stream) and returns without synchronising;
 *   - never allocates or frees device memory; every buffer is caller-owned;
 *   - all device pointers must belong to the device that is current on the
 *     calling thread;
 *   - output rows are written completely by the kernel (no -1 pre-fill needed,
 *     unlike the reference, jit_kernel/topk_indexer.py:68-70).
 */
#ifndef FFTOPK_H_
#define FFTOPK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FFTOPK_K 2048 /* k of the reference's op (TopK, topk_indexer_radix.cu:69); fftopk_select_topk takes others */

enum {
  FFTOPK_OK = 0,
  FFTOPK_EINVAL = -1,  /* bad argument (null pointer, negative size, bad stride)        */
  FFTOPK_ECUDA = -2,   /* a CUDA runtime call failed; see fftopk_last_cuda_error()      */
  FFTOPK_EDEVICE = -3, /* device is not sm_100 class or lacks cluster launch            */
  FFTOPK_ERANGE = -4,  /* size beyond what the entry point supports                     */
};

/* Bits the kernels may OR into the optional device status word. */
enum {
  FFTOPK_ST_STAGE_TIMEOUT = 1, /* fused indexer: a bounded wait on a copy / MMA barrier ran out */
  FFTOPK_ST_INTERNAL = 2,      /* an internal count did not add up (should never be seen)  */
  FFTOPK_ST_PEER_TIMEOUT = 4,  /* merge: a bounded wait on a peer's ready flag ran out      */
  FFTOPK_ST_GUESS_MISSED = 8,  /* warm start: a row's previous threshold was unusable; the row  */
                               /* was selected from scratch (informational, result is exact)   */
  FFTOPK_ST_CHECK = 16,        /* checked build (-DFFTOPK_CHECKED) only: an index the logic     */
                               /* guarantees to be in range was not; the access was skipped    */
};

/* Library version: major*10000 + minor*100 + patch. */
int fftopk_version(void);

/* Text for an FFTOPK_E* code. */
const char* fftopk_strerror(int code);

/* cudaError_t of the most recent failing CUDA call made by this library on the calling
 * thread (0 if none). */
int fftopk_last_cuda_error(void);

/*
 * Per-row top-2048 selection.
 * Replaces fast_topk_interface (topk_indexer_radix.cu:1051-1158) and topk_kernel (:854-869).
 *
 *   score        device, fp32, B rows; row b starts at score + b*row_stride (elements),
 *                inner stride 1 (reference check: topk_indexer_radix.cu:1003)
 *   row_stride   elements between consecutive rows (>= 0)
 *   B, L         rows and padded row length; B == 0 is a no-op
 *   lengths      device, int32 [B]; valid elements of row b. Values are clamped to
 *                [0, L - row_start]
 *   row_starts   device, int32 [B] or NULL; first valid element of row b
 *                (reference: topk_indexer_radix.cu:858, 541-542)
 *   out_idx      device, int32 [B, 2048]. Row b receives, in unspecified order, the indices
 *                (relative to row_starts[b]) of the 2048 largest valid elements; among equal
 *                values the lower index is selected. -0.0 compares equal to +0.0 and NaN
 *                above +inf, as torch.topk orders them. A row with len <= 2048 receives
 *                0..len-1 followed by -1 (reference: naive_topk_cuda, :152-163)
 *   out_key      device, uint32 [B, 2048] or NULL; when given, slot i receives the
 *                order-preserving radix key of the element out_idx names (0 where out_idx is
 *                -1). Used by the context-parallel merge; no reference counterpart
 *   idx_offset   added to every index written (the global position of this shard's first
 *                element in context-parallel mode; 0 otherwise)
 *   status       device, uint32 [1] or NULL; FFTOPK_ST_* bits are OR-ed in, never cleared
 */
int fftopk_select2048(const float* score, int64_t row_stride, int32_t B, int64_t L,
                      const int32_t* lengths, const int32_t* row_starts,
                      int32_t* out_idx, uint32_t* out_key, int32_t idx_offset,
                      uint32_t* status, void* cuda_stream);

/*
 * The same selection for another k: the `k` largest valid entries of every row, 1 <= k <= 4096
 * (FFTOPK_EINVAL otherwise). The reference's op is fixed at 2048 (topk_indexer.py:62-64 asserts it;
 * TopK is a compile-time constant, topk_indexer_radix.cu:69); indexer configurations with 512, 1024
 * or 4096 selected tokens need this. out_idx (and out_key) are [B, k]; rows with lengths[b] <= k
 * hold 0..len-1 followed by -1. Everything else as for fftopk_select2048.
 */
int fftopk_select_topk(const float* score, int64_t row_stride, int32_t B, int64_t L,
                       const int32_t* lengths, const int32_t* row_starts, int32_t k, int32_t* out_idx,
                       uint32_t* out_key, int32_t idx_offset, uint32_t* status, void* cuda_stream);

/*
 * fftopk_select2048 with a warm start: a decode loop calls the selector once per generated token on
 * a row that has grown by one logit, so the previous call's threshold - the key of the row's 2048-th
 * largest element - is an excellent first guess for this one. No counterpart in the reference's code;
 * its README discusses guess-and-verify selection as a competitor's idea (README.md:90-98).
 * With a guess a row skips the sample, its histograms and the cluster-wide threshold search: it is
 * filtered at once against key = prev_threshold[b] - margin, and the checks that protect a sampled
 * guess protect this one too - at least 2048 elements admitted, no candidate list overflowed. A
 * guess that fails them (too high, far too low, stale) sends the row to the full-histogram path:
 * the result is the exact top 2048, ties to the lower index, whatever the guess was, and
 * FFTOPK_ST_GUESS_MISSED is raised in the status word for information.
 *
 *   prev_threshold  device, uint32 [B] or NULL: per-row key guess (the value next_threshold received
 *                   in an earlier call, or fftopk_key_of(x) of any value x believed to be at or
 *                   below the row's 2048-th largest); 0 = no guess for that row (cold selection)
 *   margin          subtracted from every guess, in key units: 0 when the row only grew since the
 *                   guess was made (its threshold cannot have dropped); for positive fp32 values one
 *                   key unit is one ulp, so 1 << 20 lowers the guess by 12.5 % of its magnitude at most
 *   next_threshold  device, uint32 [B] or NULL: receives the key of this call's 2048-th largest
 *                   element (exact whenever the finishing pass ran; otherwise a lower bound of it;
 *                   0 for rows of at most 2048 elements). May be the same array as prev_threshold
 *   everything else as for fftopk_select2048 (no out_key / idx_offset).
 */
int fftopk_select2048_warm(const float* score, int64_t row_stride, int32_t B, int64_t L,
                           const int32_t* lengths, const int32_t* row_starts,
                           const uint32_t* prev_threshold, uint32_t margin, uint32_t* next_threshold,
                           int32_t* out_idx, uint32_t* status, void* cuda_stream);

/*
 * Selection fused with the step that follows it in a sparse-attention decode / prefill layer.
 * Replace fast_topk_transform_interface and fast_topk_transform_ragged_interface
 * (topk_indexer_radix.cu:1160-1250) with their three kernels (:871-995), which the reference
 * exports as fast_topk_transform_fused / fast_topk_transform_ragged_fused (:1255-1256). All
 * arguments shared with fftopk_select2048 mean the same.
 *
 * fftopk_select2048_page_table: dst_page_table[b, j] = table_row[idx_j], where idx_j runs over
 *   the selected indices of row b and table_row = src_page_table + i*src_stride for the request i
 *   with cu_seqlens_q[i] <= b < cu_seqlens_q[i+1] (cu_seqlens_q int32 [prefill_bs + 1], its last
 *   entry = B). cu_seqlens_q == NULL is the decode case: prefill_bs == B and i = b. Rows with
 *   len <= 2048 give table_row[0..len-1] followed by -1 (naive_topk_transform, :166-175).
 * fftopk_select2048_ragged: topk_indices_ragged[b, j] = idx_j + topk_indices_offset[b]; short rows
 *   give offset + 0..len-1 followed by -1 (naive_topk_transform_ragged, :178-184).
 */
int fftopk_select2048_page_table(const float* score, int64_t row_stride, int32_t B, int64_t L,
                                 const int32_t* lengths, const int32_t* row_starts,
                                 int32_t* dst_page_table, const int32_t* src_page_table,
                                 int64_t src_stride, const int32_t* cu_seqlens_q, int32_t prefill_bs,
                                 uint32_t* status, void* cuda_stream);
int fftopk_select2048_ragged(const float* score, int64_t row_stride, int32_t B, int64_t L,
                             const int32_t* lengths, const int32_t* row_starts,
                             int32_t* topk_indices_ragged, const int32_t* topk_indices_offset,
                             uint32_t* status, void* cuda_stream);

/*
 * Merge of per-shard candidates into the global top-2048 (context-parallel mode: every GPU
 * selected a local top-2048 over its sequence shard, the candidates were all-gathered).
 * No reference counterpart: the reference has no multi-GPU path.
 *
 *   cand_key     device, uint32 [G, B, 2048]   keys written by fftopk_select2048(out_key)
 *   cand_idx     device, int32  [G, B, 2048]   global indices (idx_offset applied); -1 = empty
 *   shard_stride elements between the planes of consecutive shards in BOTH arrays; 0 means
 *                B*2048 (dense). An all-gathered [G, 2, B, 2048] buffer (index plane, key plane
 *                per shard) is passed as cand_idx = base, cand_key = base + B*2048,
 *                shard_stride = 2*B*2048, without any repacking
 *   G            number of shards (1..8)
 *   out_idx      device, int32 [B, 2048]; the 2048 candidates largest by (key, lower index),
 *                unspecified order; -1 padded when fewer than 2048 candidates are valid
 *   out_key      device, uint32 [B, 2048] or NULL
 */
int fftopk_merge2048(const uint32_t* cand_key, const int32_t* cand_idx, int64_t shard_stride,
                     int32_t G, int32_t B, int32_t* out_idx, uint32_t* out_key, uint32_t* status,
                     void* cuda_stream);

/*
 * Fused gather-and-merge for the context-parallel mode, without a collective library call.
 * No reference counterpart. Every rank owns one "comm" buffer that its peers map through CUDA
 * IPC (NVLink peer access); a call with epoch e (1, 2, 3, ... the same on every rank) works in
 * two enqueue-only steps:
 *   fftopk_select2048_cp  local selection written into the rank's own comm buffer (half e & 1);
 *                         the last CTA of that kernel to finish fences and releases the buffer's
 *                         epoch flag;
 *   fftopk_merge2048_cp   ONE kernel per rank that waits - at most wait_ms milliseconds per
 *                         shard - until every shard's flag has reached e, pulls the candidates
 *                         out of the peers' buffers with plain loads and merges them.
 * A wait that runs out fills the row with -1, raises FFTOPK_ST_PEER_TIMEOUT in *status and lets
 * the kernel return: a peer that never publishes cannot hang the GPU. The two halves of the
 * buffer alternate, which is enough because a rank can only start call e+2 after its own merge
 * e+1 has seen every peer's flag e+1, i.e. after every peer finished reading half e.
 *
 * Set-up (these four allocate / map memory and synchronise; call them outside the hot path):
 *   fftopk_comm_create  cudaMalloc + clear a comm buffer for up to b_cap rows, export its handle
 *   fftopk_comm_open    map a peer's buffer from the 64-byte handle it exported (other process)
 *   fftopk_comm_close / fftopk_comm_destroy
 *
 *   comms        HOST array of G device pointers, shard order: comms[g] is rank g's comm buffer
 *                (the rank's own pointer for itself, fftopk_comm_open results for the peers)
 *   own          this rank's position in comms
 *   epoch        1, 2, 3, ... chosen by the host, or 0 in BOTH calls for device-side epochs: the
 *                selection then increments the buffer's own flag and the kernels derive the
 *                epoch and the buffer half from it, so the select / publish / merge sequence has no
 *                per-call host argument and a captured CUDA graph of it can be replayed
 */
int fftopk_comm_bytes(int32_t b_cap, size_t* bytes);
int fftopk_comm_create(int32_t b_cap, void** comm, unsigned char handle[64]);
int fftopk_comm_open(const unsigned char handle[64], void** peer_comm);
int fftopk_comm_close(void* peer_comm);
int fftopk_comm_destroy(void* comm);
int fftopk_select2048_cp(const float* score, int64_t row_stride, int32_t B, int64_t L,
                         const int32_t* lengths, int32_t idx_offset, void* comm, int32_t b_cap,
                         uint32_t epoch, uint32_t* status, void* cuda_stream);
int fftopk_merge2048_cp(void* const* comms, int32_t G, int32_t own, int32_t B, int32_t b_cap,
                        uint32_t epoch, int32_t wait_ms, int32_t* out_idx, uint32_t* out_key,
                        uint32_t* status, void* cuda_stream);

/*
 * The context-parallel call as ONE launch per GPU: local selection, exchange and merge in the same
 * kernel. No reference counterpart. The cluster that selects a row's local top 2048 pushes them, as
 * soon as the row is selected, into the comm buffer of every GPU as self-validating packets
 * {index, epoch, key, epoch} - plain 16-byte stores over NVLink, no flag, no fence; CTA g of the
 * cluster then polls - in its own GPU's memory, for at most wait_ms - the packets shard g sent for
 * the row, and the cluster merges the G lists into out_idx. There is no second launch, no
 * collective library call and no launch-wide synchronisation; a peer that never sends gives -1
 * rows and FFTOPK_ST_PEER_TIMEOUT, never a hang.
 *
 *   score, row_stride, B, L, lengths, idx_offset   this rank's slice, as for fftopk_select2048_cp
 *   comms, G, own, b_cap, epoch, wait_ms           as for fftopk_merge2048_cp (epoch 0: a counter
 *                per row in the buffer itself, so a captured graph can be replayed). The call uses
 *                regions of the comm buffers that the two-call sequence does not touch and keeps
 *                its own epoch count: both kinds of call may be used on the same buffers
 *   out_idx      device, int32 [B, 2048]: the global indices of the row's 2048 largest entries
 * Returns FFTOPK_ERANGE - and enqueues nothing - when the launch plan for (B, L) gives a row fewer
 * CTAs than there are shards (large batches of short slices); use the two-call sequence then. The
 * answer depends only on B, L, G and the device, so all ranks of a homogeneous job get the same one.
 */
int fftopk_topk2048_cp(const float* score, int64_t row_stride, int32_t B, int64_t L,
                       const int32_t* lengths, int32_t idx_offset, void* const* comms, int32_t G,
                       int32_t own, int32_t b_cap, uint32_t epoch, int32_t wait_ms, int32_t* out_idx,
                       uint32_t* status, void* cuda_stream);

/*
 * Top-2048 by column slices, with no allocation anywhere. (This entry point has no counterpart in
 * the reference.)
 *
 * For callers that are not allowed to obtain device memory when the call is made: a serving
 * process that handed every free byte of HBM to its KV-cache pool at start-up, or a real-time loop
 * in which cudaMalloc - which may block until the whole device is idle - is forbidden. It runs the
 * same kernels as fftopk_select2048_cp + fftopk_merge2048_cp (each row is cut into `slices`
 * column ranges, a local top-2048 is selected per range, one merge kernel picks the final 2048),
 * but the per-slice candidates and lengths sit in a scratch array that is compiled into the
 * library as a device global, instead of in buffers from fftopk_comm_create. The function calls
 * neither cudaMalloc nor cudaFree nor any allocating library routine.
 *
 *   score, row_stride, B, L, lengths, out_idx, status, cuda_stream: as for fftopk_select2048
 *   (row_starts is not supported); out_idx receives the same index set fftopk_select2048 gives.
 *   slices       1..8 column ranges per row
 * Limits: B <= 8 and slices <= 8 (the built-in scratch is 1 MiB + 256 bytes per GPU, held by
 * every GPU that loads the library until the process exits); larger values return FFTOPK_ERANGE.
 * The first call on a device looks up the scratch array's device address (cudaGetSymbolAddress);
 * make that first call before any stream capture. All calls on a device share the one array, which
 * keeps the previous call's contents (every slot a call reads is rewritten by that call first,
 * nothing needs clearing): two calls whose kernels overlap on the GPU - different streams, or one
 * stream per thread - race on it and return garbage. Serialise them.
 */
int fftopk_topk2048_sliced_noalloc(const float* score, int64_t row_stride, int32_t B, int64_t L,
                                   const int32_t* lengths, int32_t slices, int32_t* out_idx,
                                   uint32_t* status, void* cuda_stream);

/*
 * fftopk_select_topk for fp16 or bf16 scores (the reference's op takes fp32 only: CHECK of the
 * dtype, topk_indexer_radix.cu:1003-1016; it sketches a 16-bit key map and leaves it disabled,
 * :192-195). The same kernel instantiated on the 16-bit type: the row is read ONCE, in its own
 * width (8-byte granules of four elements), and every element is widened to fp32 - exactly and
 * order-preserving - in registers, so keys, ties and results are those of the fp32 selector on the
 * widened values. row_stride is in elements; score16 must be 2-byte aligned.
 * d_workspace / workspace_bytes are ignored and may be NULL / 0 (an earlier form of this entry
 * point staged fp32 copies of the rows there; fftopk_widen_workspace_bytes now returns 0).
 */
#define FFTOPK_DTYPE_FP16 0
#define FFTOPK_DTYPE_BF16 1
size_t fftopk_widen_workspace_bytes(int32_t B, int64_t L);
int fftopk_select_topk_16bit(const void* score16, int32_t dtype, int64_t row_stride, int32_t B, int64_t L,
                             const int32_t* lengths, const int32_t* row_starts, int32_t k,
                             int32_t* out_idx, void* d_workspace, size_t workspace_bytes,
                             uint32_t* status, void* cuda_stream);

/*
 * The selector for a caller whose buffers are in HOST memory: score, lengths and the result.
 * Replaces, for such a caller, the tensor.cuda() / fast_topk_v3 / .cpu() sequence of the
 * reference's benchmark driver (benchmark/bench_topk.py:90-146) with one call that enqueues, on
 * `cuda_stream`: host->device copies of the valid prefix of each row ONLY (lengths are read on the
 * host; the padding of a ragged batch never crosses PCIe), fftopk_select2048, and the
 * device->host copy of the indices. Returns once everything is enqueued; synchronise the stream
 * before reading h_out_idx. Use pinned host memory for asynchronous copies.
 *
 *   h_score, h_row_stride, B, L, h_lengths   as for fftopk_select2048, but host pointers
 *   h_out_idx      [B, 2048] int32, host
 *   d_workspace    device staging area of at least fftopk_host_workspace_bytes(B, L) bytes,
 *                  256-byte aligned; owned by the caller (nothing is allocated here)
 *   d_status       optional device status word, as for fftopk_select2048
 */
size_t fftopk_host_workspace_bytes(int32_t B, int64_t L);
int fftopk_select2048_host(const float* h_score, int64_t h_row_stride, int32_t B, int64_t L,
                           const int32_t* h_lengths, int32_t* h_out_idx, void* d_workspace,
                           size_t workspace_bytes, uint32_t* d_status, void* cuda_stream);

/*
 * The step in FRONT of the selector, fused with it: indexer logits computed on the tensor cores and
 * selected as they are produced. No counterpart in the reference, which starts from a finished fp32
 * logit matrix (jit_kernel/topk_indexer.py:42-75; README.md:24 names the step).
 *   logit[b, t] = sum over 64 heads h of  w[b, h] * relu( q[b, h, :] . k[b, t, :] ),  dimension 128, bf16
 * One kernel (TMA loads, tcgen05.mma into TMEM, one key per epilogue thread) produces the logits of a
 * row; for a row with a threshold guess (thresholds[b] != 0: what an earlier call handed back) every
 * logit is compared with the guess as it leaves the tensor core and the few that pass are kept as
 * candidates - the logit matrix is written (4 bytes per key beside the 256 read) but not read again -
 * and the last CTA of the row to finish selects the exact top 2048 of the candidates. Rows without
 * a guess, and rows whose guess did not hold (fewer than 2048 admitted, or more than the 8,192-entry
 * candidate list takes; status bit FFTOPK_ST_GUESS_MISSED), go through the selector of
 * fftopk_select2048 on `logits` (a second launch, enqueued as a programmatic dependent, that costs
 * rows in no need of it an empty CTA). Either way out_idx holds the exact top 2048 OF THE LOGITS THE KERNEL COMPUTED
 * (fp32 accumulation on the tensor cores; ties to the lower index) and thresholds[b] the key of the
 * row's 2048-th largest logit for the next call.
 *   q            device, bf16 [B, 64, 128], 16-byte aligned
 *   k_cache      device, bf16 [B, k_rows_per_seq, 128] (k_rows_per_seq >= L), 16-byte aligned
 *   w            device, fp32 [B, 64]
 *   lengths      device, int32 [B]: valid keys per row (clamped to [0, L])
 *   thresholds   device, uint32 [B], in and out (start with zeros); margin as for fftopk_select2048_warm
 *   logits       device, fp32 [B, logits_stride] (logits_stride >= L), out: logits[b, t] for t < lengths[b]
 *   out_idx      device, int32 [B, 2048]
 *   d_workspace  fftopk_indexer_workspace_bytes(B) bytes of device memory, 256-byte aligned, ZERO-FILLED
 *                before its first use; every call leaves it ready for the next one (calls with any
 *                B' <= B may share it), so no call contains a memset
 * Enqueue-only on `cuda_stream`; the first call on a device sets kernel attributes (make it outside
 * any stream capture). B <= 65535.
 */
size_t fftopk_indexer_workspace_bytes(int32_t B);
/* The same for fp8 (e4m3) operands, the storage format of the key cache this indexer was designed
 * around: q [B, 64, 128] and k_cache [B, k_rows_per_seq, 128] are one byte per element (half the
 * HBM traffic of the bf16 form), accumulation is fp32. k_scale, when given, is a device fp32 array
 * [B, k_scale_stride] (k_scale_stride >= L) with one POSITIVE scale per key, multiplied into the
 * key's finished logit (relu(s x) = s relu(x)); a scale of q belongs in w. */
int fftopk_indexer_topk2048_fp8(const void* q, const void* k_cache, int64_t k_rows_per_seq,
                                const float* k_scale, int64_t k_scale_stride, const float* w, int32_t B,
                                int64_t L, const int32_t* lengths, uint32_t* thresholds, uint32_t margin,
                                float* logits, int64_t logits_stride, int32_t* out_idx, void* d_workspace,
                                size_t workspace_bytes, uint32_t* status, void* cuda_stream);
int fftopk_indexer_topk2048(const void* q, const void* k_cache, int64_t k_rows_per_seq, const float* w,
                            int32_t B, int64_t L, const int32_t* lengths, uint32_t* thresholds,
                            uint32_t margin, float* logits, int64_t logits_stride, int32_t* out_idx,
                            void* d_workspace, size_t workspace_bytes, uint32_t* status,
                            void* cuda_stream);

/*
 * Measurement aid, not part of the selection path (no reference counterpart): a read-only bandwidth
 * probe. One kernel in which every SM reads the buffer with 128-bit loads that bypass L1, wrapping
 * around until about `bytes_to_read` bytes have been read in total; *bytes_read receives the exact
 * count. Timed by the caller (CUDA events around the call). A buffer that fits in L2 (a few MiB)
 * gives the L2 read bandwidth of the device - the roof of a selection whose row is L2-resident,
 * the regime a CUDA-graph replay over one buffer measures - and a buffer several times the L2
 * size gives the HBM read bandwidth.
 *   d_buf   device, 16-byte aligned, `bytes` bytes (>= 16), any contents
 *   d_sink  device, uint32 [1], scratch the kernel may write
 */
int fftopk_probe_read_bandwidth(const void* d_buf, size_t bytes, size_t bytes_to_read, uint32_t* d_sink,
                                size_t* bytes_read, void* cuda_stream);

/*
 * Radix key of one fp32 value, computed on the host with the same function the kernels use
 * (the order-preserving map the reference defines as convert_to_uint32,
 * topk_indexer_radix.cu:206-209, plus -0.0 / NaN canonicalisation). For tests and bindings.
 */
uint32_t fftopk_key_of(float x);

/*
 * Launch-plan introspection and overrides (experiments and tests; not needed in production).
 * fftopk_plan reports what fftopk_select2048 would launch for (B, L) on the current device:
 * plan[0] = CTAs per cluster (= CTAs per row), plan[1] = threads per CTA,
 * plan[2] = dynamic shared memory bytes, plan[3] = per-CTA candidate-list capacity,
 * plan[4] = gathered-candidate capacity of the cluster's first CTA, plan[5] = SM count.
 * fftopk_set_tuning overrides the automatic choice process-wide; pass -1 (0 for the flag) to
 * restore "auto". force_full_histogram = 1 skips the sample-and-filter path, so that every row
 * takes the full-histogram path (tests).
 * Replaces the reference's compile-time split heuristic (topk_indexer_radix.cu:1081-1111).
 */
int fftopk_plan(int32_t B, int64_t L, int32_t plan[6]);
/*
 * Back-to-back calls. Every selection launch is a programmatic dependent launch and lets its own
 * dependents become resident at once. By default the kernel executes griddepcontrol.wait before
 * its first access to global memory: plain stream order - the kernel in front of it has completed
 * and its writes are visible - and only the launch latency of a call hides behind the call in
 * front of it. Overlap (off by default; process-wide): with enable = 1 the kernel does NOT wait,
 * so when two selection kernels follow each other on a stream the second starts filling SMs as
 * soon as CTAs of the first exit (short rows finish early), instead of waiting for the whole
 * grid. Enable it only if (1) no kernel that precedes a call on the
 * stream hands over unfinished inputs through programmatic launch completion, and (2) calls that
 * may overlap do not share an output buffer. Kernels of other libraries around the calls keep
 * normal stream ordering. No reference counterpart.
 */
int fftopk_set_overlap(int32_t enable);
int fftopk_set_tuning(int32_t cluster_ctas, int32_t threads, int32_t list_cap, int32_t cand_cap,
                      int32_t force_full_histogram);

#ifdef __cplusplus
}
#endif
#endif /* FFTOPK_H_ */
