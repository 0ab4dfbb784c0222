// Interfaces shared by the translation units of libfftopk.so that are not part of the C ABI.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <atomic>
#include <mutex>

namespace fftopk {

// One selection launch. Every public selection entry point fills one of these and calls
// launch_select(); the composite entry points (host buffers, 16-bit scores, column slices,
// context-parallel publication) do the same from their own translation units.
enum : int { kDtypeF32 = 0, kDtypeF16 = 1, kDtypeBF16 = 2 };

struct SelectCall {
  const void* score = nullptr;  // elements of `dtype`
  int dtype = kDtypeF32;
  int64_t row_stride = 0;
  int32_t B = 0;
  int64_t L = 0;
  const int32_t* lengths = nullptr;
  const int32_t* row_starts = nullptr;
  int32_t* out_idx = nullptr;
  uint32_t* out_key = nullptr;
  int32_t idx_offset = 0;
  uint32_t* status = nullptr;
  void* cuda_stream = nullptr;
  int32_t k = 2048;
  // fused output transforms
  const int32_t* src_page_table = nullptr;
  int64_t src_stride = 0;
  const int32_t* cu_seqlens_q = nullptr;
  int32_t prefill_bs = 0;
  const int32_t* row_offsets = nullptr;
  // context-parallel publication (see SelectParams in fftopk_select.cu)
  const uint32_t* cp_flag = nullptr;
  int64_t cp_half_words = 0;
  uint32_t* cp_publish = nullptr;  // flag line of the comm buffer: the launch's last CTA releases it
  uint32_t cp_epoch = 0;
  // warm start (fftopk_select2048_warm): per-row key guesses in, this call's threshold keys out
  const uint32_t* prev_threshold = nullptr;
  uint32_t* next_threshold = nullptr;
  uint32_t warm_margin = 0;
  const uint32_t* only_rows = nullptr;  // with next_threshold: select only rows whose entry is non-zero
  // false: this launch consumes what a kernel enqueued just before it by the library itself has
  // produced (gathered rows, widened scores, slice lengths, indexer logits), or hands its output to
  // a kernel the library enqueues right after it. Such a launch keeps stream order whatever
  // fftopk_set_overlap says: it executes griddepcontrol.wait like every launch in the default mode
  // (a programmatic dependent launch that does not has no guarantee that its predecessor's writes
  // are visible).
  bool may_overlap = true;
};

int launch_select(const SelectCall& c);
// selection + exchange + merge in one launch (context-parallel mode); uses score, row_stride, B, L,
// lengths, idx_offset, status and cuda_stream of `c`
int launch_select_merge(const SelectCall& c, void* const* comms, int32_t G, int32_t own, int32_t b_cap, uint32_t epoch,
                        int32_t wait_ms, int32_t* out_idx);

// Once-per-device set-up slots (function attributes, symbol addresses): the first caller on a
// device runs `init` under a lock, everybody else sees `ready` with acquire semantics.
struct DeviceOnce {
  std::atomic<bool> ready{false};
  std::mutex mu;
  template <class F>
  int run(F&& init) {
    if (ready.load(std::memory_order_acquire)) return 0;
    std::lock_guard<std::mutex> lock(mu);
    if (ready.load(std::memory_order_relaxed)) return 0;
    const int rc = init();
    if (rc == 0) ready.store(true, std::memory_order_release);
    return rc;
  }
};

constexpr int kMaxDevices = 64;

// Layout of a context-parallel comm buffer for up to b_cap rows, in 32-bit words (K = 2048):
//   two-launch protocol (fftopk_select2048_cp / fftopk_merge2048_cp)
//     [half 0: index plane b_cap*K | key plane b_cap*K][half 1: the same]
//     [epoch flag peers poll: one 128-byte line][arrival counter of the publishing launch: one line]
//   single-launch protocol (fftopk_topk2048_cp)
//     [epoch counter of every row: one line each]
//     [local selection output: index plane b_cap*K | key plane b_cap*K]
//     [inbox: 2 halves x 8 source shards x b_cap rows x K packets of 4 words]
// The two protocols use disjoint regions and separate epoch counts.
constexpr int kCommFlagWords = 64;
constexpr int kCommArriveWord = 32;
constexpr int kCommRowFlagWords = 32;
constexpr int kCommMaxShards = 8;
constexpr int kCommK = 2048;
inline size_t comm_rowflag_offset(int32_t b_cap) { return (size_t)4 * b_cap * kCommK + kCommFlagWords; }
inline size_t comm_stage_offset(int32_t b_cap) { return comm_rowflag_offset(b_cap) + (size_t)b_cap * kCommRowFlagWords; }
inline size_t comm_inbox_offset(int32_t b_cap) { return comm_stage_offset(b_cap) + (size_t)2 * b_cap * kCommK; }
inline size_t comm_inbox_half_words(int32_t b_cap) { return (size_t)kCommMaxShards * b_cap * kCommK * 4; }
inline size_t comm_total_words(int32_t b_cap) { return comm_inbox_offset(b_cap) + 2 * comm_inbox_half_words(b_cap); }

#ifdef FFTOPK_CHECKED
int checked_read_merge(uint32_t rec[4]);  // fftopk_cp.cu's copy of the violation record; clears it
#endif

}  // namespace fftopk
