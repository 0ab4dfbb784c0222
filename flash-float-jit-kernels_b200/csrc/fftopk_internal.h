// Interfaces shared by the translation units of libfftopk.so that are not part of the C ABI.
#pragma once
#include <stdint.h>

#include <atomic>
#include <mutex>

namespace fftopk {

// One selection launch. Every public selection entry point fills one of these and calls
// launch_select(); the composite entry points (host buffers, 16-bit scores, column slices,
// context-parallel publication) do the same from their own translation units.
struct SelectCall {
  const float* score = nullptr;
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
  // false: this launch consumes what a kernel enqueued just before it by the library itself has
  // produced (gathered rows, widened scores, slice lengths), or hands its output to a kernel the
  // library enqueues right after it. Such a launch keeps plain stream order whatever
  // fftopk_set_overlap says: a programmatic dependent launch that never executes
  // griddepcontrol.wait has no guarantee that its predecessor's writes are visible.
  bool may_overlap = true;
};

int launch_select(const SelectCall& c);

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

#ifdef FFTOPK_CHECKED
int checked_read_merge(uint32_t rec[4]);  // fftopk_cp.cu's copy of the violation record; clears it
#endif

}  // namespace fftopk
