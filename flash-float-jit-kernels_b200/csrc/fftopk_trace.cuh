// Phase timestamps for debugging (compiled in only with -DFFTOPK_TRACE; the production build
// turns every mark into nothing). Thread 0 of block 0 appends (id, %globaltimer) pairs to a log.
#pragma once
#include <stdint.h>
namespace fftopk {
#ifdef FFTOPK_TRACE
constexpr int kTraceCap = 128;
static __device__ unsigned long long g_trace_t[kTraceCap];
static __device__ int g_trace_id[kTraceCap];
static __device__ int g_trace_n;
__device__ __forceinline__ void trace_mark(int id, bool who) {
  if (who) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    const int i = g_trace_n;
    if (i < kTraceCap) {
      g_trace_t[i] = t;
      g_trace_id[i] = id;
      g_trace_n = i + 1;
    }
  }
}
#define FFTOPK_MARK(id) trace_mark((id), blockIdx.x == 0 && threadIdx.x == 0)
#elif defined(FFTOPK_STOP_AFTER)
// Instruction-count experiments: the kernel body returns at mark FFTOPK_STOP_AFTER (only marks
// placed directly in a kernel of one-CTA clusters make sense here; results are then garbage).
#define FFTOPK_MARK(id) do { if ((id) == FFTOPK_STOP_AFTER) return; } while (0)
#else
#define FFTOPK_MARK(id) ((void)0)
#endif
}  // namespace fftopk
