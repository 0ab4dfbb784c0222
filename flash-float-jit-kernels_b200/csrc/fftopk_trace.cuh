// Phase timestamps for debugging (compiled in only with -DFFTOPK_TRACE; the production build
// turns every mark into nothing).
#pragma once
#include <stdint.h>
namespace fftopk {
#ifdef FFTOPK_TRACE
// Debug build only: phase timestamps (ns, %globaltimer) of row 0 / rank 0 / thread 0.
__device__ unsigned long long g_trace[32];
__device__ __forceinline__ void trace_mark(int slot, bool who) {
  if (who) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_trace[slot] = t;
  }
}
#define FFTOPK_MARK(slot) trace_mark((slot), blockIdx.x == 0 && threadIdx.x == 0)
#else
#define FFTOPK_MARK(slot) ((void)0)
#endif
}  // namespace fftopk
