// Phase timestamps for debugging (compiled in only with -DFFTOPK_TRACE; the production build
// turns every mark into nothing and exports neither function below). Thread 0 of block 0 appends
// (id, %globaltimer) pairs to a log, which a -DFFTOPK_TRACE build of the library hands out through
//   int fftopk_trace_read(unsigned long long times[128], int ids[128], int* n);
//   int fftopk_trace_clear(void);
// (both return a cudaError_t). A trace build changes no result.
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
#else
#define FFTOPK_MARK(id) ((void)0)
#endif
}  // namespace fftopk
