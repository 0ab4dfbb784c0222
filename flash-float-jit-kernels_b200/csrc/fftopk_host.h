// Host-side helpers shared by the translation units of libfftopk.so.
#pragma once
#include <cuda_runtime.h>

#include "../../include/fftopk.h"

namespace fftopk {

// cudaError_t of the last failing runtime call on this thread (fftopk_last_cuda_error()).
inline thread_local int g_last_cuda_error = 0;

inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = (int)e;
  return FFTOPK_ECUDA;
}

}  // namespace fftopk
