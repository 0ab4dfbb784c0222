// Order-preserving fp32 -> uint32 radix key, shared by device code and host code.
//
// key(x) >= key(y)  <=>  x >= y under torch.topk's ordering: -0.0 == +0.0, every NaN is
// larger than +inf and all NaNs are equal. Any most-significant-digit slice of the key is
// therefore monotone: bin(x) >= bin(y) whenever x >= y.
//
// The reference defines the plain sign-flip map (convert_to_uint32,
// jit_kernel/csrc/topk_indexer/topk_indexer_radix.cu:206-209) but bins with
// floor(x) mod 256 instead (:198-204), which is only monotone on [0, 256).
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define FFTOPK_HD __host__ __device__ __forceinline__
#else
#define FFTOPK_HD static inline
#endif

FFTOPK_HD uint32_t fftopk_key_from_bits(uint32_t bits) {
  // NaN (exponent all ones, mantissa non-zero) -> the largest key.
  if ((bits & 0x7fffffffu) > 0x7f800000u) return 0xffffffffu;
  // -0.0 -> +0.0
  if (bits == 0x80000000u) bits = 0u;
  // negative: flip all bits; non-negative: set the sign bit.
  const uint32_t mask = (uint32_t)((int32_t)bits >> 31) | 0x80000000u;
  return bits ^ mask;
}

// Inverse on canonical keys (NaN comes back as one quiet NaN pattern).
FFTOPK_HD uint32_t fftopk_bits_from_key(uint32_t key) {
  if (key == 0xffffffffu) return 0x7fc00000u;
  const uint32_t mask = (key & 0x80000000u) ? 0x80000000u : 0xffffffffu;
  return key ^ mask;
}
