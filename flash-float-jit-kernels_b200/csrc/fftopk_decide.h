// Decision rules of the selector that do not depend on where they run: the sample-rank bounds,
// the choice between the two sample histograms, the float edge of a key guess, the digit rule of
// the finish and the conditions under which the sampled attempt is abandoned. The kernels call
// these functions; a host compiler can compile them too (tests drive them with generated inputs
// where no GPU is present).
#pragma once
#include <math.h>
#include <stdint.h>

#include "fftopk_key.h"

#if defined(__CUDACC__)
#define FFTOPK_DECIDE_HD __host__ __device__ __forceinline__
#else
#define FFTOPK_DECIDE_HD inline
#endif

namespace fftopk {

constexpr int kFinishBits = 11;  // digit width of the single-CTA finish
constexpr int kFinishBins = 1 << kFinishBits;

FFTOPK_DECIDE_HD int clz64(uint64_t v) {
#if defined(__CUDA_ARCH__)
  return __clzll((long long)v);
#else
  return v ? __builtin_clzll(v) : 64;
#endif
}

// ---------------------------------------------------------------------------------------------
// Sample ranks. A row of `len` elements is sampled at n_s positions; m = k * n_s / len of the
// sample are expected among the row's k largest. The element of sample rank
//     lower_rank = m + 5 sqrt(m) + 14   (capped at n_s)
// is, except with probability of the order 1e-6, not larger than the row's k-th largest: filtering
// with it admits at least k elements. The mirror image,
//     upper_rank = m - 5 sqrt(m) - 14   (0 when there is no such rank),
// is a sample element the k-th largest does not exceed with the same confidence.
// ---------------------------------------------------------------------------------------------
FFTOPK_DECIDE_HD uint32_t sample_lower_rank(uint32_t k, uint32_t n_s, float len) {
  const float m = (float)k * (float)n_s / len;
  const uint32_t rk = (uint32_t)(m + 5.0f * sqrtf(m) + 14.0f);
  return rk < n_s ? rk : n_s;
}

FFTOPK_DECIDE_HD uint32_t sample_upper_rank(uint32_t k, uint32_t n_s, float len) {
  const float m = (float)k * (float)n_s / len;
  const float rk = m - 5.0f * sqrtf(m) - 14.0f;
  return rk >= 1.0f ? (uint32_t)rk : 0u;
}

// A second sample round sharpens the guess when the guessed bin alone would admit more than
// factor * k row elements (estimated from the bin's share of the sample).
FFTOPK_DECIDE_HD bool sample_bin_too_coarse(uint32_t bin_count, uint32_t sample_total, float len, uint32_t k,
                                            float factor) {
  const float in_bin = (float)bin_count * len / (float)(sample_total ? sample_total : 1u);
  return in_bin > factor * (float)k;
}

// The finer sample histogram (key bits [27:16]) may replace the coarse one (bits [31:20]) only if
// one group of four consecutive coarse super-bins - one value of the key's top four bits - holds
// the whole sample.
FFTOPK_DECIDE_HD bool fine_histogram_usable(bool built, uint32_t sample_total, uint32_t group_total) {
  return built && sample_total > 0u && group_total == sample_total;
}

// Key guess from a bin: prefix of pbits bits (12: the coarse bin; 16: top nibble, then the fine bin).
FFTOPK_DECIDE_HD uint32_t guess_prefix(bool fine, uint32_t top_nibble, uint32_t bin) {
  return fine ? ((top_nibble << 12) | bin) : bin;
}
FFTOPK_DECIDE_HD uint32_t guess_key(uint32_t prefix, int pbits) { return prefix << (32 - pbits); }

// Lower edge of a key guess as float bits: key(x) >= gkey <=> !(x < edge), NaN included. Keys
// outside the range that real values map to (below -inf's key, above +inf's) give -inf: the filter
// then admits everything, which only lengthens the lists.
FFTOPK_DECIDE_HD bool guess_has_edge(uint32_t gkey) { return gkey > 0x007fffffu && gkey <= 0xff800000u; }
FFTOPK_DECIDE_HD uint32_t guess_edge_bits(uint32_t gkey) {
  return guess_has_edge(gkey) ? fftopk_bits_from_key(gkey) : 0xff800000u;
}
// ... and the smallest key the filter can then admit (what the finish may assume as its lower bound)
FFTOPK_DECIDE_HD uint32_t guess_low_key(uint32_t gkey) { return guess_has_edge(gkey) ? gkey : 0u; }

// After the filter: keep the sampled attempt only if no list overflowed, at least k elements were
// admitted and they fit where they were gathered; otherwise the full-histogram path takes over.
FFTOPK_DECIDE_HD bool sampled_attempt_ok(uint32_t overflowed, uint32_t admitted, uint32_t k, uint32_t room) {
  return overflowed == 0u && admitted >= k && admitted <= room;
}

// ---------------------------------------------------------------------------------------------
// Digit rule of a finish round over the composite range [lo, cap]: digit(c) = min((c - lo) >>
// shift, kFinishBins - 1). The shift is chosen so that [lo, focus] spreads over the bins below the
// last one; everything above `focus` (cap >= focus >= lo) lands in the last bin. With focus == cap
// this is a plain radix digit of the range; a caller that knows where in the range the threshold
// will fall passes a tighter focus and gets finer bins there.
// ---------------------------------------------------------------------------------------------
struct FinishDigit {
  uint64_t lo;
  int shift;
  FFTOPK_DECIDE_HD uint32_t of(uint64_t c) const {
    const uint64_t d = (c - lo) >> shift;
    return d < (uint64_t)(kFinishBins - 1) ? (uint32_t)d : (uint32_t)(kFinishBins - 1);
  }
  // the same for a digit that depends on the key alone (shift >= 32 and the low word of lo is 0)
  FFTOPK_DECIDE_HD uint32_t of_key(uint32_t k) const {
    const uint32_t d = (k - (uint32_t)(lo >> 32)) >> (shift - 32);
    return d < (uint32_t)(kFinishBins - 1) ? d : (uint32_t)(kFinishBins - 1);
  }
  FFTOPK_DECIDE_HD bool key_only() const { return shift >= 32 && (uint32_t)lo == 0u; }
};

FFTOPK_DECIDE_HD FinishDigit make_finish_digit(uint64_t lo, uint64_t focus) {
  const uint64_t width = focus - lo;
  const int bits = width ? 64 - clz64(width) : 0;
  int shift = bits > kFinishBits ? bits - kFinishBits : 0;
  if ((width >> shift) >= (uint64_t)(kFinishBins - 1)) ++shift;  // keep the last bin for what lies above
  return FinishDigit{lo, shift};
}

// Composite range of finish bin t under digit rule dg over [lo, cap].
FFTOPK_DECIDE_HD void finish_bin_range(const FinishDigit& dg, uint64_t lo, uint64_t cap, int t, uint64_t& t_lo,
                                       uint64_t& t_hi) {
  t_lo = lo + ((uint64_t)t << dg.shift);
  t_hi = (t == kFinishBins - 1) ? cap : t_lo + ((1ull << dg.shift) - 1ull);
  if (t_hi > cap || t_hi < t_lo) t_hi = cap;
}

// When a round has narrowed the range to one key, every composite there starts its low word with
// the same run of ones (indices are < 2^idx_bits and stored inverted): the smallest possible one.
FFTOPK_DECIDE_HD uint64_t single_key_floor(uint64_t lo, int idx_bits) {
  return (lo & 0xffffffff00000000ull) | (uint64_t)(~((idx_bits >= 32 ? 0u : (1u << idx_bits)) - 1u));
}

// ---------------------------------------------------------------------------------------------
// Work split of the fused indexer's producer. The tiles of all rows, row after row, form one
// sequence of `total` tiles; first_tile[r] (r <= rows) is the number of tiles of the rows before r.
// CTA c of `ctas` takes the run [g0, g1): total = each * ctas + rest, and the first `rest` CTAs
// take one tile more. The part of a run inside one row is a segment.
// ---------------------------------------------------------------------------------------------
struct TileRun {
  uint32_t g0, g1;
};
FFTOPK_DECIDE_HD TileRun tile_run(uint32_t total, uint32_t ctas, uint32_t cta) {
  const uint32_t each = total / ctas, rest = total % ctas;
  const uint32_t g0 = cta * each + (cta < rest ? cta : rest);
  return TileRun{g0, g0 + each + (cta < rest ? 1u : 0u)};
}
// the last row that starts at or before tile g (rows >= 1)
FFTOPK_DECIDE_HD int tile_row_at(const uint32_t* first_tile, int rows, uint32_t g) {
  int lo = 0, hi = rows;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (first_tile[mid] <= g) lo = mid; else hi = mid;
  }
  return lo;
}
// Segment of the run [g, g1) inside a row that starts at tile row_g0 and has ntiles tiles: the
// first row-local tile and the tile count; false if the row has no tile at or behind g.
FFTOPK_DECIDE_HD bool tile_segment(uint32_t row_g0, uint32_t ntiles, uint32_t g, uint32_t g1, int& t_lo, int& n) {
  if (row_g0 + ntiles <= g) return false;
  const uint32_t end = g1 < row_g0 + ntiles ? g1 : row_g0 + ntiles;
  t_lo = (int)(g - row_g0);
  n = (int)(end - g);
  return true;
}

}  // namespace fftopk
