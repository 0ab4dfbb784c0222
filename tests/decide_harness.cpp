// Host build of the selector's decision rules (csrc/fftopk_decide.h) for the CPU tests: the same
// header the kernels include, compiled by g++ and exposed as plain C functions.
#include "fftopk_decide.h"

using namespace fftopk;

extern "C" {

uint32_t dh_key_from_bits(uint32_t bits) { return fftopk_key_from_bits(bits); }
uint32_t dh_bits_from_key(uint32_t key) { return fftopk_bits_from_key(key); }
uint32_t dh_sample_lower_rank(uint32_t k, uint32_t n_s, float len) { return sample_lower_rank(k, n_s, len); }
uint32_t dh_sample_upper_rank(uint32_t k, uint32_t n_s, float len) { return sample_upper_rank(k, n_s, len); }
int dh_sample_bin_too_coarse(uint32_t cnt, uint32_t total, float len, uint32_t k, float factor) {
  return sample_bin_too_coarse(cnt, total, len, k, factor) ? 1 : 0;
}
int dh_fine_histogram_usable(int built, uint32_t total, uint32_t group) {
  return fine_histogram_usable(built != 0, total, group) ? 1 : 0;
}
uint32_t dh_guess_key(int fine, uint32_t nibble, uint32_t bin) {
  return guess_key(guess_prefix(fine != 0, nibble, bin), fine ? 16 : 12);
}
uint32_t dh_guess_edge_bits(uint32_t gkey) { return guess_edge_bits(gkey); }
uint32_t dh_guess_low_key(uint32_t gkey) { return guess_low_key(gkey); }
int dh_sampled_attempt_ok(uint32_t over, uint32_t admitted, uint32_t k, uint32_t room) {
  return sampled_attempt_ok(over, admitted, k, room) ? 1 : 0;
}
int dh_finish_bins(void) { return kFinishBins; }
int dh_finish_shift(uint64_t lo, uint64_t focus) { return make_finish_digit(lo, focus).shift; }
int dh_finish_key_only(uint64_t lo, uint64_t focus) { return make_finish_digit(lo, focus).key_only() ? 1 : 0; }
uint32_t dh_finish_digit(uint64_t lo, uint64_t focus, uint64_t c) { return make_finish_digit(lo, focus).of(c); }
uint32_t dh_finish_digit_of_key(uint64_t lo, uint64_t focus, uint32_t key) {
  return make_finish_digit(lo, focus).of_key(key);
}
void dh_finish_bin_range(uint64_t lo, uint64_t focus, uint64_t cap, int t, uint64_t* t_lo, uint64_t* t_hi) {
  finish_bin_range(make_finish_digit(lo, focus), lo, cap, t, *t_lo, *t_hi);
}
uint64_t dh_single_key_floor(uint64_t lo, int idx_bits) { return single_key_floor(lo, idx_bits); }


// Walks every CTA's run of tiles the way the fused indexer's producer does (tile_run, tile_row_at,
// then tile_segment row after row) and adds, for every (row, row-local tile) the CTAs visit, one to
// visits[first_tile[row] + tile]. segs_out receives the number of segments each CTA went through.
// Returns 0, or a negative code when a walk leaves the table.
int dh_walk_tile_split(const uint32_t* first_tile, int rows, uint32_t ctas, uint32_t* visits, uint32_t* segs_out) {
  const uint32_t total = first_tile[rows];
  for (uint32_t c = 0; c < ctas; ++c) {
    const TileRun run = tile_run(total, ctas, c);
    if (run.g1 < run.g0 || run.g1 > total) return -1;
    uint32_t segs = 0;
    if (run.g0 < run.g1) {
      int row = tile_row_at(first_tile, rows, run.g0);
      for (uint32_t g = run.g0; g < run.g1; ++row) {
        if (row >= rows) return -2;
        int t_lo, n;
        if (!tile_segment(first_tile[row], first_tile[row + 1] - first_tile[row], g, run.g1, t_lo, n)) continue;
        if (n <= 0 || t_lo < 0 || (uint32_t)(t_lo + n) > first_tile[row + 1] - first_tile[row]) return -3;
        for (int i = 0; i < n; ++i) ++visits[first_tile[row] + (uint32_t)(t_lo + i)];
        g += (uint32_t)n;
        ++segs;
      }
    }
    segs_out[c] = segs;
  }
  return 0;
}
void dh_tile_run(uint32_t total, uint32_t ctas, uint32_t cta, uint32_t* g0, uint32_t* g1) {
  const TileRun r = tile_run(total, ctas, cta);
  *g0 = r.g0;
  *g1 = r.g1;
}

}  // extern "C"
