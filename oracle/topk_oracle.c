/*
 * CPU oracle for the per-row top-2048 selector.  TEST INFRASTRUCTURE ONLY: nothing in the
 * product path may call, link or import this file; it exists so that tests, the smoke check
 * and the CPU-baseline leg of the benchmark have something to compare the CUDA path with.
 *
 * What it restates, and from where:
 *   - the contract of the reference op: indices of the k largest valid entries of every row,
 *     relative to row_starts, rows with len <= k hold 0..len-1 then -1
 *     (jit_kernel/topk_indexer.py:42-75; jit_kernel/csrc/topk_indexer/topk_indexer_radix.cu:152-163
 *     for short rows, :541-542 and :600 for the row_starts offset);
 *   - the reference's own ground truth for "largest": torch.topk(score[:, :len], k, sorted=False)
 *     (benchmark/bench_topk.py:25-42), compared as index sets with equal-value swaps allowed
 *     (benchmark/bench_topk.py:55-87).  torch.topk's arithmetic lives in PyTorch, a third-party
 *     dependency that is not part of the reference tree (pinned there as torch==2.8.0,
 *     requirements/common.txt:6; 2.11.0 in this image).  Its ordering is restated here as a
 *     total order on fp32: -0.0 == +0.0, NaN above +inf, and - because torch leaves ties
 *     unspecified while this build fixes them - the lower index first among equal values;
 *   - oracle_ref_floor_radix: the reference kernel's own selection scheme, an 8-bit
 *     floor(x) bin followed by rounds that peel 8 fractional bits with (x - bin) * 256
 *     (topk_indexer_radix.cu:198-204, 541-548, 555-566, 634-635, 695-705), written as plain
 *     scalar C.  It is only defined for inputs in [0, 256), the domain the reference's benchmark
 *     normalises to (benchmark/bench_topk.py:101-104).
 *
 * Pinning: tests/golden holds index sets produced by torch.topk / torch.sort(stable) on seeded
 * inputs in this image (tests/golden/make_golden.py); tests/test_oracle.py checks both functions
 * below against them.  The reference itself ships no golden vectors for this path.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* Order-preserving key (the map the reference defines as convert_to_uint32,
 * topk_indexer_radix.cu:206-209) with torch's -0.0 / NaN conventions. */
uint32_t oracle_key_of(float x) {
  uint32_t bits;
  memcpy(&bits, &x, 4);
  if ((bits & 0x7fffffffu) > 0x7f800000u) return 0xffffffffu;
  if (bits == 0x80000000u) bits = 0u;
  return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

static int cmp_desc_u64(const void* a, const void* b) {
  const uint64_t x = *(const uint64_t*)a, y = *(const uint64_t*)b;
  return (x < y) - (x > y);
}

/*
 * One row.  row: len valid values.  out: k int32.  Returns 0, or -1 on allocation failure.
 * len <= k: identity layout.  Otherwise the k largest under (value desc, index asc), written in
 * that order (callers compare as sets).
 */
int oracle_topk_row(const float* row, int32_t len, int32_t k, int32_t* out) {
  if (len <= k) {
    for (int32_t i = 0; i < k; ++i) out[i] = i < len ? i : -1;
    return 0;
  }
  uint64_t* c = (uint64_t*)malloc((size_t)len * sizeof(uint64_t));
  if (!c) return -1;
  for (int32_t i = 0; i < len; ++i) c[i] = ((uint64_t)oracle_key_of(row[i]) << 32) | (uint64_t)(~(uint32_t)i);
  qsort(c, (size_t)len, sizeof(uint64_t), cmp_desc_u64);
  for (int32_t i = 0; i < k; ++i) out[i] = (int32_t)(~(uint32_t)c[i]);
  free(c);
  return 0;
}

/* Batched form with the op's full signature (row_starts may be NULL). */
int oracle_topk(const float* score, int64_t row_stride, int32_t B, int64_t L, const int32_t* lengths,
                const int32_t* row_starts, int32_t k, int32_t* out) {
  for (int32_t b = 0; b < B; ++b) {
    int64_t rs = row_starts ? row_starts[b] : 0;
    if (rs < 0) rs = 0;
    if (rs > L) rs = L;
    int64_t len = lengths[b];
    if (len < 0) len = 0;
    if (len > L - rs) len = L - rs;
    if (oracle_topk_row(score + (int64_t)b * row_stride + rs, (int32_t)len, k, out + (int64_t)b * k)) return -1;
  }
  return 0;
}

/*
 * The reference kernel's selection scheme on one row with values in [0, 256).
 * Round 0 bins by floor(x); each later round rescales the survivors' fractional part by 256 and
 * bins by its floor, exactly as the device code does in fp32.  After `max_rounds` refinement
 * rounds (the kernel runs at most 4) the remaining ties are taken in index order.
 * Returns the number of indices written (k), or -1 on failure.
 */
int oracle_ref_floor_radix(const float* row, int32_t len, int32_t k, int32_t max_rounds, int32_t* out) {
  if (len <= k) {
    for (int32_t i = 0; i < k; ++i) out[i] = i < len ? i : -1;
    return k;
  }
  float* val = (float*)malloc((size_t)len * sizeof(float));
  int32_t* idx = (int32_t*)malloc((size_t)len * sizeof(int32_t));
  if (!val || !idx) {
    free(val);
    free(idx);
    return -1;
  }
  int32_t n = len, nout = 0, need = k;
  for (int32_t i = 0; i < len; ++i) {
    val[i] = row[i];
    idx[i] = i;
  }
  for (int32_t round = 0; round <= max_rounds && need > 0; ++round) {
    int32_t hist[256] = {0};
    for (int32_t i = 0; i < n; ++i) hist[(uint8_t)(int)floorf(val[i])]++;
    /* suffix sums S[b] = sum_{j>=b} hist[j]; threshold bin t: S[t] > need >= S[t+1] */
    int32_t above = 0, t = 255;
    for (t = 255; t >= 0; --t) {
      if (above + hist[t] >= need) break; /* equivalently S[t] >= need; S[t] == need keeps all */
      above += hist[t];
    }
    if (t < 0) t = 0;
    int32_t m = 0;
    for (int32_t i = 0; i < n; ++i) {
      const int32_t b = (uint8_t)(int)floorf(val[i]);
      if (b > t) {
        out[nout++] = idx[i];
      } else if (b == t) {
        val[m] = (val[i] - (float)b) * 256.0f; /* next 8 fractional bits, exact in fp32 */
        idx[m] = idx[i];
        ++m;
      }
    }
    need = k - nout;
    n = m;
    if (n == need) break;
  }
  for (int32_t i = 0; i < n && nout < k; ++i) out[nout++] = idx[i]; /* leftovers: index order */
  free(val);
  free(idx);
  return nout;
}
