// The per-row softmax arithmetic of the FP8 attention kernels (pytorch-labs/helion
// examples/fp8_attention.py:74-94) on 128 scores held in one thread's registers: row max, p = exp2(s*c - m) on
// packed pairs, row sum from the fp32 values, e4m3 pack.  Shared by the two-tile attention kernel and by the
// softmax-only ceiling kernel, so that the ceiling is measured on the instruction stream the kernel runs.
#pragma once

#include "common.cuh"

namespace hb {

// max over the 128 scores of a row: 3-input max, four independent chains
__device__ __forceinline__ float row_max128(const uint32_t (&s)[4][32]) {
  float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      mx0 = fmax3(mx0, __uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
      mx1 = fmax3(mx1, __uint_as_float(s[c][i + 2]), __uint_as_float(s[c][i + 3]));
      mx2 = fmax3(mx2, __uint_as_float(s[c][i + 4]), __uint_as_float(s[c][i + 5]));
      mx3 = fmax3(mx3, __uint_as_float(s[c][i + 6]), __uint_as_float(s[c][i + 7]));
    }
  }
  return fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
}

// scores at or beyond `valid` (keys that do not exist, or that the row may not see) count as -inf
__device__ __forceinline__ void mask_scores128(uint32_t (&s)[4][32], int valid) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if (c * 32 + i >= valid) s[c][i] = __float_as_uint(-INFINITY);
    }
  }
}

// One 32-score chunk (chunk index c of the row): p = exp2(s*scale - m) for every score, both running pair
// sums updated from the fp32 values, and the 32 e4m3 codes packed four to a word.  Of every eight pairs,
// POLY_OF8 take the degree-5 polynomial on the FMA pipes (exp2_pair_poly5, as accurate as ex2.approx) and
// the others the MUFU unit.
template <int POLY_OF8>
__device__ __forceinline__ void exp_chunk32(const uint32_t (&s)[32], int c, uint64_t c2, uint64_t negm2, uint64_t& sum_a,
                                            uint64_t& sum_b, uint32_t (&packed)[8]) {
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    const int pair0 = (c * 32 + i) / 2;
    const uint64_t t0 = ffma2(pack2(s[i], s[i + 1]), c2, negm2);
    const uint64_t t1 = ffma2(pack2(s[i + 2], s[i + 3]), c2, negm2);
    const uint64_t p0 = (pair0 % 8) < POLY_OF8 ? exp2_pair_poly5(t0) : exp2_pair_mufu(t0);
    const uint64_t p1 = ((pair0 + 1) % 8) < POLY_OF8 ? exp2_pair_poly5(t1) : exp2_pair_mufu(t1);
    sum_a = fadd2(sum_a, p0);
    sum_b = fadd2(sum_b, p1);
    uint32_t a0, a1, b0, b1;
    unpack2(p0, a0, a1);
    unpack2(p1, b0, b1);
    packed[i / 4] = pack_e4m3x4(__uint_as_float(a0), __uint_as_float(a1), __uint_as_float(b0), __uint_as_float(b1));
  }
}

}  // namespace hb
