// Output scaling shared by the GEMM epilogues (fp8_gemm.cu, fp8_gemm_skinny.cu).
#pragma once

#include "common.cuh"
#include "host.h"

namespace hb {

// Optional output scaling of the GEMM epilogues: out = cast((acc * a) * b), the multiplications in
// fp32 in that order.  mode 0: none.  mode 1: a and b point to one float each (per-tensor scales).
// mode 2: a has one float per row of out, b one per column (row-wise scales).
struct EpiScale {
  const float* a;
  const float* b;
  int mode;
};

// Scales 32 consecutive columns [col0, col0 + 32) of one output row held as fp32 bit patterns.
__device__ __forceinline__ void scale_chunk(uint32_t (&r)[32], const EpiScale& sc, int row, int M, int col0, int N) {
  if (sc.mode == 0) return;
  if (sc.mode == 1) {
    const float sa = __ldg(sc.a), sb = __ldg(sc.b);
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint((__uint_as_float(r[i]) * sa) * sb);
  } else {
    const float sa = row < M ? __ldg(sc.a + row) : 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float sb = col0 + i < N ? __ldg(sc.b + col0 + i) : 0.0f;
      r[i] = __float_as_uint((__uint_as_float(r[i]) * sa) * sb);
    }
  }
}

inline EpiScale epi_scale(const GemmArgs& a) { return EpiScale{a.scale_a, a.scale_b, a.scale_mode}; }

}  // namespace hb
