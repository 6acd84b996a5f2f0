// Output scaling shared by the GEMM epilogues (fp8_gemm.cu, fp8_gemm_skinny.cu).
#pragma once

#include "common.cuh"
#include "host.h"

namespace hb {

// Optional output scaling of the GEMM epilogues: out = cast((acc * a) * b), the multiplications in
// fp32 in that order.  mode 0: none.  mode 1: a and b point to one float each (per-tensor scales).
// mode 2: a has one float per row of out, b one per column (row-wise scales).
// Then, optionally, `+ bias[column]` (fp32, one per column of out) and `max(., 0)`: the two epilogues
// of the reference's matmul example (examples/matmul.py:96-117, `acc + bias[tile[1]]` and
// `relu(acc + bias[tile[1]])`).
struct EpiScale {
  const float* a;
  const float* b;
  int mode;
  const float* bias;
  int relu;
};

// Scales 32 consecutive columns [col0, col0 + 32) of one output row held as fp32 bit patterns.
__device__ __forceinline__ void bias_relu_chunk(uint32_t (&r)[32], const EpiScale& sc, int col0, int N) {
  if (sc.bias != nullptr) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float b = col0 + i < N ? __ldg(sc.bias + col0 + i) : 0.0f;
      r[i] = __float_as_uint(__uint_as_float(r[i]) + b);
    }
  }
  if (sc.relu) {
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(fmaxf(__uint_as_float(r[i]), 0.0f));
  }
}

__device__ __forceinline__ void scales_only_chunk(uint32_t (&r)[32], const EpiScale& sc, int row, int M, int col0, int N) {
  if (sc.mode == 0) return;
  if (sc.mode == 1) {
    const float sa = __ldg(sc.a), sb = __ldg(sc.b);
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint((__uint_as_float(r[i]) * sa) * sb);
  } else {
    const float sa = row < M ? __ldg(sc.a + row) : 0.0f;
    const float* pb = sc.b + col0;
    if (col0 + 32 <= N && (reinterpret_cast<uintptr_t>(pb) & 15u) == 0) {
      // the common case: eight 16-byte loads (the same addresses in every lane, so one broadcast each)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 b4 = __ldg(reinterpret_cast<const float4*>(pb) + i);
        r[4 * i] = __float_as_uint((__uint_as_float(r[4 * i]) * sa) * b4.x);
        r[4 * i + 1] = __float_as_uint((__uint_as_float(r[4 * i + 1]) * sa) * b4.y);
        r[4 * i + 2] = __float_as_uint((__uint_as_float(r[4 * i + 2]) * sa) * b4.z);
        r[4 * i + 3] = __float_as_uint((__uint_as_float(r[4 * i + 3]) * sa) * b4.w);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float sb = col0 + i < N ? __ldg(pb + i) : 0.0f;
        r[i] = __float_as_uint((__uint_as_float(r[i]) * sa) * sb);
      }
    }
  }
}

// The whole epilogue on one chunk: scales, then bias, then ReLU.  (Kept free of recursion and of copies
// of `r`, so that the 32 values stay in registers.)
__device__ __forceinline__ void scale_chunk(uint32_t (&r)[32], const EpiScale& sc, int row, int M, int col0, int N) {
  scales_only_chunk(r, sc, row, M, col0, N);
  bias_relu_chunk(r, sc, col0, N);
}

inline EpiScale epi_scale(const GemmArgs& a) { return EpiScale{a.scale_a, a.scale_b, a.scale_mode, a.bias, a.relu}; }

}  // namespace hb
