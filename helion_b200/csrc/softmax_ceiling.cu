// Softmax-only ceiling of the FP8 attention kernels: the per-score work of pytorch-labs/helion
// examples/fp8_attention.py:74-94 (row max, exp2, row sum, cast of P to e4m3) with nothing around it -- no
// loads of Q/K/V, no tensor-core instructions, no barriers between roles.  Every softmax warpgroup owns 128
// rows: per step each thread pulls its 128 scores out of tensor memory, takes the row max, exponentiates,
// sums, packs P to e4m3 and stores P back to tensor memory, exactly the instruction stream of the attention
// kernel's softmax warps (attention_softmax.cuh).  The time per 128x128 step per SM that this kernel reaches
// is the floor for an attention kernel whose softmax runs in fp32 with this arithmetic, whatever its pipeline.
#include <cstdio>

#include "attention_softmax.cuh"
#include "host.h"

namespace hb {

namespace {

// MODE 0: the full step.  1: without the row max.  2: without the exponentials (p = s*c - m).  3: tensor-memory
// loads and stores only.
template <int WGS, int POLY_OF8, int MODE>
__global__ void __maxnreg__(176)  // the register budget of a softmax thread in the attention kernel
softmax_ceiling_kernel(int steps, float scale_log2, unsigned long long* cycles, float* sink) {
  constexpr int TMEM_COLS = WGS == 1 ? 256 : 512;  // S of warpgroup g at 128*g, its P at 128*WGS + 32*g
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (warp == 0) {
    tmem_alloc(&tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  const int wg = warp >> 2;
  const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
  const uint32_t t_s = tmem_base + lane_sel + wg * 128;
  const uint32_t t_p = tmem_base + lane_sel + 128 * WGS + wg * 32;

  // scores: a fixed pseudo-random pattern in [-4, 4), different for every row and column
  {
    uint32_t x = (blockIdx.x * 1024u + threadIdx.x) * 2654435761u + 12345u;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        x = x * 1664525u + 1013904223u;
        v[i] = __float_as_uint(static_cast<float>(x >> 8) * (8.0f / 16777216.0f) - 4.0f);
      }
      tmem_st_32x32b_x32(t_s + c * 32, v);
    }
    tmem_wait_st();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  float m_i = -INFINITY, l_i = 0.0f;
  const long long t0 = clock64();
  for (int step = 0; step < steps; ++step) {
    uint32_t s[4][32];
#pragma unroll
    for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(t_s + c * 32, s[c]);
    tmem_wait_ld();
    float m_new = m_i;
    if constexpr (MODE == 0 || MODE == 2) {
      m_new = fmaxf(m_i, row_max128(s) * scale_log2);
    } else {
      m_new = 4.0f * scale_log2;
    }
    const float alpha = fast_exp2(m_i - m_new);
    const uint64_t c2 = pack2f(scale_log2, scale_log2);
    const uint64_t negm2 = pack2f(-m_new, -m_new);
    uint64_t sum_a = 0ull, sum_b = 0ull;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t packed[8];
      if constexpr (MODE == 0 || MODE == 1) {
        exp_chunk32<POLY_OF8>(s[c], c, c2, negm2, sum_a, sum_b, packed);
      } else if constexpr (MODE == 2) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const uint64_t p0 = ffma2(pack2(s[c][i], s[c][i + 1]), c2, negm2);
          const uint64_t p1 = ffma2(pack2(s[c][i + 2], s[c][i + 3]), c2, negm2);
          sum_a = fadd2(sum_a, p0);
          sum_b = fadd2(sum_b, p1);
          uint32_t a0, a1, b0, b1;
          unpack2(p0, a0, a1);
          unpack2(p1, b0, b1);
          packed[i / 4] = pack_e4m3x4(__uint_as_float(a0), __uint_as_float(a1), __uint_as_float(b0), __uint_as_float(b1));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) packed[i] = s[c][4 * i] ^ s[c][4 * i + 1] ^ s[c][4 * i + 2] ^ s[c][4 * i + 3];
      }
      tmem_st_32x32b_x8(t_p + c * 8, packed);
    }
    tmem_wait_st();
    uint32_t sl, sh;
    unpack2(fadd2(sum_a, sum_b), sl, sh);
    l_i = l_i * alpha + (__uint_as_float(sl) + __uint_as_float(sh));
    m_i = m_new;
  }
  const long long t1 = clock64();
  if (sink != nullptr) sink[blockIdx.x * blockDim.x + threadIdx.x] = m_i + l_i;
  // the slowest warp of the CTA
  __shared__ unsigned long long span;
  if (threadIdx.x == 0) span = 0ull;
  __syncthreads();
  if (lane == 0) atomicMax(&span, static_cast<unsigned long long>(t1 - t0));
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) cycles[blockIdx.x] = span;
  if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int WGS, int POLY_OF8, int MODE>
int launch_ceiling(int ctas_per_sm, int steps, float scale_log2, unsigned long long* cycles, int num_sms, cudaStream_t stream) {
  softmax_ceiling_kernel<WGS, POLY_OF8, MODE><<<num_sms * ctas_per_sm, 128 * WGS, 0, stream>>>(steps, scale_log2, cycles,
                                                                                            nullptr);
  HB_CUDA_CHECK(cudaGetLastError());
  return HB200_OK;
}

template <int WGS>
int launch_ceiling_wgs(int ctas_per_sm, int poly_of8, int mode, int steps, float scale_log2, unsigned long long* cycles,
                       int num_sms, cudaStream_t stream) {
  if (mode == 1) return launch_ceiling<WGS, 0, 1>(ctas_per_sm, steps, scale_log2, cycles, num_sms, stream);
  if (mode == 2) return launch_ceiling<WGS, 0, 2>(ctas_per_sm, steps, scale_log2, cycles, num_sms, stream);
  if (mode == 3) return launch_ceiling<WGS, 0, 3>(ctas_per_sm, steps, scale_log2, cycles, num_sms, stream);
  switch (poly_of8) {
    case 0:
      return launch_ceiling<WGS, 0, 0>(ctas_per_sm, steps, scale_log2, cycles, num_sms, stream);
    case 2:
      return launch_ceiling<WGS, 2, 0>(ctas_per_sm, steps, scale_log2, cycles, num_sms, stream);
    case 3:
      return launch_ceiling<WGS, 3, 0>(ctas_per_sm, steps, scale_log2, cycles, num_sms, stream);
    case 4:
      return launch_ceiling<WGS, 4, 0>(ctas_per_sm, steps, scale_log2, cycles, num_sms, stream);
    default:
      return set_error(HB200_ERR_BAD_CONFIG, "softmax_ceiling: poly_of8 must be 0, 2, 3 or 4");
  }
}

}  // namespace

int launch_softmax_ceiling(int wgs, int ctas_per_sm, int poly_of8, int mode, int steps, unsigned long long* cycles,
                           DeviceCtx* ctx, cudaStream_t stream) {
  const float scale_log2 = 0.18033688f;  // log2(e) / sqrt(64)
  if (wgs == 1) return launch_ceiling_wgs<1>(ctas_per_sm, poly_of8, mode, steps, scale_log2, cycles, ctx->num_sms, stream);
  return launch_ceiling_wgs<2>(ctas_per_sm, poly_of8, mode, steps, scale_log2, cycles, ctx->num_sms, stream);
}

}  // namespace hb
