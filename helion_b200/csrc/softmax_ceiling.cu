// Softmax-only ceiling of the FP8 attention kernels: the per-score work of pytorch-labs/helion
// examples/fp8_attention.py:74-94 (row max, exp2, row sum, cast of P to e4m3) with nothing around it -- no
// loads of Q/K/V, no tensor-core instructions, no barriers between roles.  Every softmax warpgroup owns 128
// rows: per step each thread pulls its 128 scores out of tensor memory, takes the row max, exponentiates,
// sums, packs P to e4m3 and stores P back to tensor memory, exactly the instruction stream of the attention
// kernel's softmax warps (attention_softmax.cuh).  The time per 128x128 step per SM that this kernel reaches
// is the floor for an attention kernel whose softmax runs in fp32 with this arithmetic, whatever its pipeline.
//
// The same kernel can add, one piece at a time, what else an attention kernel runs on the SM while its softmax
// warps work ("noise"), to see what each piece costs the softmax loop.
#include <cstdio>

#include "attention_softmax.cuh"
#include "host.h"

namespace hb {

namespace {

constexpr int CEIL_NOISE_WARPS = 12;  // 4 pollers, 1 tensor-core issuer, 4 rescalers, 3 idle (whole warpgroups; only with NOISE != 0)

// MODE 0: the full step.  1: without the row max.  2: without the exponentials (p = s*c - m).  3: tensor-memory
// loads and stores only.
// NOISE (bit mask, two warpgroups only):
//   1  four more warps that poll an mbarrier which completes only at the end (roles waiting for their turn)
//   2  one more warp whose first thread issues tensor-core instructions back to back (128x128x32 e4m3, six per
//      commit, on shared-memory operands) into tensor-memory columns of its own
//   4  four more warps that rescale 64 columns of tensor memory in a loop (load, multiply, store)
//   8  the softmax threads themselves add, per step, the barrier traffic of the attention kernel's protocol:
//      four arrivals and three waits that find their barrier complete, per thread
template <int WGS, int POLY_OF8, int MODE, int NOISE>
__device__ __forceinline__ void softmax_ceiling_body(int steps, float scale_log2, unsigned long long* cycles, float* sink) {
  constexpr int TMEM_COLS = WGS == 1 ? 256 : 512;  // S of warpgroup g at 128*g, its P at 128*WGS + 32*g
  constexpr int SOFTMAX_WARPS = 4 * WGS;
  __shared__ uint32_t tmem_slot;
  __shared__ unsigned long long span;
  __shared__ __align__(8) uint64_t noise_bars[8];  // 0: end of the run, 1: tensor-core commits, 2-5: dummy protocol
  __shared__ volatile int noise_stop;
  extern __shared__ __align__(1024) uint8_t noise_smem[];  // operands of the tensor-core noise (32 KB when used)
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(&noise_bars[0], 1);
    mbar_init(&noise_bars[1], 1);
    for (int i = 2; i < 6; ++i) mbar_init(&noise_bars[i], 128 * WGS);
    noise_stop = 0;
    span = 0ull;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
  if constexpr (NOISE != 0) {
    // 640 threads x 96 registers at launch -> softmax threads 176 (their budget in the attention kernel), the rest 40
    if (warp < SOFTMAX_WARPS) asm volatile("setmaxnreg.inc.sync.aligned.u32 176;");
    else asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
  }

  if (warp < SOFTMAX_WARPS) {
    const int wg = warp >> 2;
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
    float m_i = -INFINITY, l_i = 0.0f;
    uint32_t nph = 0;
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
      if constexpr ((NOISE & 8) != 0) {
        // four arrivals per thread; the last thread's arrival completes the phase, which everybody then waits
        // for three times (every wait is bounded)
#pragma unroll
        for (int i = 2; i < 6; ++i) mbar_arrive(&noise_bars[i]);
#pragma unroll
        for (int i = 2; i < 5; ++i) {
          const long long w0 = clock64();
          while (!mbar_try_wait(&noise_bars[i], nph) && clock64() - w0 < 4000000) {
          }
        }
        nph ^= 1u;
      }
      uint32_t sl, sh;
      unpack2(fadd2(sum_a, sum_b), sl, sh);
      l_i = l_i * alpha + (__uint_as_float(sl) + __uint_as_float(sh));
      m_i = m_new;
    }
    const long long t1 = clock64();
    if (sink != nullptr) sink[blockIdx.x * blockDim.x + threadIdx.x] = m_i + l_i;
    if (lane == 0) atomicMax(&span, static_cast<unsigned long long>(t1 - t0));  // the slowest softmax warp
    // the noise roles stop when every softmax warp is through
    asm volatile("bar.sync 1, %0;" ::"n"(128 * WGS) : "memory");
    if (threadIdx.x == 0) {
      noise_stop = 1;
      mbar_arrive(&noise_bars[0]);
    }
  } else {
    // ---- noise roles; they end when the softmax warps are done, and every loop is bounded ----------------
    const int nw = warp - SOFTMAX_WARPS;
    const long long budget = static_cast<long long>(steps) * 20000 + 1000000;  // SM clocks
    const long long n0 = clock64();
    float acc = 0.0f;
    if ((NOISE & 1) != 0 && nw < 4) {
      while (!mbar_try_wait(&noise_bars[0], 0) && clock64() - n0 < budget) {
      }
    } else if ((NOISE & 2) != 0 && nw == 4) {
      if (lane == 0) {
        constexpr uint32_t idesc = make_idesc_e4m3(128, 128, false, false);
        const uint32_t a = (smem_u32(noise_smem) + 1023u) & ~1023u;
        const uint64_t a_desc = make_smem_desc(a, 16, 1024, SWZ_128B);
        const uint64_t b_desc = make_smem_desc(a + 16384, 16, 1024, SWZ_128B);
        uint32_t ph = 0;
        while (noise_stop == 0 && clock64() - n0 < budget) {
#pragma unroll 1
          for (int i = 0; i < 6; ++i) {
            umma_f8_ss(tmem_base + 384, desc_advance(a_desc, (i & 3) * 32), desc_advance(b_desc, (i & 3) * 32), idesc,
                       i != 0 ? 1u : 0u);
          }
          umma_commit(&noise_bars[1]);
          while (!mbar_try_wait(&noise_bars[1], ph) && clock64() - n0 < budget) {
          }
          ph ^= 1u;
        }
      }
      __syncwarp();
    } else if ((NOISE & 4) != 0 && nw >= 5) {
      const uint32_t t_o = tmem_base + lane_sel + 320;
      while (noise_stop == 0 && clock64() - n0 < budget) {
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(t_o + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * 0.999f);
          tmem_st_32x32b_x32(t_o + c * 32, o);
          acc += __uint_as_float(o[0]);
        }
        tmem_wait_st();
      }
    }
    if (sink != nullptr) sink[blockIdx.x * blockDim.x + threadIdx.x] = acc;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) cycles[blockIdx.x] = span;
  if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int WGS, int POLY_OF8, int MODE>
__global__ void __maxnreg__(176)  // the register budget of a softmax thread in the attention kernel
softmax_ceiling_kernel(int steps, float scale_log2, unsigned long long* cycles, float* sink) {
  softmax_ceiling_body<WGS, POLY_OF8, MODE, 0>(steps, scale_log2, cycles, sink);
}

template <int NOISE>
__global__ void __launch_bounds__(256 + 32 * CEIL_NOISE_WARPS, 1)
softmax_ceiling_noise_kernel(int steps, float scale_log2, unsigned long long* cycles, float* sink) {
  softmax_ceiling_body<2, 0, 0, NOISE>(steps, scale_log2, cycles, sink);
}

template <int WGS, int POLY_OF8, int MODE>
int launch_ceiling(int ctas_per_sm, int steps, float scale_log2, unsigned long long* cycles, int num_sms, cudaStream_t stream) {
  softmax_ceiling_kernel<WGS, POLY_OF8, MODE><<<num_sms * ctas_per_sm, 128 * WGS, 0, stream>>>(steps, scale_log2, cycles, nullptr);
  HB_CUDA_CHECK(cudaGetLastError());
  return HB200_OK;
}

template <int NOISE>
int launch_noise(int steps, float scale_log2, unsigned long long* cycles, int num_sms, cudaStream_t stream) {
  softmax_ceiling_noise_kernel<NOISE><<<num_sms, 256 + 32 * CEIL_NOISE_WARPS, 32768 + 2048, stream>>>(steps, scale_log2, cycles,
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

int launch_ceiling_noise(int noise, int steps, float scale_log2, unsigned long long* cycles, int num_sms, cudaStream_t stream) {
  switch (noise) {
    case 1:
      return launch_noise<1>(steps, scale_log2, cycles, num_sms, stream);
    case 2:
      return launch_noise<2>(steps, scale_log2, cycles, num_sms, stream);
    case 4:
      return launch_noise<4>(steps, scale_log2, cycles, num_sms, stream);
    case 8:
      return launch_noise<8>(steps, scale_log2, cycles, num_sms, stream);
    case 15:
      return launch_noise<15>(steps, scale_log2, cycles, num_sms, stream);
    default:
      return set_error(HB200_ERR_BAD_CONFIG, "softmax_ceiling: noise must be 1, 2, 4, 8 or 15");
  }
}

}  // namespace

// mode 0..3 as above; mode 16 + n runs the full step of two warpgroups with noise mask n.
int launch_softmax_ceiling(int wgs, int ctas_per_sm, int poly_of8, int mode, int steps, unsigned long long* cycles,
                           DeviceCtx* ctx, cudaStream_t stream) {
  const float scale_log2 = 0.18033688f;  // log2(e) / sqrt(64)
  if (mode >= 16) return launch_ceiling_noise(mode - 16, steps, scale_log2, cycles, ctx->num_sms, stream);
  if (wgs == 1) return launch_ceiling_wgs<1>(ctas_per_sm, poly_of8, mode, steps, scale_log2, cycles, ctx->num_sms, stream);
  return launch_ceiling_wgs<2>(ctas_per_sm, poly_of8, mode, steps, scale_log2, cycles, ctx->num_sms, stream);
}

}  // namespace hb
