// FP8 GEMM for few rows of x (M <= 64) against a column-major y: out[M,N] = cast(x[M,K] @ y[K,N]),
// the decode-time shape of examples/fp8_gemm.py:29-57 (a handful of tokens against a weight matrix).
//
// Such a call is bound by streaming y from HBM once, so the kernel is built to keep as many bytes
// of y in flight per SM as shared memory allows.  It computes out^T: the 128 rows of the UMMA are
// 128 columns of y (its "A" operand, K-major as stored), and the few rows of x are the UMMA's N
// dimension (16, 32 or 64).  A pipeline stage is then 16 KB of y plus only 2-8 KB of x -- the
// 128 x 128 tile of the general kernel spends half of every stage on rows of x that do not exist --
// and 9 to 12 stages fit instead of 6.  No tensor-core work is wasted on padding rows either.
//
//   warp 0     TMA producer: y tile [128 columns x 128 K] and x tile [NM rows x 128 K] per stage
//   warp 1     MMA issuer: tcgen05.mma kind::f8f6f4, M = 128, N = NM, fp32 accumulator of NM columns
//              in tensor memory (two of them, so the epilogue of one unit overlaps the next)
//   warps 2-5  epilogue: lane = column of y, registers = rows of x; stores one 64- or 128-byte row
//              segment per warp and row
//
// Work units are (128-column block of y, K range); with splits > 1 every unit writes fp32 partial
// sums and the ordered reduction kernel of the general GEMM finishes the job.
//
// MODE 0: as many stages as shared memory holds (12 / 11 / 9), one CTA per SM.
// MODE 1: half the stages (6 / 5 / 4), so that the CTAs of two consecutive launches fit on one SM: in a
//         chain of launches with programmatic dependent launch the next kernel's CTAs are resident, set
//         up and waiting when their predecessor ends, instead of being scheduled then.
// MODE 2: MODE 1, and the producer requests its first stages of y BEFORE it waits for the predecessor
//         (x is still read after the wait, out written after it).  Only for a y that the preceding
//         kernel on the stream does not write -- a weight matrix in a decode loop; the caller says so by
//         choosing the table row.  The weight stream then runs across the boundary between two layers.
//         (Also asking for the rest of the panel to be prefetched into the L2 at that point, with evict-first
//         loads into shared memory, was measured and dropped: 26 prefetch requests per CTA took 4-9 us to issue
//         and the later loads were no faster -- 17.4 us per layer against 14.6.)
#include <algorithm>
#include <string>

#include "common.cuh"
#include "host.h"
#include "epilogue.cuh"

// Build with -DHB_SKINNY_TRACE to record, per CTA, wall-clock (globaltimer) and SM-clock stamps of the kernel's
// phases (a development aid; hb200_debug_skinny_trace copies them to the host).  Product builds compile none of it.
#ifdef HB_SKINNY_TRACE
namespace hb {
__device__ unsigned long long g_skinny_trace[8192][12];
__shared__ unsigned long long sk_prod[4];  // the producer thread's stamps
__device__ unsigned int g_skinny_trace_n;
__device__ __forceinline__ unsigned long long sk_gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
}
extern "C" __attribute__((visibility("default"))) int hb200_debug_skinny_trace(unsigned long long* host_dst, unsigned int* n) {
  cudaError_t e = cudaMemcpyFromSymbol(host_dst, hb::g_skinny_trace, sizeof(unsigned long long) * 8192 * 12);
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(n, hb::g_skinny_trace_n, sizeof(unsigned int));
  return static_cast<int>(e);
}
#define SK_STAMP(slot) do { sk_t[slot] = hb::sk_gtime(); } while (0)
#else
#define SK_STAMP(slot) do { } while (0)
#endif

namespace hb {

namespace {

constexpr int SK_BN = 128;  // columns of y per unit = UMMA M
constexpr int SK_BK = 128;  // bytes of K per stage = one swizzle row
constexpr int SK_THREADS = 192;
constexpr int SK_EPI_THREADS = 128;
constexpr int SK_ACC_STRIDE = 64;  // tensor-memory columns between the two accumulators
constexpr int SK_TMEM_COLS = 128;

template <int NM, int MODE>
struct SkinnyLayout {
  static constexpr int W_BYTES = SK_BN * SK_BK;
  static constexpr int X_BYTES = NM * SK_BK;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  static constexpr int DEEP_STAGES = NM == 16 ? 12 : (NM == 32 ? 11 : 9);
  static constexpr int STAGES = MODE == 0 ? DEEP_STAGES : (NM == 16 ? 6 : (NM == 32 ? 5 : 4));  // modes 1, 2
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  // full[STAGES] empty[STAGES] acc_full[2] acc_empty[2] drain[1]
  static constexpr int NUM_BARS = 2 * STAGES + 5;
  static constexpr int BAR_OFFSET = RING_BYTES;
  static constexpr int MISC_OFFSET = BAR_OFFSET + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = MISC_OFFSET + 16 + 1024;
  static_assert(STAGE_BYTES % 1024 == 0, "stages must keep the 1024-byte alignment of the swizzle atoms");
  static_assert(SMEM_BYTES <= (MODE == 0 ? 227 : 113) * 1024, "shared memory budget (two CTAs per SM in modes 1 and 2)");
};

template <int NM, int OUT_DT, int MODE>
__global__ void __launch_bounds__(SK_THREADS, MODE == 0 ? 1 : 2)
fp8_gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, void* out,
                       int M, int N, int K, int64_t ldc, uint32_t* status, int splits, float* partials, EpiScale sc) {
  using L = SkinnyLayout<NM, MODE>;
  constexpr bool EARLY_Y = MODE == 2;
  constexpr int STAGES = L::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;
  uint64_t* acc_empty = bars + 2 * STAGES + 2;
  uint64_t* drain = bars + 2 * STAGES + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::MISC_OFFSET);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::MISC_OFFSET + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tiles = (N + SK_BN - 1) / SK_BN;
  const int k_blocks = (K + SK_BK - 1) / SK_BK;
  const int kb_per_split = (k_blocks + splits - 1) / splits;
  const int num_units = n_tiles * splits;  // unit u = (column block u % n_tiles, K range u / n_tiles)
  const WaitCtx wctx{abort_flag, status};
#ifdef HB_SKINNY_TRACE
  unsigned long long sk_t[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  SK_STAMP(0);  // entry
#endif

  if (threadIdx.x == 0) {
    // descriptor fetches overlap the barrier set-up and the tensor-memory allocation
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], SK_EPI_THREADS);
    }
    mbar_init(drain, 1);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, SK_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // everything above overlapped the previous kernel's tail (launch_pdl); global memory from here on
  // (with EARLY_Y the producer warp does not wait here -- a thread cannot run ahead of a warp that is parked in
  // the wait; its one working thread waits by itself after it has requested its first stages of y)
  SK_STAMP(1);  // set-up done
  if (!(EARLY_Y && warp == 0)) pdl_wait();
  SK_STAMP(2);  // predecessor ended
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------- TMA producer --------------------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      int prefetched = 0;  // K blocks of this CTA's first unit requested before the main loop
      if constexpr (EARLY_Y) {
        if (static_cast<int>(blockIdx.x) < num_units) {
          const int split = blockIdx.x / n_tiles;
          const int n_blk = blockIdx.x - split * n_tiles;
          const int kb_begin = split * kb_per_split;
          const int kb_end = min(k_blocks, kb_begin + kb_per_split);
          prefetched = min(STAGES, kb_end - kb_begin);
          for (int j = 0; j < prefetched; ++j) {  // fresh stages: nothing to wait for
            mbar_arrive_expect_tx(&full[j], L::STAGE_BYTES);
            tma_load_2d(smem + j * L::STAGE_BYTES, &tmap_w, &full[j], (kb_begin + j) * SK_BK, n_blk * SK_BN);
          }
#ifdef HB_SKINNY_TRACE
          sk_prod[0] = hb::sk_gtime();
#endif
          pdl_wait();  // x may be the predecessor's output
#ifdef HB_SKINNY_TRACE
          sk_prod[1] = hb::sk_gtime();
#endif
          for (int j = 0; j < prefetched; ++j) {
            tma_load_2d(smem + j * L::STAGE_BYTES + L::W_BYTES, &tmap_x, &full[j], (kb_begin + j) * SK_BK, 0);
          }
#ifdef HB_SKINNY_TRACE
          sk_prod[2] = hb::sk_gtime();
#endif
          it = static_cast<uint32_t>(prefetched);
        } else {
          pdl_wait();
        }
      }
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
        const int split = unit / n_tiles;
        const int n_blk = unit - split * n_tiles;
        const int kb_begin = split * kb_per_split + (unit == static_cast<int>(blockIdx.x) ? prefetched : 0);
        const int kb_end = min(k_blocks, split * kb_per_split + kb_per_split);
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u, wctx, SITE_GEMM_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* w_dst = smem + s * L::STAGE_BYTES;
          uint8_t* x_dst = w_dst + L::W_BYTES;
          mbar_arrive_expect_tx(&full[s], L::STAGE_BYTES);
          // rows of the y map are columns of y (K contiguous); rows beyond N / M arrive as zeros
          tma_load_2d(w_dst, &tmap_w, &full[s], kb * SK_BK, n_blk * SK_BN);
          tma_load_2d(x_dst, &tmap_x, &full[s], kb * SK_BK, 0);
        }
      }
      if (!ok) {
        const uint32_t back = it < static_cast<uint32_t>(STAGES) ? it : static_cast<uint32_t>(STAGES);
        for (uint32_t j = it - back; j < it; ++j) mbar_drain(&full[j % STAGES], (j / STAGES) & 1u);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ----------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_e4m3(SK_BN, NM, false, false);
      uint32_t it = 0;
      uint32_t unit_iter = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x, ++unit_iter) {
        const int kb_begin = (unit / n_tiles) * kb_per_split;
        const int kb_end = min(k_blocks, kb_begin + kb_per_split);
        const uint32_t acc = unit_iter & 1u;
        const uint32_t acc_ph = (unit_iter >> 1) & 1u;
        if (!mbar_wait(&acc_empty[acc], acc_ph ^ 1u, wctx, SITE_GEMM_ACC_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * SK_ACC_STRIDE;
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(&full[s], ph, wctx, SITE_GEMM_FULL)) {
            ok = false;
            break;
          }
#ifdef HB_SKINNY_TRACE
          if (it == 0) SK_STAMP(3);                                  // first stage landed
          if (it == static_cast<uint32_t>(STAGES)) SK_STAMP(4);      // first refilled stage landed
          if (kb == kb_end - 1) SK_STAMP(5);                         // last stage landed
#endif
          tc_fence_after_sync();
          const uint32_t w_addr = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t x_addr = w_addr + L::W_BYTES;
          // both operands K-major: 128-byte rows, 8-row swizzle atoms 1024 B apart
          const uint64_t w_desc = make_smem_desc(w_addr, 16, 1024, SWZ_128B);
          const uint64_t x_desc = make_smem_desc(x_addr, 16, 1024, SWZ_128B);
#pragma unroll
          for (int k = 0; k < SK_BK / 32; ++k) {
            umma_f8_ss(d_tmem, desc_advance(w_desc, k * 32), desc_advance(x_desc, k * 32), idesc,
                       (kb != kb_begin || k != 0) ? 1u : 0u);
          }
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&acc_full[acc]);
      }
      if (!ok) {
        umma_commit(drain);
        mbar_drain(drain, 0);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------- epilogue ------------------------------------------------
    const int quarter = warp & 3;  // a warp may only touch TMEM lanes [32*(warp%4), +32)
    uint32_t unit_iter = 0;
    for (int unit = blockIdx.x; unit < num_units; unit += gridDim.x, ++unit_iter) {
      const int split = unit / n_tiles;
      const int n_blk = unit - split * n_tiles;
      const uint32_t acc = unit_iter & 1u;
      const uint32_t acc_ph = (unit_iter >> 1) & 1u;
      bool ok = mbar_wait(&acc_full[acc], acc_ph, wctx, SITE_GEMM_ACC_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int n = n_blk * SK_BN + quarter * 32 + lane;  // this thread's column of y / out
      const uint32_t t_row = tmem_base + acc * SK_ACC_STRIDE + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll
      for (int c = 0; c < NM; c += 32) {
        uint32_t r[32];
        if constexpr (NM == 16) {
          uint32_t r16[16];
          tmem_ld_32x32b_x16(t_row, r16);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) r[i] = r16[i];
        } else {
          tmem_ld_32x32b_x32(t_row + c, r);
          tmem_wait_ld();
        }
        if (n < N) {
          // optional scales: this thread's column scale, one row scale per register
          const bool scaled = sc.mode != 0 && splits == 1;
          const float sb = scaled ? __ldg(sc.mode == 1 ? sc.b : sc.b + n) : 1.0f;
#pragma unroll
          for (int i = 0; i < (NM < 32 ? NM : 32); ++i) {
            const int m = c + i;
            if (m < M) {
              float v = __uint_as_float(r[i]);
              if (scaled) v = (v * __ldg(sc.mode == 1 ? sc.a : sc.a + m)) * sb;
              if (splits > 1) {
                partials[(static_cast<int64_t>(split) * M + m) * N + n] = v;
              } else if constexpr (OUT_DT == HB200_DT_FP32) {
                reinterpret_cast<float*>(out)[static_cast<int64_t>(m) * ldc + n] = v;
              } else if constexpr (OUT_DT == HB200_DT_BF16) {
                reinterpret_cast<uint16_t*>(out)[static_cast<int64_t>(m) * ldc + n] =
                    static_cast<uint16_t>(pack_bf16x2(v, 0.0f) & 0xffffu);
              } else {
                reinterpret_cast<uint16_t*>(out)[static_cast<int64_t>(m) * ldc + n] =
                    static_cast<uint16_t>(pack_f16x2(v, 0.0f) & 0xffffu);
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&acc_empty[acc]);
    }
  }

  // ------------------------------- teardown ----------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
#ifdef HB_SKINNY_TRACE
  if (threadIdx.x == 32) {  // the MMA thread holds the stamps; the epilogue warps have stored their outputs by now
    SK_STAMP(6);
    const unsigned int idx = atomicAdd(&g_skinny_trace_n, 1u) % 8192u;
    unsigned int smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    sk_t[7] = (static_cast<unsigned long long>(blockIdx.x) << 32) | smid;
    for (int i = 0; i < 8; ++i) g_skinny_trace[idx][i] = sk_t[i];
    for (int i = 0; i < 3; ++i) g_skinny_trace[idx][8 + i] = sk_prod[i];
  }
#endif
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, SK_TMEM_COLS);
  }
}

template <int NM, int OUT_DT, int MODE>
int launch_skinny_instance(const GemmArgs& a, DeviceCtx* ctx, const CUtensorMap& tw, const CUtensorMap& tx, int splits) {
  using L = SkinnyLayout<NM, MODE>;
  auto kernel = fp8_gemm_skinny_kernel<NM, OUT_DT, MODE>;
  static std::atomic<uint64_t> smem_attr_done{0};
  HB_CUDA_CHECK(set_max_dynamic_smem_once(smem_attr_done, reinterpret_cast<const void*>(kernel), L::SMEM_BYTES, a.device));
  const int64_t n_tiles = (a.N + SK_BN - 1) / SK_BN;
  const int grid = static_cast<int>(std::min<int64_t>(n_tiles * splits, ctx->num_sms));
  HB_CUDA_CHECK(launch_pdl(kernel, static_cast<unsigned>(grid), SK_THREADS, L::SMEM_BYTES, a.stream, tw, tx, a.out,
                           static_cast<int>(a.M), static_cast<int>(a.N), static_cast<int>(a.K), a.ldc, ctx->status_dev, splits,
                           static_cast<float*>(a.workspace), epi_scale(a)));
  return HB200_OK;
}

template <int NM, int MODE>
int launch_skinny_by_dtype(const GemmArgs& a, DeviceCtx* ctx, const CUtensorMap& tw, const CUtensorMap& tx, int splits) {
  switch (a.out_dtype) {
    case HB200_DT_FP16:
      return launch_skinny_instance<NM, HB200_DT_FP16, MODE>(a, ctx, tw, tx, splits);
    case HB200_DT_BF16:
      return launch_skinny_instance<NM, HB200_DT_BF16, MODE>(a, ctx, tw, tx, splits);
    case HB200_DT_FP32:
      return launch_skinny_instance<NM, HB200_DT_FP32, MODE>(a, ctx, tw, tx, splits);
    default:
      return set_error(HB200_ERR_BAD_DTYPE, "fp8_gemm: unsupported out_dtype");
  }
}

template <int NM>
int launch_skinny_by_mode(const GemmArgs& a, DeviceCtx* ctx, const CUtensorMap& tw, const CUtensorMap& tx, int splits, int mode) {
  switch (mode) {
    case 0:
      return launch_skinny_by_dtype<NM, 0>(a, ctx, tw, tx, splits);
    case 1:
      return launch_skinny_by_dtype<NM, 1>(a, ctx, tw, tx, splits);
    case 2:
      return launch_skinny_by_dtype<NM, 2>(a, ctx, tw, tx, splits);
    default:
      return set_error(HB200_ERR_BAD_CONFIG, "fp8_gemm: unknown mode of the few-row kernel");
  }
}

}  // namespace

bool gemm_skinny_supported(int64_t M, bool y_colmajor) { return y_colmajor && M >= 1 && M <= 64; }

int launch_fp8_gemm_skinny(const GemmArgs& a, DeviceCtx* ctx, int splits, int mode) {
  if (!gemm_skinny_supported(a.M, a.y_colmajor)) {
    return set_error(HB200_ERR_BAD_CONFIG, "fp8_gemm: the skinny rows need M <= 64 and a column-major y");
  }
  if (splits > 1) {
    const size_t need = static_cast<size_t>(splits) * a.M * a.N * sizeof(float);
    if (a.workspace == nullptr || a.workspace_bytes < need || (reinterpret_cast<uintptr_t>(a.workspace) & 15u)) {
      return set_error(HB200_ERR_WORKSPACE, "fp8_gemm: this split-K config needs a 16-byte aligned workspace of " +
                                                std::to_string(need) + " bytes (hb200_fp8_gemm_workspace_bytes)");
    }
  }
  const int nm = a.M <= 16 ? 16 : (a.M <= 32 ? 32 : 64);
  CUtensorMap tw, tx;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(a.K), static_cast<uint64_t>(a.N)};
    const uint64_t strides[1] = {static_cast<uint64_t>(a.ldb)};
    const uint32_t box[2] = {SK_BK, SK_BN};
    int rc = encode_tmap_u8(&tw, a.y, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HB200_OK) return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(a.K), static_cast<uint64_t>(a.M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(a.lda)};
    const uint32_t box[2] = {SK_BK, static_cast<uint32_t>(nm)};
    int rc = encode_tmap_u8(&tx, a.x, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HB200_OK) return rc;
  }
  int rc;
  switch (nm) {
    case 16:
      rc = launch_skinny_by_mode<16>(a, ctx, tw, tx, splits, mode);
      break;
    case 32:
      rc = launch_skinny_by_mode<32>(a, ctx, tw, tx, splits, mode);
      break;
    default:
      rc = launch_skinny_by_mode<64>(a, ctx, tw, tx, splits, mode);
      break;
  }
  if (rc != HB200_OK) return rc;
  return splits > 1 ? launch_splitk_reduce(a, splits) : HB200_OK;
}

}  // namespace hb
