// FP8 (e4m3 x e4m3 -> fp32) GEMM for sm_100a: out[M,N] = cast(x[M,K] @ y[K,N]).
//
// Computes what examples/fp8_gemm.py:29-57 of pytorch-labs/helion computes (zero-initialised
// fp32 accumulator, hl.dot over K tiles, cast on store), as one persistent, warp-specialised
// kernel:
//
//   warp 0   TMA producer: x and y tiles -> STAGES-deep ring of 128B-swizzled smem buffers
//   warp 1   MMA issuer: one thread issues tcgen05.mma kind::f8f6f4 (M=128, N=BN, K=32) into one
//            of two fp32 accumulators in tensor memory; tcgen05.commit releases smem stages and
//            publishes finished accumulators
//   warps 2-5 epilogue: tcgen05.ld the finished accumulator (while the MMA warp already fills the
//            other one), convert to fp16/bf16/fp32, store
//
// Tiles are walked in the L2-friendly grouped order (GROUP_M row blocks share their column
// blocks), the grid is one CTA per SM.  y may be column-major (B operand K-major) or row-major
// (B operand MN-major); both are fed straight from TMA without a transpose pass.
#include <algorithm>
#include <cstdio>
#include <mutex>
#include <string>

#include "common.cuh"
#include "host.h"
#include "epilogue.cuh"

namespace hb {

namespace {

constexpr int BM = 128;      // rows of one output tile = UMMA M
constexpr int BK = 128;      // BYTES of K per pipeline stage = one swizzle row (128 e4m3 or 64 16-bit elements)
constexpr int UMMA_K = 32;   // bytes of K per instruction (32 e4m3 elements for kind::f8f6f4, 16 for kind::f16)
// The kernels are written over bytes: K arrives as the byte length of a row of x, and operands with
// K contiguous look the same for every element size.  Only an operand with N contiguous ("MN-major":
// a row-major y) depends on the element size ES: a stage then holds BK/ES rows of K, and a 128-byte
// swizzle row spans 128/ES columns.
constexpr int NUM_THREADS = 192;
constexpr int NUM_EPI_THREADS = 128;

template <int BN, int STAGES>
struct GemmLayout {
  static constexpr int A_BYTES = BM * BK;
  static constexpr int B_BYTES = BN * BK;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  // full[STAGES] empty[STAGES] acc_full[2] acc_empty[2] drain[1]
  static constexpr int NUM_BARS = 2 * STAGES + 5;
  static constexpr int BAR_OFFSET = RING_BYTES;
  static constexpr int MISC_OFFSET = BAR_OFFSET + NUM_BARS * 8;  // tmem base (4 B) + abort flag (4 B)
  static constexpr int SMEM_BYTES = MISC_OFFSET + 16 + 1024;     // + slack to align the ring to 1024 B
  static constexpr int TMEM_COLS = 2 * BN;                       // two accumulators; power of two >= 32
  static_assert(TMEM_COLS == 512 || TMEM_COLS == 256 || TMEM_COLS == 128 || TMEM_COLS == 64, "tmem");
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

struct TileCoord {
  int m_blk;
  int n_blk;
};

// Grouped ("L2 swizzled") order: consecutive tile indices walk down GROUP_M row blocks before
// moving to the next column block, so CTAs that run at the same time share x and y tiles in L2.
__device__ __forceinline__ TileCoord tile_coord(int tile, int m_tiles, int n_tiles, int group_m) {
  const int per_group = group_m * n_tiles;
  const int group = tile / per_group;
  const int first_m = group * group_m;
  const int rows = min(m_tiles - first_m, group_m);
  const int in_group = tile - group * per_group;
  TileCoord c;
  c.m_blk = first_m + in_group % rows;
  c.n_blk = in_group / rows;
  return c;
}

template <int OUT_DT>
__device__ __forceinline__ void store_row_chunk(void* out, int64_t row_offset_elems, int col0, int N,
                                                const uint32_t (&r)[32]) {
  if constexpr (OUT_DT == HB200_DT_FP32) {
    float* dst = reinterpret_cast<float*>(out) + row_offset_elems + col0;
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      if (col0 + g * 4 + 4 <= N) {
        *reinterpret_cast<uint4*>(dst + g * 4) = make_uint4(r[g * 4], r[g * 4 + 1], r[g * 4 + 2], r[g * 4 + 3]);
      }
    }
  } else {
    uint16_t* dst = reinterpret_cast<uint16_t*>(out) + row_offset_elems + col0;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (col0 + g * 8 + 8 <= N) {
        uint32_t p[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float lo = __uint_as_float(r[g * 8 + 2 * j]);
          const float hi = __uint_as_float(r[g * 8 + 2 * j + 1]);
          p[j] = (OUT_DT == HB200_DT_BF16) ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi);
        }
        *reinterpret_cast<uint4*>(dst + g * 8) = make_uint4(p[0], p[1], p[2], p[3]);
      }
    }
  }
}

// Epilogue through shared memory and TMA: one warp stages a 32-row x 32-column block of converted
// outputs (row = lane) in a swizzled buffer and one lane stores it with a tiled bulk copy, which
// writes full row segments (instead of 32 scattered 16-byte pieces per store instruction) and clips
// rows beyond M / columns beyond N.  `stage` holds NBUF buffers of 32 x ROW_BYTES; the store that last
// used a buffer is waited for (its smem reads only) before the buffer is rewritten.
template <int OUT_DT>
struct StagedStore {
  static constexpr bool OUT32 = OUT_DT == HB200_DT_FP32;
  static constexpr int ROW_BYTES = OUT32 ? 128 : 64;
  static constexpr int STG_BYTES = 32 * ROW_BYTES;
  static constexpr int NBUF = OUT32 ? 1 : 2;  // 4 KB per warp either way

  __device__ static __forceinline__ void store(const uint32_t (&r)[32], uint8_t* stage, uint32_t chunk_count, int lane,
                                               const CUtensorMap* tmap_out, int col, int row0, bool inside,
                                               unsigned long long* trace = nullptr) {
    uint8_t* buf = stage + (chunk_count % NBUF) * STG_BYTES;
    if (lane == 0) tma_store_wait_read<NBUF - 1>();
    __syncwarp();
#ifdef HB_GEMM_TRACE
    if (trace != nullptr) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(trace[0]));
#endif
    // 16-byte chunk j of row r lives at chunk j ^ ((r >> 1) & 3) (64-byte rows, SWIZZLE_64B) or
    // j ^ (r & 7) (128-byte rows, SWIZZLE_128B): the pattern the output tensor map expects
    const uint32_t swz = OUT32 ? static_cast<uint32_t>(lane & 7) : static_cast<uint32_t>((lane >> 1) & 3);
    uint8_t* dst_row = buf + lane * ROW_BYTES;
    if constexpr (OUT32) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        *reinterpret_cast<uint4*>(dst_row + ((static_cast<uint32_t>(j) ^ swz) << 4)) =
            make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t p[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float lo = __uint_as_float(r[8 * j + 2 * q]);
          const float hi = __uint_as_float(r[8 * j + 2 * q + 1]);
          p[q] = (OUT_DT == HB200_DT_BF16) ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi);
        }
        *reinterpret_cast<uint4*>(dst_row + ((static_cast<uint32_t>(j) ^ swz) << 4)) = make_uint4(p[0], p[1], p[2], p[3]);
      }
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      // blocks that lie wholly outside the matrix are not stored at all (partial ones are clipped)
      if (inside) tma_store_2d(tmap_out, buf, col, row0);
      tma_store_commit();
    }
  }
};

template <int BN, int STAGES, bool B_MN_MAJOR, int OUT_DT, int KIND = KIND_E4M3>
__global__ void __launch_bounds__(NUM_THREADS, 1)
fp8_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, void* out,
                int M, int N, int K, int64_t ldc, int group_m, uint32_t* status, int splits, float* partials,
                EpiScale sc) {
  // splits > 1: split-K.  Work unit u = (tile u % num_tiles, K range u / num_tiles); every unit writes
  // its fp32 partial tile to partials[split][M][N] and splitk_reduce_kernel sums and converts.
  using L = GemmLayout<BN, STAGES>;
  constexpr int ES = KIND == KIND_E4M3 ? 1 : 2;  // element size of x and y
  constexpr int KROWS = BK / ES;                 // K rows of an MN-major B stage
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
  const int m_tiles = (M + BM - 1) / BM;
  const int n_tiles = (N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int k_blocks = (K + BK - 1) / BK;
  const int kb_per_split = (k_blocks + splits - 1) / splits;
  const int num_units = num_tiles * splits;
  const WaitCtx wctx{abort_flag, status};

  if (threadIdx.x == 0) {
    // descriptor fetches overlap the barrier set-up and the tensor-memory allocation
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], NUM_EPI_THREADS);
    }
    mbar_init(drain, 1);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, L::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // everything above overlapped the previous kernel's tail (launch_pdl); global memory from here on
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------- TMA producer --------------------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
        const int split = unit / num_tiles;
        const TileCoord tc = tile_coord(unit - split * num_tiles, m_tiles, n_tiles, group_m);
        const int kb_begin = split * kb_per_split;
        const int kb_end = min(k_blocks, kb_begin + kb_per_split);
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u, wctx, SITE_GEMM_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + s * L::STAGE_BYTES;
          uint8_t* b_dst = a_dst + L::A_BYTES;
          mbar_arrive_expect_tx(&full[s], L::STAGE_BYTES);
          tma_load_2d(a_dst, &tmap_a, &full[s], kb * BK, tc.m_blk * BM);
          if constexpr (!B_MN_MAJOR) {
            // y column-major: rows of the map are columns of y, K is contiguous.
            tma_load_2d(b_dst, &tmap_b, &full[s], kb * BK, tc.n_blk * BN);
          } else {
            // y row-major: N is contiguous; one box = BK/ES K rows x 128 bytes of N (coordinates in bytes / rows).
#pragma unroll
            for (int j = 0; j < BN * ES / 128; ++j) {
              tma_load_2d(b_dst + j * (KROWS * 128), &tmap_b, &full[s], tc.n_blk * BN * ES + j * 128, kb * KROWS);
            }
          }
        }
      }
      if (!ok) {
        // Abort path: let the copies that were issued land before the CTA exits.
        const uint32_t back = it < static_cast<uint32_t>(STAGES) ? it : static_cast<uint32_t>(STAGES);
        for (uint32_t j = it - back; j < it; ++j) mbar_drain(&full[j % STAGES], (j / STAGES) & 1u);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ----------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc<KIND>(BM, BN, false, B_MN_MAJOR);
      uint32_t it = 0;
      uint32_t tile_iter = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x, ++tile_iter) {
        const int kb_begin = (unit / num_tiles) * kb_per_split;
        const int kb_end = min(k_blocks, kb_begin + kb_per_split);
        const uint32_t acc = tile_iter & 1u;
        const uint32_t acc_ph = (tile_iter >> 1) & 1u;
        if (!mbar_wait(&acc_empty[acc], acc_ph ^ 1u, wctx, SITE_GEMM_ACC_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(&full[s], ph, wctx, SITE_GEMM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t b_addr = a_addr + L::A_BYTES;
          // A: K-major, 128-byte rows, 8-row atoms 1024 B apart.
          const uint64_t a_desc = make_smem_desc(a_addr, 16, 1024, SWZ_128B);
          // B K-major: same shape of atom.  B MN-major: 128 bytes of N contiguous, 8 K rows per
          // atom (1024 B apart), consecutive 128-byte column blocks KROWS*128 bytes apart; one
          // instruction consumes UMMA_K/ES rows of K.
          const uint64_t b_desc = B_MN_MAJOR ? make_smem_desc(b_addr, KROWS * 128, 1024, SWZ_128B)
                                             : make_smem_desc(b_addr, 16, 1024, SWZ_128B);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = desc_advance(a_desc, k * UMMA_K);
            const uint64_t bd = desc_advance(b_desc, B_MN_MAJOR ? k * (UMMA_K / ES) * 128 : k * UMMA_K);
            umma_ss<KIND>(d_tmem, ad, bd, idesc, (kb != kb_begin || k != 0) ? 1u : 0u);
          }
          umma_commit(&empty[s]);  // smem stage is free once these MMAs have read it
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
    uint32_t tile_iter = 0;
    for (int unit = blockIdx.x; unit < num_units; unit += gridDim.x, ++tile_iter) {
      const int split = unit / num_tiles;
      const TileCoord tc = tile_coord(unit - split * num_tiles, m_tiles, n_tiles, group_m);
      const uint32_t acc = tile_iter & 1u;
      const uint32_t acc_ph = (tile_iter >> 1) & 1u;
      bool ok = mbar_wait(&acc_full[acc], acc_ph, wctx, SITE_GEMM_ACC_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int row = tc.m_blk * BM + quarter * 32 + lane;
      const int64_t row_off = static_cast<int64_t>(row) * ldc;
      float* part = partials + (static_cast<int64_t>(split) * M + row) * N;  // used when splits > 1
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 2
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c, r);
        tmem_wait_ld();
        const int col0 = tc.n_blk * BN + c;
        if (row < M && col0 < N) {
          if (splits > 1) {
            store_row_chunk<HB200_DT_FP32>(part, 0, col0, N, r);  // unscaled; the reduce pass scales
          } else {
            scale_chunk(r, sc, row, M, col0, N);
            store_row_chunk<OUT_DT>(out, row_off, col0, N, r);
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
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, L::TMEM_COLS);
  }
}

// Split-K second pass: out[m, n] = cast(sum over splits of partials[s][m][n]), summed in split order
// (deterministic).  One thread per 8 consecutive columns.
template <int OUT_DT>
__global__ void splitk_reduce_kernel(const float* __restrict__ partials, void* out, int M, int N, int64_t ldc,
                                     int splits, EpiScale sc) {
  const int64_t groups_per_row = N / 8;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(M) * groups_per_row) return;
  const int64_t row = idx / groups_per_row;
  const int col = static_cast<int>(idx - row * groups_per_row) * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < splits; ++s) {
    const float4* src = reinterpret_cast<const float4*>(partials + (static_cast<int64_t>(s) * M + row) * N + col);
    const float4 a = src[0], b = src[1];
    acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
    acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
  }
  if (sc.mode != 0) {
    const float sa = sc.mode == 1 ? __ldg(sc.a) : __ldg(sc.a + row);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = (acc[j] * sa) * (sc.mode == 1 ? __ldg(sc.b) : __ldg(sc.b + col + j));
  }
  if constexpr (OUT_DT == HB200_DT_FP32) {
    float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + row * ldc + col);
    dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  } else {
    uint32_t p[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      p[j] = (OUT_DT == HB200_DT_BF16) ? pack_bf16x2(acc[2 * j], acc[2 * j + 1]) : pack_f16x2(acc[2 * j], acc[2 * j + 1]);
    }
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(out) + row * ldc + col) = make_uint4(p[0], p[1], p[2], p[3]);
  }
}

// ------------------------------------------------------------------------------------------------
// CTA-pair variant: two CTAs on one TPC compute one 256 x 256 tile with M = 256 UMMAs
// (tcgen05.mma.cta_group::2).  Each CTA loads its own 128 rows of x and HALF of the y tile (128
// columns), so a pair moves 64 KB per 128-deep K block for 256x256 outputs -- half the L2->SM
// traffic and half the smem read rate per flop of the 128x256 single-CTA tile -- and 6-7 stages fit.
//
//   both CTAs, warp 0     TMA producer for the CTA's own smem; completion bytes of BOTH CTAs are
//                         counted on the leader's `full` barrier
//   leader CTA, warp 1    issues the MMAs; tcgen05.commit signals `empty` / `acc_full` in each CTA
//   both CTAs, warps 2-5  epilogue of the CTA's own 128 accumulator rows; one arrival per warp on the
//                         leader's `acc_empty` barrier (remote arrive from the peer)
// ------------------------------------------------------------------------------------------------
template <int STAGES>
struct PairLayout {
  static constexpr int A_BYTES = BM * BK;   // 128 rows of x
  static constexpr int B_BYTES = 128 * BK;  // 128 of the tile's 256 columns of y
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 5;
  static constexpr int EPI_OFFSET = RING_BYTES;  // 4 KB of output staging per epilogue warp
  static constexpr int EPI_BYTES = 4 * 4096;
  static constexpr int BAR_OFFSET = EPI_OFFSET + EPI_BYTES;
  static constexpr int MISC_OFFSET = BAR_OFFSET + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = MISC_OFFSET + 16 + 1024;
  static constexpr int TMEM_COLS = 512;  // two 256-column accumulators
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

constexpr int PAIR_BM = 256;
constexpr int PAIR_BN = 256;

template <int STAGES, bool B_MN_MAJOR, int OUT_DT, int KIND = KIND_E4M3>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
fp8_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_out, int M, int N, int K, int group_m, uint32_t* status,
                     EpiScale sc) {
  using L = PairLayout<STAGES>;
  constexpr int ES = KIND == KIND_E4M3 ? 1 : 2;
  constexpr int KROWS = BK / ES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* full = bars;                       // used in the leader only
  uint64_t* empty = bars + STAGES;             // one set per CTA
  uint64_t* acc_full = bars + 2 * STAGES;      // one set per CTA
  uint64_t* acc_empty = bars + 2 * STAGES + 2; // used in the leader only (8 arrivals: 4 warps x 2 CTAs)
  uint64_t* drain = bars + 2 * STAGES + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::MISC_OFFSET);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::MISC_OFFSET + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int m_tiles = (M + PAIR_BM - 1) / PAIR_BM;
  const int n_tiles = (N + PAIR_BN - 1) / PAIR_BN;
  const int num_tiles = m_tiles * n_tiles;
  const int k_blocks = (K + BK - 1) / BK;
  const WaitCtx wctx{abort_flag, status};

  if (threadIdx.x == 0) {
    // descriptor fetches overlap the barrier set-up and the tensor-memory allocation
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_out);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 8);
    }
    mbar_init(drain, 1);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, L::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // everything above may overlap the previous kernel's tail (launch_pdl); global memory from here on
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) --------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
        const TileCoord tc = tile_coord(tile, m_tiles, n_tiles, group_m);
        const int row0 = tc.m_blk * PAIR_BM + static_cast<int>(rank) * 128;
        const int col0 = tc.n_blk * PAIR_BN + static_cast<int>(rank) * 128;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u, wctx, SITE_GEMM_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + s * L::STAGE_BYTES;
          uint8_t* b_dst = a_dst + L::A_BYTES;
          const uint32_t full_leader = map_to_cta(smem_u32(&full[s]), 0);
          if (leader) mbar_arrive_expect_tx(&full[s], 2 * L::STAGE_BYTES);
          tma_load_2d_pair(a_dst, &tmap_a, full_leader, kb * BK, row0);
          if constexpr (!B_MN_MAJOR) {
            tma_load_2d_pair(b_dst, &tmap_b, full_leader, kb * BK, col0);
          } else {
            // this CTA's 128 columns = ES blocks of 128 bytes x KROWS rows of K
#pragma unroll
            for (int j = 0; j < ES; ++j) {
              tma_load_2d_pair(b_dst + j * (KROWS * 128), &tmap_b, full_leader, col0 * ES + j * 128, kb * KROWS);
            }
          }
        }
      }
      if (!ok && leader) {
        // Abort path: the leader's `full` barriers count the bytes of both CTAs; let them land.
        const uint32_t back = it < static_cast<uint32_t>(STAGES) ? it : static_cast<uint32_t>(STAGES);
        for (uint32_t j = it - back; j < it; ++j) mbar_drain(&full[j % STAGES], (j / STAGES) & 1u);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader CTA only) -----------------------------
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc<KIND>(PAIR_BM, PAIR_BN, false, B_MN_MAJOR);
      uint32_t it = 0;
      uint32_t tile_iter = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs, ++tile_iter) {
        const uint32_t acc = tile_iter & 1u;
        const uint32_t acc_ph = (tile_iter >> 1) & 1u;
        if (!mbar_wait(&acc_empty[acc], acc_ph ^ 1u, wctx, SITE_GEMM_ACC_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * PAIR_BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(&full[s], ph, wctx, SITE_GEMM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t b_addr = a_addr + L::A_BYTES;
          const uint64_t a_desc = make_smem_desc(a_addr, 16, 1024, SWZ_128B);
          const uint64_t b_desc = B_MN_MAJOR ? make_smem_desc(b_addr, KROWS * 128, 1024, SWZ_128B)
                                             : make_smem_desc(b_addr, 16, 1024, SWZ_128B);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = desc_advance(a_desc, k * UMMA_K);
            const uint64_t bd = desc_advance(b_desc, B_MN_MAJOR ? k * (UMMA_K / ES) * 128 : k * UMMA_K);
            umma_ss_pair<KIND>(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // the stage is free in BOTH CTAs once these MMAs have read it
          const uint32_t e_local = smem_u32(&empty[s]);
          umma_commit_pair(e_local);
          umma_commit_pair(map_to_cta(e_local, 1));
        }
        if (ok) {
          const uint32_t f_local = smem_u32(&acc_full[acc]);
          umma_commit_pair(f_local);
          umma_commit_pair(map_to_cta(f_local, 1));
        }
      }
      if (!ok) {
        umma_commit_pair(smem_u32(drain));
        mbar_drain(drain, 0);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------- epilogue (both CTAs) -------------------------------------
    const int quarter = warp & 3;
    uint8_t* stage = smem + L::EPI_OFFSET + (warp - 2) * 4096;
    uint32_t chunk_count = 0;
    uint32_t tile_iter = 0;
    for (int tile = pair_id; tile < num_tiles; tile += num_pairs, ++tile_iter) {
      const TileCoord tc = tile_coord(tile, m_tiles, n_tiles, group_m);
      const uint32_t acc = tile_iter & 1u;
      const uint32_t acc_ph = (tile_iter >> 1) & 1u;
      bool ok = mbar_wait(&acc_full[acc], acc_ph, wctx, SITE_GEMM_ACC_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int row0 = tc.m_blk * PAIR_BM + static_cast<int>(rank) * 128 + quarter * 32;
      const uint32_t t_row = tmem_base + acc * PAIR_BN + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 2
      for (int c = 0; c < PAIR_BN; c += 32, ++chunk_count) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c, r);
        tmem_wait_ld();
        const int col = tc.n_blk * PAIR_BN + c;
        scale_chunk(r, sc, row0 + lane, M, col, N);
        StagedStore<OUT_DT>::store(r, stage, chunk_count, lane, &tmap_out, col, row0, row0 < M && col < N);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[acc]), 0));
    }
    if (lane == 0) tma_store_wait<0>();  // all output blocks written before the CTA exits
  }

  // ------------------------------- teardown ----------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves (or frees tensor memory) while the other may still use it
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc_pair(tmem_base, L::TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------
// CTA-pair variant with 256 x 256 outputs per CTA (512 x 256 per pair).  Each CTA keeps 256 rows of
// x and 128 columns of y per K block in shared memory and feeds TWO M = 256 UMMAs per K step from
// them (rows [0,128) of both CTAs -> accumulator 0, rows [128,256) -> accumulator 1), so the y tile
// is loaded once for twice the outputs: 48 KB per CTA per 128-deep K block for 256 x 256 outputs,
// a quarter less L2->SM traffic per flop than the 256 x 256 pair tile.  The two accumulators fill
// all 512 tensor-memory columns, so the epilogue cannot overlap the next tile's MMAs; instead eight
// epilogue warps drain the two accumulators in parallel and each accumulator is handed back on its
// own barrier, and the producer keeps prefetching the next tile's stages meanwhile.
// ------------------------------------------------------------------------------------------------
// Build with -DHB_GEMM_TRACE to record wall-clock stamps of the 512-row pair kernel's phases per leader CTA
// (a development aid; hb200_debug_gemm_trace copies them to the host).  Product builds compile none of it.
#ifdef HB_GEMM_TRACE
}  // namespace
}  // namespace hb
namespace hb {
__device__ unsigned long long g_gemm_trace[8192][32];
__device__ unsigned int g_gemm_trace_n;
__device__ __forceinline__ unsigned long long gm_gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
}  // namespace hb
extern "C" __attribute__((visibility("default"))) int hb200_debug_gemm_trace(unsigned long long* host_dst, unsigned int* n) {
  cudaError_t e = cudaMemcpyFromSymbol(host_dst, hb::g_gemm_trace, sizeof(unsigned long long) * 8192 * 32);
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(n, hb::g_gemm_trace_n, sizeof(unsigned int));
  return static_cast<int>(e);
}
namespace hb {
namespace {
#define GM_STAMP(slot) do { gm_t[slot] = hb::gm_gtime(); } while (0)
#else
#define GM_STAMP(slot) do { } while (0)
#endif

template <int STAGES, int TILE_N = 256>
struct Pair2Layout {
  static constexpr int A_BYTES = 256 * BK;  // 256 rows of x (two 128-row MMA operands)
  static constexpr int B_BYTES = (TILE_N / 2) * BK;  // this CTA's half of the tile's columns of y
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  // full[ST] empty[ST] acc_full[1] acc_empty[2] drain[1]
  static constexpr int NUM_BARS = 2 * STAGES + 4;
  // epilogue staging: per epilogue warp 4 KB (two 32-row x 64-byte buffers for 16-bit outputs, one
  // 32-row x 128-byte buffer for fp32), written swizzled and drained by TMA stores
  static constexpr int EPI_OFFSET = RING_BYTES;
  static constexpr int EPI_BYTES = 8 * 4096;
  static constexpr int BAR_OFFSET = EPI_OFFSET + EPI_BYTES;
  static constexpr int MISC_OFFSET = BAR_OFFSET + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = MISC_OFFSET + 16 + 1024;
  static constexpr int TMEM_COLS = 512;
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

constexpr int PAIR2_BM = 512;
constexpr int PAIR2_THREADS = 320;  // TMA warp, MMA warp, 8 epilogue warps

// PAIR2_BN = 224 (column-major e4m3 y only) exists for problems whose 256-wide tiles leave a round of pairs
// partly empty: 8192 columns are 37 blocks of 224, and 2 x 37 = 74 = one tile for every CTA pair.
template <int STAGES, bool B_MN_MAJOR, int OUT_DT, int KIND = KIND_E4M3, int PAIR2_BN = 256>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR2_THREADS, 1)
fp8_gemm_pair2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_out, int M, int N, int K, int group_m,
                      uint32_t* status, EpiScale sc) {
  using L = Pair2Layout<STAGES, PAIR2_BN>;
  static_assert(PAIR2_BN == 256 || (PAIR2_BN == 224 && !B_MN_MAJOR && KIND == KIND_E4M3), "tile widths built");
  static_assert(L::STAGE_BYTES % 1024 == 0 && 2 * PAIR2_BN <= L::TMEM_COLS, "swizzle alignment / tensor memory");
  constexpr int ES = KIND == KIND_E4M3 ? 1 : 2;
  constexpr int KROWS = BK / ES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* full = bars;                       // used in the leader only
  uint64_t* empty = bars + STAGES;             // one set per CTA
  uint64_t* acc_full = bars + 2 * STAGES;      // one per CTA: both accumulators of the tile are complete
  uint64_t* acc_empty = bars + 2 * STAGES + 1; // [2] used in the leader only (8 arrivals each: 4 warps x 2 CTAs)
  uint64_t* drain = bars + 2 * STAGES + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::MISC_OFFSET);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::MISC_OFFSET + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int m_tiles = (M + PAIR2_BM - 1) / PAIR2_BM;
  const int n_tiles = (N + PAIR2_BN - 1) / PAIR2_BN;
  const int num_tiles = m_tiles * n_tiles;
  const int k_blocks = (K + BK - 1) / BK;
  const WaitCtx wctx{abort_flag, status};
#ifdef HB_GEMM_TRACE
  unsigned long long gm_t[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  __shared__ unsigned long long gm_epi[2];
  __shared__ unsigned long long gm_chunk[24];  // per chunk of warp 2's first tile: scores loaded, staging buffer free, store issued
  GM_STAMP(0);  // entry
#endif

  if (threadIdx.x == 0) {
    // descriptor fetches overlap the barrier set-up and the tensor-memory allocation
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_out);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(&acc_empty[0], 8);
    mbar_init(&acc_empty[1], 8);
    mbar_init(drain, 1);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, L::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // everything above may overlap the previous kernel's tail (launch_pdl); global memory from here on
  GM_STAMP(1);  // set-up done
  pdl_wait();
  GM_STAMP(2);  // predecessor ended
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) --------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
        const TileCoord tc = tile_coord(tile, m_tiles, n_tiles, group_m);
        const int row0 = tc.m_blk * PAIR2_BM + static_cast<int>(rank) * 256;
        const int col0 = tc.n_blk * PAIR2_BN + static_cast<int>(rank) * (PAIR2_BN / 2);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u, wctx, SITE_GEMM_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + s * L::STAGE_BYTES;
          uint8_t* b_dst = a_dst + L::A_BYTES;
          const uint32_t full_leader = map_to_cta(smem_u32(&full[s]), 0);
          if (leader) mbar_arrive_expect_tx(&full[s], 2 * L::STAGE_BYTES);
          tma_load_2d_pair(a_dst, &tmap_a, full_leader, kb * BK, row0);  // box: 128 bytes x 256 rows
          if constexpr (!B_MN_MAJOR) {
            tma_load_2d_pair(b_dst, &tmap_b, full_leader, kb * BK, col0);
          } else {
#pragma unroll
            for (int j = 0; j < ES; ++j) {
              tma_load_2d_pair(b_dst + j * (KROWS * 128), &tmap_b, full_leader, col0 * ES + j * 128, kb * KROWS);
            }
          }
        }
      }
      if (!ok && leader) {
        const uint32_t back = it < static_cast<uint32_t>(STAGES) ? it : static_cast<uint32_t>(STAGES);
        for (uint32_t j = it - back; j < it; ++j) mbar_drain(&full[j % STAGES], (j / STAGES) & 1u);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader CTA only) -----------------------------
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc<KIND>(256, PAIR2_BN, false, B_MN_MAJOR);
      uint32_t it = 0;
      uint32_t tile_iter = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs, ++tile_iter) {
        const uint32_t free_parity = (tile_iter & 1u) ^ 1u;
        for (int kb = 0; kb < k_blocks && ok; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(&full[s], ph, wctx, SITE_GEMM_FULL)) {
            ok = false;
            break;
          }
#ifdef HB_GEMM_TRACE
          if (it == 0) GM_STAMP(3);                                   // first operands landed
          if (tile_iter == 0 && kb == k_blocks - 1) GM_STAMP(4);      // last operands of the first tile landed
#endif
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t b_addr = a_addr + L::A_BYTES;
          const uint64_t b_desc = B_MN_MAJOR ? make_smem_desc(b_addr, KROWS * 128, 1024, SWZ_128B)
                                             : make_smem_desc(b_addr, 16, 1024, SWZ_128B);
          // accumulator by accumulator, so that in the first K block of a tile the MMAs into
          // accumulator 0 can start while the epilogue still drains accumulator 1
#pragma unroll
          for (int acc = 0; acc < 2; ++acc) {
            if (kb == 0) {
              if (!mbar_wait(&acc_empty[acc], free_parity, wctx, SITE_GEMM_ACC_EMPTY)) {
                ok = false;
                break;
              }
              tc_fence_after_sync();
            }
            const uint64_t a_desc = make_smem_desc(a_addr + acc * (128 * BK), 16, 1024, SWZ_128B);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t ad = desc_advance(a_desc, k * UMMA_K);
              const uint64_t bd = desc_advance(b_desc, B_MN_MAJOR ? k * (UMMA_K / ES) * 128 : k * UMMA_K);
              umma_ss_pair<KIND>(tmem_base + acc * PAIR2_BN, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
            }
          }
          if (!ok) break;
          const uint32_t e_local = smem_u32(&empty[s]);
          umma_commit_pair(e_local);
          umma_commit_pair(map_to_cta(e_local, 1));
        }
        if (ok) {
          const uint32_t f_local = smem_u32(acc_full);
          umma_commit_pair(f_local);
          umma_commit_pair(map_to_cta(f_local, 1));
        }
      }
      if (!ok) {
        umma_commit_pair(smem_u32(drain));
        mbar_drain(drain, 0);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------- epilogue (both CTAs, 8 warps) ----------------------------
    // Each warp moves its 32 rows x 256 columns in 32-column chunks: tcgen05.ld -> convert -> swizzled
    // st.shared into a staging buffer -> one TMA store of the 32 x 32 block (which also clips rows
    // beyond M and columns beyond N).  Stores stay in flight while the next chunk is converted.
    const int quarter = warp & 3;
    const int acc = (warp - 2) >> 2;  // warps 2-5 drain accumulator 0, warps 6-9 accumulator 1
    uint8_t* stage = smem + L::EPI_OFFSET + (warp - 2) * 4096;
    uint32_t chunk_count = 0;
    uint32_t tile_iter = 0;
    for (int tile = pair_id; tile < num_tiles; tile += num_pairs, ++tile_iter) {
      const TileCoord tc = tile_coord(tile, m_tiles, n_tiles, group_m);
      bool ok = mbar_wait(acc_full, tile_iter & 1u, wctx, SITE_GEMM_ACC_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
#ifdef HB_GEMM_TRACE
      if (threadIdx.x == 64 && tile_iter == 0) gm_epi[0] = hb::gm_gtime();  // first tile's accumulators complete
#endif
      tc_fence_after_sync();
      const int row0 = tc.m_blk * PAIR2_BM + static_cast<int>(rank) * 256 + acc * 128 + quarter * 32;
      const uint32_t t_row = tmem_base + acc * PAIR2_BN + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 2
      for (int c = 0; c < PAIR2_BN; c += 32, ++chunk_count) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c, r);
        tmem_wait_ld();
        const int col = tc.n_blk * PAIR2_BN + c;
        scale_chunk(r, sc, row0 + lane, M, col, N);
#ifdef HB_GEMM_TRACE
        const bool tr = threadIdx.x == 64 && tile_iter == 0 && c < 256;
        if (tr) gm_chunk[(c / 32) * 3] = hb::gm_gtime();
        StagedStore<OUT_DT>::store(r, stage, chunk_count, lane, &tmap_out, col, row0, row0 < M && col < N,
                                   tr ? &gm_chunk[(c / 32) * 3 + 1] : nullptr);
        if (tr) gm_chunk[(c / 32) * 3 + 2] = hb::gm_gtime();
#else
        StagedStore<OUT_DT>::store(r, stage, chunk_count, lane, &tmap_out, col, row0, row0 < M && col < N);
#endif
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[acc]), 0));
#ifdef HB_GEMM_TRACE
      if (threadIdx.x == 64 && tile_iter == 0) gm_epi[1] = hb::gm_gtime();  // this warp's share of the first tile handed to TMA
#endif
    }
    if (lane == 0) tma_store_wait<0>();  // all output blocks written before the CTA exits
  }

  // ------------------------------- teardown ----------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
#ifdef HB_GEMM_TRACE
  if (threadIdx.x == 32 && leader) {
    GM_STAMP(7);
    gm_t[5] = gm_epi[0];
    gm_t[6] = gm_epi[1];
    const unsigned int idx = atomicAdd(&g_gemm_trace_n, 1u) % 8192u;
    for (int i = 0; i < 8; ++i) g_gemm_trace[idx][i] = gm_t[i];
    for (int i = 0; i < 24; ++i) g_gemm_trace[idx][8 + i] = gm_chunk[i];
  }
#endif
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc_pair(tmem_base, L::TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------
// tile-config table
// ------------------------------------------------------------------------------------------------
struct GemmConfig {
  int bn;        // tile width (columns of out per tile)
  int stages;
  int group_m;   // row blocks per rasterisation group
  bool pair;     // CTA-pair kernel (256 x 256 tiles) instead of the single-CTA kernel (128 x bn)
  int splits;    // split-K factor (needs a workspace of splits x M x N floats when > 1)
  const char* note;
  bool skinny = false;  // operand-swapped kernel for M <= 64, column-major y (fp8_gemm_skinny.cu)
  int skinny_mode = 0;  // 0: deepest ring, one CTA per SM; 1: half the stages, two CTAs per SM; 2: as 1, y requested before the predecessor ends
};

const GemmConfig kGemmConfigs[] = {
    {256, 4, 8, false, 1, "1 CTA, 128x256x128 tiles, 4 stages, group_m 8"},
    {128, 6, 8, false, 1, "1 CTA, 128x128x128 tiles, 6 stages, group_m 8: small problems, better wave fill"},
    {64, 8, 8, false, 1, "1 CTA, 128x64x128 tiles, 8 stages, group_m 8: very small N (column-major y only)"},
    {256, 4, 16, false, 1, "1 CTA, 128x256x128 tiles, 4 stages, group_m 16"},
    {256, 4, 4, false, 1, "1 CTA, 128x256x128 tiles, 4 stages, group_m 4"},
    {128, 6, 16, false, 1, "1 CTA, 128x128x128 tiles, 6 stages, group_m 16"},
    {256, 6, 8, true, 1, "CTA pair, 256x256x128 tiles, 6 stages, group_m 8 (of 256-row blocks)"},
    {256, 6, 12, true, 1, "CTA pair, 256x256x128 tiles, 6 stages, group_m 12"},
    {256, 6, 2, true, 1, "CTA pair, 256x256x128 tiles, 6 stages, group_m 2"},
    {256, 6, 16, true, 1, "CTA pair, 256x256x128 tiles, 6 stages, group_m 16"},
    {256, 6, 4, true, 1, "CTA pair, 256x256x128 tiles, 6 stages, group_m 4"},
    {128, 6, 8, false, 2, "1 CTA, 128x128x128 tiles, split-K 2: skinny M, HBM-bound"},
    {128, 6, 8, false, 4, "1 CTA, 128x128x128 tiles, split-K 4: skinny M, HBM-bound"},
    {128, 6, 8, false, 8, "1 CTA, 128x128x128 tiles, split-K 8: skinny M, HBM-bound"},
    {512, 4, 8, true, 1, "CTA pair, 512x256x128 tiles (256x256 per CTA, two accumulators), 4 stages, group_m 8"},
    {512, 4, 4, true, 1, "CTA pair, 512x256x128 tiles (256x256 per CTA, two accumulators), 4 stages, group_m 4"},
    {512, 4, 2, true, 1, "CTA pair, 512x256x128 tiles (256x256 per CTA, two accumulators), 4 stages, group_m 2"},
    {512, 4, 16, true, 1, "CTA pair, 512x256x128 tiles (256x256 per CTA, two accumulators), 4 stages, group_m 16"},
    {128, 12, 1, false, 1, "M <= 64, column-major y: operands swapped (128 columns of y x 16/32/64 rows of x), 9-12 stages", true},
    {128, 12, 1, false, 2, "M <= 64, column-major y: operands swapped, split-K 2", true},
    {128, 12, 1, false, 4, "M <= 64, column-major y: operands swapped, split-K 4", true},
    {448, 4, 8, true, 1, "CTA pair, 512x224x128 tiles (two accumulators), 4 stages, group_m 8: 37 column blocks per 8192 (column-major y only)"},
    {128, 6, 1, false, 1, "M <= 64, column-major y: operands swapped, 4-6 stages so that the CTAs of consecutive launches share an SM", true, 1},
    {128, 6, 1, false, 1, "M <= 64, column-major y: operands swapped, 4-6 stages, y requested before the preceding kernel on the stream has ended (the caller vouches that that kernel does not write y: a weight matrix)", true, 2},
};
constexpr int kNumGemmConfigs = sizeof(kGemmConfigs) / sizeof(kGemmConfigs[0]);
// Rows of the 512-row CTA-pair kernel carry its tile as bn = 512 (256 columns) or bn = 448 (224 columns).
static bool is_pair2(const GemmConfig& c) { return c.pair && c.bn >= 448; }
static int pair2_width(const GemmConfig& c) { return c.bn == 448 ? 224 : 256; }

// Output tensor map for the staged epilogue: 32 x 32 element boxes, swizzled like the staging buffers.
template <int OUT_DT>
int encode_out_map(CUtensorMap* tout, const GemmArgs& a) {
  constexpr bool out32 = OUT_DT == HB200_DT_FP32;
  const uint64_t elem = out32 ? 4 : 2;
  const uint64_t dims[2] = {static_cast<uint64_t>(a.N), static_cast<uint64_t>(a.M)};
  const uint64_t strides[1] = {static_cast<uint64_t>(a.ldc) * elem};
  const uint32_t box[2] = {32, 32};
  return encode_tmap(tout, out32 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, a.out, 2, dims, strides,
                     box, out32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
}

// K as the kernels see it: the byte length of a row of x.
template <int KIND>
int k_bytes(const GemmArgs& a) {
  return static_cast<int>(a.K * (KIND == KIND_E4M3 ? 1 : 2));
}

template <int STAGES, bool B_MN, int OUT_DT, int KIND = KIND_E4M3>
int launch_pair_instance(const GemmArgs& a, DeviceCtx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, int group_m) {
  using L = PairLayout<STAGES>;
  auto kernel = fp8_gemm_pair_kernel<STAGES, B_MN, OUT_DT, KIND>;
  static std::atomic<uint64_t> smem_attr_done{0};
  HB_CUDA_CHECK(set_max_dynamic_smem_once(smem_attr_done, reinterpret_cast<const void*>(kernel), L::SMEM_BYTES, a.device));
  const int64_t m_tiles = (a.M + PAIR_BM - 1) / PAIR_BM;
  const int64_t n_tiles = (a.N + PAIR_BN - 1) / PAIR_BN;
  const int64_t num_tiles = m_tiles * n_tiles;
  const int pairs = static_cast<int>(std::min<int64_t>(num_tiles, ctx->num_sms / 2));
  CUtensorMap tout;
  {
    int rc = encode_out_map<OUT_DT>(&tout, a);
    if (rc != HB200_OK) return rc;
  }
  HB_CUDA_CHECK(launch_pdl(kernel, static_cast<unsigned>(2 * pairs), NUM_THREADS, L::SMEM_BYTES, a.stream, ta, tb, tout,
                           static_cast<int>(a.M), static_cast<int>(a.N), k_bytes<KIND>(a), group_m, ctx->status_dev,
                           epi_scale(a)));
  return HB200_OK;
}

template <bool B_MN, int OUT_DT, int KIND = KIND_E4M3, int PAIR2_BN = 256>
int launch_pair2_instance(const GemmArgs& a, DeviceCtx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, int group_m) {
  using L = Pair2Layout<4, PAIR2_BN>;
  auto kernel = fp8_gemm_pair2_kernel<4, B_MN, OUT_DT, KIND, PAIR2_BN>;
  static std::atomic<uint64_t> smem_attr_done{0};
  HB_CUDA_CHECK(set_max_dynamic_smem_once(smem_attr_done, reinterpret_cast<const void*>(kernel), L::SMEM_BYTES, a.device));
  const int64_t m_tiles = (a.M + PAIR2_BM - 1) / PAIR2_BM;
  const int64_t n_tiles = (a.N + PAIR2_BN - 1) / PAIR2_BN;
  const int pairs = static_cast<int>(std::min<int64_t>(m_tiles * n_tiles, ctx->num_sms / 2));
  CUtensorMap tout;
  {
    int rc = encode_out_map<OUT_DT>(&tout, a);
    if (rc != HB200_OK) return rc;
  }
  HB_CUDA_CHECK(launch_pdl(kernel, static_cast<unsigned>(2 * pairs), PAIR2_THREADS, L::SMEM_BYTES, a.stream, ta, tb, tout,
                           static_cast<int>(a.M), static_cast<int>(a.N), k_bytes<KIND>(a), group_m, ctx->status_dev,
                           epi_scale(a)));
  return HB200_OK;
}

template <bool B_MN, int PAIR2_BN = 256>
int launch_pair2_by_dtype(const GemmArgs& a, DeviceCtx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, int group_m) {
  switch (a.out_dtype) {
    case HB200_DT_FP16:
      return launch_pair2_instance<B_MN, HB200_DT_FP16, KIND_E4M3, PAIR2_BN>(a, ctx, ta, tb, group_m);
    case HB200_DT_BF16:
      return launch_pair2_instance<B_MN, HB200_DT_BF16, KIND_E4M3, PAIR2_BN>(a, ctx, ta, tb, group_m);
    case HB200_DT_FP32:
      return launch_pair2_instance<B_MN, HB200_DT_FP32, KIND_E4M3, PAIR2_BN>(a, ctx, ta, tb, group_m);
    default:
      return set_error(HB200_ERR_BAD_DTYPE, "fp8_gemm: unsupported out_dtype");
  }
}

template <int STAGES, bool B_MN>
int launch_pair_by_dtype(const GemmArgs& a, DeviceCtx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, int group_m) {
  switch (a.out_dtype) {
    case HB200_DT_FP16:
      return launch_pair_instance<STAGES, B_MN, HB200_DT_FP16>(a, ctx, ta, tb, group_m);
    case HB200_DT_BF16:
      return launch_pair_instance<STAGES, B_MN, HB200_DT_BF16>(a, ctx, ta, tb, group_m);
    case HB200_DT_FP32:
      return launch_pair_instance<STAGES, B_MN, HB200_DT_FP32>(a, ctx, ta, tb, group_m);
    default:
      return set_error(HB200_ERR_BAD_DTYPE, "fp8_gemm: unsupported out_dtype");
  }
}

// K blocks each split handles and the number of non-empty splits for a requested split factor.
static int effective_splits(int64_t K, int requested) {
  const int k_blocks = static_cast<int>((K + BK - 1) / BK);
  const int want = std::max(1, std::min(requested, k_blocks));
  const int per = (k_blocks + want - 1) / want;
  return (k_blocks + per - 1) / per;
}

template <int BN, int STAGES, bool B_MN, int OUT_DT, int KIND = KIND_E4M3>
int launch_instance(const GemmArgs& a, DeviceCtx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, int group_m,
                    int splits_requested = 1) {
  using L = GemmLayout<BN, STAGES>;
  auto kernel = fp8_gemm_kernel<BN, STAGES, B_MN, OUT_DT, KIND>;
  static std::atomic<uint64_t> smem_attr_done{0};
  HB_CUDA_CHECK(set_max_dynamic_smem_once(smem_attr_done, reinterpret_cast<const void*>(kernel), L::SMEM_BYTES, a.device));
  const int m_tiles = static_cast<int>((a.M + BM - 1) / BM);
  const int n_tiles = static_cast<int>((a.N + BN - 1) / BN);
  const int64_t num_tiles = static_cast<int64_t>(m_tiles) * n_tiles;
  const int splits = effective_splits(k_bytes<KIND>(a), splits_requested);
  if (splits > 1) {
    const size_t need = static_cast<size_t>(splits) * a.M * a.N * sizeof(float);
    if (a.workspace == nullptr || a.workspace_bytes < need || (reinterpret_cast<uintptr_t>(a.workspace) & 15u)) {
      return set_error(HB200_ERR_WORKSPACE, "fp8_gemm: this split-K config needs a 16-byte aligned workspace of " +
                                                std::to_string(need) + " bytes (hb200_fp8_gemm_workspace_bytes)");
    }
  }
  const int grid = static_cast<int>(std::min<int64_t>(num_tiles * splits, ctx->num_sms));
  HB_CUDA_CHECK(launch_pdl(kernel, static_cast<unsigned>(grid), NUM_THREADS, L::SMEM_BYTES, a.stream, ta, tb, a.out,
                           static_cast<int>(a.M), static_cast<int>(a.N), k_bytes<KIND>(a), a.ldc, group_m, ctx->status_dev,
                           splits, static_cast<float*>(a.workspace), epi_scale(a)));
  return splits > 1 ? launch_splitk_reduce(a, splits) : HB200_OK;
}

template <int BN, int STAGES, bool B_MN>
int launch_by_dtype(const GemmArgs& a, DeviceCtx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, int group_m,
                    int splits = 1) {
  switch (a.out_dtype) {
    case HB200_DT_FP16:
      return launch_instance<BN, STAGES, B_MN, HB200_DT_FP16>(a, ctx, ta, tb, group_m, splits);
    case HB200_DT_BF16:
      return launch_instance<BN, STAGES, B_MN, HB200_DT_BF16>(a, ctx, ta, tb, group_m, splits);
    case HB200_DT_FP32:
      return launch_instance<BN, STAGES, B_MN, HB200_DT_FP32>(a, ctx, ta, tb, group_m, splits);
    default:
      return set_error(HB200_ERR_BAD_DTYPE, "fp8_gemm: unsupported out_dtype");
  }
}

}  // namespace

int launch_splitk_reduce(const GemmArgs& a, int splits) {
  const int64_t threads_total = a.M * (a.N / 8);
  const int blocks = static_cast<int>((threads_total + 255) / 256);
  const float* partials = static_cast<const float*>(a.workspace);
  const int m = static_cast<int>(a.M), n = static_cast<int>(a.N);
  switch (a.out_dtype) {
    case HB200_DT_FP16:
      splitk_reduce_kernel<HB200_DT_FP16><<<blocks, 256, 0, a.stream>>>(partials, a.out, m, n, a.ldc, splits, epi_scale(a));
      break;
    case HB200_DT_BF16:
      splitk_reduce_kernel<HB200_DT_BF16><<<blocks, 256, 0, a.stream>>>(partials, a.out, m, n, a.ldc, splits, epi_scale(a));
      break;
    case HB200_DT_FP32:
      splitk_reduce_kernel<HB200_DT_FP32><<<blocks, 256, 0, a.stream>>>(partials, a.out, m, n, a.ldc, splits, epi_scale(a));
      break;
    default:
      return set_error(HB200_ERR_BAD_DTYPE, "fp8_gemm: unsupported out_dtype");
  }
  HB_CUDA_CHECK(cudaGetLastError());
  return HB200_OK;
}

int gemm_num_configs() { return kNumGemmConfigs; }

int gemm_describe_config(int cfg_id, char* buf, int buf_len) {
  if (cfg_id < 0 || cfg_id >= kNumGemmConfigs) return set_error(HB200_ERR_BAD_CONFIG, "fp8_gemm: no such config");
  const GemmConfig& c = kGemmConfigs[cfg_id];
  if (c.skinny) return std::snprintf(buf, buf_len, "gemm cfg %d: split_k=%d (%s)", cfg_id, c.splits, c.note);
  return std::snprintf(buf, buf_len, "gemm cfg %d: BM=%d BN=%d BK=128 stages=%d group_m=%d split_k=%d (%s)", cfg_id,
                       is_pair2(c) ? 512 : (c.pair ? 256 : 128), is_pair2(c) ? pair2_width(c) : c.bn, c.stages, c.group_m,
                       c.splits, c.note);
}

size_t gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int out_dtype, int cfg_id) {
  if (cfg_id < 0) cfg_id = gemm_select_config(M, N, K, true, out_dtype, 148);
  if (cfg_id >= kNumGemmConfigs) return 0;
  const int splits = effective_splits(K, kGemmConfigs[cfg_id].splits);
  return splits > 1 ? static_cast<size_t>(splits) * M * N * sizeof(float) : 0;
}

// Chooses the table row with the smallest estimated time of the persistent schedule, in SM cycles:
//   rounds of tiles x (K blocks x cycles per K block + exposed cycles per tile).
// Single-CTA rows: 512 / 256 / 128 cycles per K block at full tensor rate over the tensor-pipe-active
// fractions measured at 8192^3 (128x256: 0.75, 128x128: 0.51, 128x64: 0.26).  The CTA-pair rows are fitted
// to launches timed back to back (20 per event pair, rows interleaved, the GPU at its power cap) on
// K = 4096 and K = 8192 problems; per round of tiles, in microseconds at K = 8192 / K = 4096:
//   256x256: 31.5-33.6 / 14.5-15.9    512x256: 59.8-62.6 / 29.1-32.5    512x224: 52.8-55.3 / 26.3-29.3
// (the 512x224 round took 0.88-0.95 of a 512x256 round, depending on the GPU).  What decides between
// them is mostly the number of rounds: 8192^3 is 7 rounds of 512x256 tiles, 8 of 512x224, 14 of 256x256;
// its 1024-, 2048- and 4096-row shards are 1, 2, 4 rounds of 512x224 tiles (37 column blocks x 2, 4, 8 row
// blocks on 74 CTA pairs) where 512x256 tiles leave 10, 20, 40 of 74 x rounds slots empty.
// A pair tile occupies two SMs.  The 224-wide row is built for a column-major y only.
static int gemm_select_config_nosplit(int64_t M, int64_t N, int64_t K, bool y_colmajor, int num_sms) {
  struct Candidate {
    int cfg;
    int64_t bm, bn;          // outputs per tile
    bool pair;
    double cycles_per_kb;    // per K block of one tile
    double exposed;          // cycles per tile that no overlap hides
  };
  const Candidate candidates[6] = {
      {3, 128, 256, false, 512.0 / 0.75, 0.0}, {1, 128, 128, false, 256.0 / 0.51, 0.0},
      {2, 128, 64, false, 128.0 / 0.26, 0.0},  {6, 256, 256, true, 620.0, 1500.0},
      {14, 512, 256, true, 1100.0, 6000.0},    {21, 512, 224, true, 1012.0, 6000.0},
  };
  const double k_blocks = static_cast<double>((K + BK - 1) / BK);
  int best = 3;
  double best_cost = -1.0;
  for (const Candidate& c : candidates) {
    if (!y_colmajor && (c.bn < 128 || c.bn == 224)) continue;
    const int64_t slots = c.pair ? num_sms / 2 : num_sms;
    const int64_t tiles = ((M + c.bm - 1) / c.bm) * ((N + c.bn - 1) / c.bn);
    const int64_t waves = (tiles + slots - 1) / slots;
    const double cost = static_cast<double>(waves) * (k_blocks * c.cycles_per_kb + c.exposed);
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = c.cfg;
    }
  }
  return best;
}

// Split-K row of the table for a problem, or -1.  Depends on the sizes only (not on layouts), so the
// workspace query and the launch agree.  Skinny problems (one row block, less than a wave of 128-wide
// tiles) are HBM-bound on reading y: splitting K puts ~3 waves of CTAs on the weight stream.
static int select_splitk_config(int64_t M, int64_t N, int64_t K, int num_sms) {
  const int64_t tiles = ((M + BM - 1) / BM) * ((N + 127) / 128);
  const int64_t k_blocks = (K + BK - 1) / BK;
  // Measured on B200 (M=16 and 128, N=14336, K=4096, cold L2): the split rows are 10-50 % SLOWER than
  // the plain 128x128 row (26.6 vs 29.7 us and 24.6 vs 37.9 us), so the automatic choice does not use
  // them yet; they stay in the table for explicit selection.
  constexpr bool kAutoSplitK = false;
  if (!kAutoSplitK || M > BM || tiles >= num_sms || k_blocks < 8) return -1;
  const int64_t want = (3 * num_sms + tiles - 1) / tiles;
  int splits = 2;
  while (splits < 8 && splits < want) splits *= 2;
  while (splits > 2 && k_blocks / splits < 4) splits /= 2;
  return splits == 2 ? 11 : (splits == 4 ? 12 : 13);
}

// Rows of the operand-swapped kernel.  Measured on B200, cold L2, bf16 out, K = 4096, N = 14336:
// M = 16: 21.5 us against 25.6 us for the 128x128 row (cuBLASLt 19.5 us); from M = 33 up (64 rows of x
// per stage, 9 stages) the general row is as fast or faster, so the automatic choice stops at 32.
// Split-K pays only when the column blocks alone leave most SMs idle (N = 4096, K = 14336: 25.6 us with
// 4 splits against 41.1 us without); with 112 column blocks its second kernel costs more than it gains.
static int select_skinny_config(int64_t M, int64_t N, int64_t K, bool y_colmajor, int num_sms) {
  if (!gemm_skinny_supported(M, y_colmajor) || M > 32) return -1;
  const int64_t n_tiles = (N + 127) / 128;
  const int64_t k_blocks = (K + BK - 1) / BK;
  if (n_tiles * 4 <= num_sms && k_blocks >= 32) return 20;
  if (n_tiles * 2 <= num_sms && k_blocks >= 16) return 19;
  return 18;
}

int gemm_select_config(int64_t M, int64_t N, int64_t K, bool y_colmajor, int out_dtype, int num_sms) {
  (void)out_dtype;
  const int skinny_cfg = select_skinny_config(M, N, K, y_colmajor, num_sms);
  if (skinny_cfg >= 0) return skinny_cfg;
  const int split_cfg = select_splitk_config(M, N, K, num_sms);
  if (split_cfg >= 0) return split_cfg;
  return gemm_select_config_nosplit(M, N, K, y_colmajor, num_sms);
}

// ------------------------------------------------------------------------------------------------
// Split-K with the partial sums in a fixed device array (hb200_fp8_gemm_splitk_static): for callers
// that must not allocate.  The array's NAME is only a host-side handle; its device address is
// looked up once per device with cudaGetSymbolAddress and that pointer is what the kernels get.
// Every call on a device uses the same array, so calls that can overlap on the GPU race on it.
// Nothing has to be cleared between calls: each (split, row < M, column < N) element is written by
// exactly one CTA of the first kernel before the reduce kernel reads it.
// ------------------------------------------------------------------------------------------------
namespace {
static __device__ __align__(256) float g_splitk_static_scratch[HB200_STATIC_SCRATCH_BYTES / sizeof(float)];

struct StaticScratchState {
  bool ready = false;
  float* scratch = nullptr;  // device address of g_splitk_static_scratch on this device
  int num_sms = 0;
};
StaticScratchState g_static_state[64];
std::mutex g_static_mutex;
}  // namespace

int launch_fp8_gemm_static_scratch(const GemmArgs& a_in, int splits_requested) {
  const int splits = effective_splits(a_in.K, splits_requested);
  if (splits < 2) {
    return set_error(HB200_ERR_BAD_CONFIG, "fp8_gemm_splitk_static: K is too short to split (needs at least 2 blocks of 128)");
  }
  // M*N against the elements one split may take, by division: the product of the sizes cannot wrap that way
  const uint64_t elems_per_split = HB200_STATIC_SCRATCH_BYTES / (sizeof(float) * static_cast<uint64_t>(splits));
  if (static_cast<uint64_t>(a_in.M) > elems_per_split / static_cast<uint64_t>(a_in.N)) {
    return set_error(HB200_ERR_WORKSPACE,
                     "fp8_gemm_splitk_static: splits*M*N*4 bytes (M = " + std::to_string(a_in.M) + ", N = " +
                         std::to_string(a_in.N) + ", " + std::to_string(splits) + " splits) exceeds the static scratch of " +
                         std::to_string(HB200_STATIC_SCRATCH_BYTES) + " bytes; use hb200_fp8_gemm with a workspace");
  }
  StaticScratchState* st = &g_static_state[a_in.device];
  {
    // First call on this device (the device is current here): resolve the array's device address.
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!st->ready) {
      int major = 0, sms = 0, current = -1;
      // the symbol's address belongs to the CURRENT device: it must be the one this call is for
      HB_CUDA_CHECK(cudaGetDevice(&current));
      if (current != a_in.device) {
        return set_error(HB200_ERR_CUDA, "fp8_gemm_splitk_static: device " + std::to_string(a_in.device) + " is not current");
      }
      HB_CUDA_CHECK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, a_in.device));
      HB_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, a_in.device));
      if (major != 10) return set_error(HB200_ERR_UNSUPPORTED_ARCH, "this library holds sm_100a code only");
      void* ptr = nullptr;
      HB_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_splitk_static_scratch));
      int rc = ensure_tmap_encoder();
      if (rc != HB200_OK) return rc;
      st->scratch = static_cast<float*>(ptr);
      st->num_sms = sms;
      st->ready = true;
    }
  }
  GemmArgs a = a_in;
  a.workspace = st->scratch;
  a.workspace_bytes = HB200_STATIC_SCRATCH_BYTES;
  // Only the fields the launcher reads.  The status word belongs to the device context, which this entry
  // point must not create (that allocates): it is used when another entry point has created it already;
  // until then a wait that runs out here still ends the kernel early but is not reported.
  DeviceCtx ctx;
  ctx.initialised = true;
  ctx.num_sms = st->num_sms;
  ctx.status_dev = peek_status_dev(a_in.device);

  CUtensorMap ta, tb;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(a.K), static_cast<uint64_t>(a.M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(a.lda)};
    const uint32_t box[2] = {BK, BM};
    int rc = encode_tmap_u8(&ta, a.x, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HB200_OK) return rc;
  }
  if (a.y_colmajor) {
    const uint64_t dims[2] = {static_cast<uint64_t>(a.K), static_cast<uint64_t>(a.N)};
    const uint64_t strides[1] = {static_cast<uint64_t>(a.ldb)};
    const uint32_t box[2] = {BK, 128};
    int rc = encode_tmap_u8(&tb, a.y, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HB200_OK) return rc;
    return launch_by_dtype<128, 6, false>(a, &ctx, ta, tb, 8, splits);
  }
  const uint64_t dims[2] = {static_cast<uint64_t>(a.N), static_cast<uint64_t>(a.K)};
  const uint64_t strides[1] = {static_cast<uint64_t>(a.ldb)};
  const uint32_t box[2] = {128, BK};
  int rc = encode_tmap_u8(&tb, a.y, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != HB200_OK) return rc;
  return launch_by_dtype<128, 6, true>(a, &ctx, ta, tb, 8, splits);
}

int launch_fp8_gemm(const GemmArgs& a, DeviceCtx* ctx) {
  int cfg_id = a.cfg_id;
  if (cfg_id < 0) {
    cfg_id = gemm_select_config(a.M, a.N, a.K, a.y_colmajor, a.out_dtype, ctx->num_sms);
    // The table's split-K rows need scratch; a caller that passed none gets the best row without.
    if (kGemmConfigs[cfg_id].splits > 1 &&
        (a.workspace == nullptr || a.workspace_bytes < gemm_workspace_bytes(a.M, a.N, a.K, a.out_dtype, cfg_id))) {
      cfg_id = kGemmConfigs[cfg_id].skinny ? 18 : gemm_select_config_nosplit(a.M, a.N, a.K, a.y_colmajor, ctx->num_sms);
    }
  }
  if (cfg_id >= kNumGemmConfigs) return set_error(HB200_ERR_BAD_CONFIG, "fp8_gemm: no such config");
  const GemmConfig& c = kGemmConfigs[cfg_id];
  if (c.skinny) return launch_fp8_gemm_skinny(a, ctx, effective_splits(a.K, c.splits), c.skinny_mode);
  if (!a.y_colmajor && (c.bn < 128 || c.bn == 448)) {
    return set_error(HB200_ERR_BAD_CONFIG, "fp8_gemm: this config supports column-major y only");
  }

  CUtensorMap ta, tb;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(a.K), static_cast<uint64_t>(a.M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(a.lda)};
    const uint32_t box[2] = {BK, static_cast<uint32_t>(is_pair2(c) ? 256 : BM)};  // the 512-row pair tile loads 256 rows per CTA
    int rc = encode_tmap_u8(&ta, a.x, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HB200_OK) return rc;
  }
  if (a.y_colmajor) {
    const uint64_t dims[2] = {static_cast<uint64_t>(a.K), static_cast<uint64_t>(a.N)};
    const uint64_t strides[1] = {static_cast<uint64_t>(a.ldb)};
    const uint32_t box[2] = {BK, static_cast<uint32_t>(is_pair2(c) ? pair2_width(c) / 2 : (c.pair ? 128 : c.bn))};
    int rc = encode_tmap_u8(&tb, a.y, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HB200_OK) return rc;
  } else {
    const uint64_t dims[2] = {static_cast<uint64_t>(a.N), static_cast<uint64_t>(a.K)};
    const uint64_t strides[1] = {static_cast<uint64_t>(a.ldb)};
    const uint32_t box[2] = {128, BK};
    int rc = encode_tmap_u8(&tb, a.y, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HB200_OK) return rc;
  }

  if (c.pair && c.bn == 448) return launch_pair2_by_dtype<false, 224>(a, ctx, ta, tb, c.group_m);
  if (c.pair && c.bn == 512) {
    return a.y_colmajor ? launch_pair2_by_dtype<false>(a, ctx, ta, tb, c.group_m)
                        : launch_pair2_by_dtype<true>(a, ctx, ta, tb, c.group_m);
  }
  if (c.pair) {
    return a.y_colmajor ? launch_pair_by_dtype<6, false>(a, ctx, ta, tb, c.group_m)
                        : launch_pair_by_dtype<6, true>(a, ctx, ta, tb, c.group_m);
  }
  if (a.y_colmajor) {
    switch (c.bn) {
      case 256:
        return launch_by_dtype<256, 4, false>(a, ctx, ta, tb, c.group_m);
      case 128:
        return launch_by_dtype<128, 6, false>(a, ctx, ta, tb, c.group_m, c.splits);
      case 64:
        return launch_by_dtype<64, 8, false>(a, ctx, ta, tb, c.group_m);
    }
  } else {
    switch (c.bn) {
      case 256:
        return launch_by_dtype<256, 4, true>(a, ctx, ta, tb, c.group_m);
      case 128:
        return launch_by_dtype<128, 6, true>(a, ctx, ta, tb, c.group_m, c.splits);
    }
  }
  return set_error(HB200_ERR_BAD_CONFIG, "fp8_gemm: config has no kernel instance");
}

// ------------------------------------------------------------------------------------------------
// fp16 / bf16 operands through the same kernels (hb200_gemm_16bit).  The pipelines are byte-oriented, so
// the tensor maps are built over bytes: a row of x is 2K bytes long, a 128-byte stage row is 64
// elements of K, and the kernels get K as that byte length.
// ------------------------------------------------------------------------------------------------
namespace {

template <int KIND, int OUT_DT, bool B_MN>
int launch16_row(const GemmArgs& a, DeviceCtx* ctx, const GemmConfig& c, const CUtensorMap& ta, const CUtensorMap& tb) {
  if (c.skinny || c.splits > 1 || c.bn == 64 || c.bn == 448) {
    return set_error(HB200_ERR_BAD_CONFIG, "gemm_16bit: this table row exists for e4m3 operands only");
  }
  if (c.pair && c.bn == 512) return launch_pair2_instance<B_MN, OUT_DT, KIND>(a, ctx, ta, tb, c.group_m);
  if (c.pair) return launch_pair_instance<6, B_MN, OUT_DT, KIND>(a, ctx, ta, tb, c.group_m);
  if (c.bn == 256) return launch_instance<256, 4, B_MN, OUT_DT, KIND>(a, ctx, ta, tb, c.group_m);
  return launch_instance<128, 6, B_MN, OUT_DT, KIND>(a, ctx, ta, tb, c.group_m);
}

template <int KIND, int OUT_DT>
int launch16_layout(const GemmArgs& a, DeviceCtx* ctx, const GemmConfig& c, const CUtensorMap& ta, const CUtensorMap& tb) {
  return a.y_colmajor ? launch16_row<KIND, OUT_DT, false>(a, ctx, c, ta, tb)
                      : launch16_row<KIND, OUT_DT, true>(a, ctx, c, ta, tb);
}

}  // namespace

int launch_gemm_16bit(const GemmArgs& a, DeviceCtx* ctx) {
  constexpr int64_t ES = 2;
  int cfg_id = a.cfg_id;
  if (cfg_id < 0) {
    cfg_id = gemm_select_config_nosplit(a.M, a.N, a.K * ES, a.y_colmajor, ctx->num_sms);
    if (kGemmConfigs[cfg_id].bn == 64) cfg_id = 1;  // the 64-wide tile is not built for 16-bit operands
    // Measured at 8192^3 (bf16 / fp16, either layout of y): the 256x256 pair tile runs 768-814 us, the
    // 512x256 pair tile 786-998 us -- at half the tensor rate per byte of K its exposed epilogue no longer
    // pays for the saved operand traffic.
    if (kGemmConfigs[cfg_id].bn >= 448) cfg_id = 6;
  }
  if (cfg_id >= kNumGemmConfigs) return set_error(HB200_ERR_BAD_CONFIG, "gemm_16bit: no such config");
  const GemmConfig& c = kGemmConfigs[cfg_id];

  CUtensorMap ta, tb;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(a.K * ES), static_cast<uint64_t>(a.M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(a.lda * ES)};
    const uint32_t box[2] = {BK, static_cast<uint32_t>(c.bn == 512 ? 256 : BM)};
    int rc = encode_tmap_u8(&ta, a.x, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HB200_OK) return rc;
  }
  if (a.y_colmajor) {
    const uint64_t dims[2] = {static_cast<uint64_t>(a.K * ES), static_cast<uint64_t>(a.N)};
    const uint64_t strides[1] = {static_cast<uint64_t>(a.ldb * ES)};
    const uint32_t box[2] = {BK, static_cast<uint32_t>(is_pair2(c) ? pair2_width(c) / 2 : (c.pair ? 128 : c.bn))};
    int rc = encode_tmap_u8(&tb, a.y, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HB200_OK) return rc;
  } else {
    // row-major y: rows of the map are rows of K, 2N bytes long; a box is 64 K rows x 128 bytes (64 columns)
    const uint64_t dims[2] = {static_cast<uint64_t>(a.N * ES), static_cast<uint64_t>(a.K)};
    const uint64_t strides[1] = {static_cast<uint64_t>(a.ldb * ES)};
    const uint32_t box[2] = {128, static_cast<uint32_t>(BK / ES)};
    int rc = encode_tmap_u8(&tb, a.y, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HB200_OK) return rc;
  }
  if (a.kind == KIND_F16) {
    if (a.out_dtype == HB200_DT_FP16) return launch16_layout<KIND_F16, HB200_DT_FP16>(a, ctx, c, ta, tb);
    if (a.out_dtype == HB200_DT_FP32) return launch16_layout<KIND_F16, HB200_DT_FP32>(a, ctx, c, ta, tb);
    return set_error(HB200_ERR_BAD_DTYPE, "gemm_16bit: fp16 operands give an FP16 or FP32 result");
  }
  if (a.kind == KIND_BF16) {
    if (a.out_dtype == HB200_DT_BF16) return launch16_layout<KIND_BF16, HB200_DT_BF16>(a, ctx, c, ta, tb);
    if (a.out_dtype == HB200_DT_FP32) return launch16_layout<KIND_BF16, HB200_DT_FP32>(a, ctx, c, ta, tb);
    return set_error(HB200_ERR_BAD_DTYPE, "gemm_16bit: bf16 operands give a BF16 or FP32 result");
  }
  return set_error(HB200_ERR_BAD_DTYPE, "gemm_16bit: operands must be FP16 or BF16");
}

}  // namespace hb
