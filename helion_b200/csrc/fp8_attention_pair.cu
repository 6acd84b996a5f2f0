// FP8 attention forward for sm_100a, two query tiles per CTA ("pair" rows of the attention table), with the
// numerics of pytorch-labs/helion examples/fp8_attention.py:54-105 (see fp8_attention.cu for the formulas;
// the per-row arithmetic is the shared code of attention_softmax.cuh, so a pair row that follows the running
// max gives the results of table row 0 bit for bit).
//
// Why a second pipeline.  With one query tile and one softmax warpgroup per CTA the softmax warps run a
// serial chain per key step (scores -> max -> exp2 -> rescale O -> store P) and the MUFU unit idles whenever
// both warps that share a scheduler are outside their exp2 phase.  Here one CTA per SM owns TWO 128-row query
// tiles of the same batch*head slice:
//
//   warp 0        TMA producer: the two Q tiles (double-buffered across units), K and V tiles through two rings;
//                 every K / V tile feeds both query tiles
//   warp 1        the one MMA thread.  Issue order  S0(j+1) after P0(j) V,  S1(j+1) after P1(j) V:  while the
//                 softmax warpgroup of one tile works, the tensor pipe serves the other tile (ping-pong)
//   warp 2        allocates / frees the 512 columns of tensor memory: S0 S1 (128 each), O0 O1 (D each);
//                 P (e4m3, 32 columns) overwrites the first columns of its S once the scores are in registers
//   warps 4-7     correction: rescale O in tensor memory by alpha = exp2(m_old - m_new) when a row max moved
//                 (off the softmax warps' chain: it overlaps their exp2 phase), and the epilogue out = O / l
//   warps 8-11    softmax of tile 0, warps 12-15 softmax of tile 1: one row per thread
//
// Units of work are (batch*head, pair of row blocks); the second tile of the last pair of a slice with an odd
// number of row blocks runs on zero-filled rows and stores nothing.  Non-causal only, at least two key steps
// (with a single step per unit the softmax warps could finish a second unit before the correction warps have
// looked at the first one's row sums, which a parity wait cannot tell apart); the launcher sends masked
// problems, single row blocks and up to 128 keys to the one-tile kernel.
#include <algorithm>
#include <cstdio>

#include "attention_softmax.cuh"
#include "host.h"

// Build with -DHB_PAIR_TRACE to record SM-clock stamps of the roles of CTA 0 during its second unit (a
// development aid; hb200_debug_pair_trace copies them to the host).  Product builds compile none of it.
#ifdef HB_PAIR_TRACE
namespace hb {
__device__ unsigned long long g_pair_trace[4][1024];  // softmax 0, softmax 1, correction, MMA thread
}
#define PAIR_TRACE_DECL(role) const int trace_role = (role); int trace_n = 0;
#define PAIR_TRACE(it)                                                                        \
  do {                                                                                        \
    if (blockIdx.x == 0 && (it) == 1u && (threadIdx.x & 31) == 0 && trace_n < 1024) {         \
      hb::g_pair_trace[trace_role][trace_n++] = static_cast<unsigned long long>(clock64());   \
    }                                                                                         \
  } while (0)
extern "C" __attribute__((visibility("default"))) int hb200_debug_pair_trace(unsigned long long* host_dst) {
  return static_cast<int>(cudaMemcpyFromSymbol(host_dst, hb::g_pair_trace, sizeof(unsigned long long) * 4 * 1024));
}
#else
#define PAIR_TRACE_DECL(role)
#define PAIR_TRACE(it) \
  do {                 \
  } while (0)
#endif

namespace hb {

namespace {

constexpr int PAIR_THREADS = 512;
constexpr int PAIR_BM = 128;   // rows per query tile
constexpr int PAIR_BN = 128;   // keys per step
constexpr int PAIR_TMEM_COLS = 512;

template <int D>
struct PairLayout {
  static constexpr int K_STAGES = 4;
  static constexpr int V_STAGES = K_STAGES;
  static constexpr int Q_TILE_BYTES = PAIR_BM * D;
  static constexpr int KV_TILE_BYTES = PAIR_BN * D;
  static constexpr int Q_OFFSET = 0;  // [buffer 0: tile 0, tile 1][buffer 1: tile 0, tile 1]
  static constexpr int K_OFFSET = Q_OFFSET + 4 * Q_TILE_BYTES;
  static constexpr int V_OFFSET = K_OFFSET + K_STAGES * KV_TILE_BYTES;
  static constexpr int BAR_OFFSET = V_OFFSET + V_STAGES * KV_TILE_BYTES;
  // q_full[2] q_empty[2] | per tile: s_full alpha_ready p_full o_ready pv_done l_ready | drain | k_full[] k_empty[] v_full[] v_empty[]
  static constexpr int NUM_BARS = 4 + 12 + 1 + 2 * K_STAGES + 2 * V_STAGES;
  static constexpr int ALPHA_OFFSET = BAR_OFFSET + ((NUM_BARS * 8 + 15) / 16) * 16;  // float [2][128]
  static constexpr int LFINAL_OFFSET = ALPHA_OFFSET + 2 * 128 * 4;                   // float [2 unit parities][2][128]
  static constexpr int MISC_OFFSET = LFINAL_OFFSET + 4 * 128 * 4;
  static constexpr int SMEM_BYTES = MISC_OFFSET + 32 + 1024;
  static_assert(SMEM_BYTES <= 227 * 1024, "does not fit one SM");
};

// 512 threads x 128 registers at launch -> warps 0-3: 64, correction: 88, softmax: 176 (sum = 64 K registers)
__device__ __forceinline__ void reg_set_misc() { asm volatile("setmaxnreg.dec.sync.aligned.u32 64;"); }
__device__ __forceinline__ void reg_set_correction() { asm volatile("setmaxnreg.dec.sync.aligned.u32 88;"); }
__device__ __forceinline__ void reg_set_softmax() { asm volatile("setmaxnreg.inc.sync.aligned.u32 176;"); }

template <int D, bool V_KMAJOR, int OUT_DT, int POLY_OF8, bool LAZY>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
fp8_attention_pair_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                          const __grid_constant__ CUtensorMap tmap_v, void* out, int BH, int S, int Sk,
                          int64_t out_stride_bh, int64_t out_stride_s, float scale_log2, uint32_t* status,
                          unsigned int* sched) {
  using L = PairLayout<D>;
  constexpr int KST = L::K_STAGES;
  constexpr int VST = L::V_STAGES;
  constexpr uint32_t SWZ_QK = (D == 128) ? SWZ_128B : SWZ_64B;  // rows of Q / K / V tiles are D bytes long
  constexpr uint32_t SBO_QK = 8 * D;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* q_full = bars + 0;        // [2]
  uint64_t* q_empty = bars + 2;       // [2]
  uint64_t* s_full = bars + 4;        // [2] per tile
  uint64_t* alpha_ready = bars + 6;   // [2]
  uint64_t* p_full = bars + 8;        // [2]
  uint64_t* o_ready = bars + 10;      // [2]
  uint64_t* pv_done = bars + 12;      // [2]
  uint64_t* l_ready = bars + 14;      // [2]
  uint64_t* drain = bars + 16;
  uint64_t* k_full = bars + 17;
  uint64_t* k_empty = k_full + KST;
  uint64_t* v_full = k_empty + KST;
  uint64_t* v_empty = v_full + VST;
  float* alpha_s = reinterpret_cast<float*>(smem + L::ALPHA_OFFSET);    // [tile][row]
  float* lfinal_s = reinterpret_cast<float*>(smem + L::LFINAL_OFFSET);  // [unit parity][tile][row]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::MISC_OFFSET);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::MISC_OFFSET + 4);
  volatile int* unit_q = reinterpret_cast<volatile int*>(smem + L::MISC_OFFSET + 8);  // [2], by Q buffer

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = (S + PAIR_BM - 1) / PAIR_BM;
  const int pairs = (m_tiles + 1) / 2;
  const int num_units = BH * pairs;
  const int n_steps = (Sk + PAIR_BN - 1) / PAIR_BN;
  const WaitCtx wctx{abort_flag, status};

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&q_full[b], 1);
      // the last Q K^T of the unit, and every softmax and correction thread has read the unit id
      mbar_init(&q_empty[b], 1 + 256 + 128);
      mbar_init(&s_full[b], 1);
      mbar_init(&alpha_ready[b], 128);
      mbar_init(&p_full[b], 128);
      mbar_init(&o_ready[b], 128);
      mbar_init(&pv_done[b], 1);
      mbar_init(&l_ready[b], 128);
    }
    mbar_init(drain, 1);
    for (int s = 0; s < KST; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < VST; ++s) {
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, PAIR_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // tensor-memory columns: S of tile t at 128 t (its P in the first 32 of them), O of tile t at 256 + D t

  if (warp < 4) {
    reg_set_misc();
    if (warp == 0) {
      // ------------------------------- TMA producer --------------------------------------------
      if (lane == 0) {
        uint32_t kc = 0, vc = 0;  // K / V tiles issued so far (ring positions)
        uint32_t it = 0;
        bool ok = true;
        int unit = blockIdx.x;  // gridDim.x <= num_units
        for (;; ++it) {
          const uint32_t b = it & 1u;
          // the Q buffer and the queue entry are free once the unit two back no longer needs them
          if (!mbar_wait_relaxed(&q_empty[b], ((it >> 1) & 1u) ^ 1u, wctx, SITE_ATTN_Q, 200)) {
            ok = false;
            break;
          }
          unit_q[b] = unit;
          if (unit < 0) {
            mbar_arrive(&q_full[b]);  // publishes the end marker
            break;
          }
          const int bh = unit / pairs;
          const int pr = unit - bh * pairs;
          uint8_t* qdst = smem + L::Q_OFFSET + b * 2 * L::Q_TILE_BYTES;
          mbar_arrive_expect_tx(&q_full[b], 2 * L::Q_TILE_BYTES);
          tma_load_3d(qdst, &tmap_q, &q_full[b], 0, (2 * pr) * PAIR_BM, bh);
          tma_load_3d(qdst + L::Q_TILE_BYTES, &tmap_q, &q_full[b], 0, (2 * pr + 1) * PAIR_BM, bh);
          int next = sched != nullptr ? static_cast<int>(gridDim.x + atomicAdd(sched, 1u)) : unit + static_cast<int>(gridDim.x);
          if (next >= num_units || next < 0) next = -1;
          for (int j = 0; j < n_steps && ok; ++j) {
            {
              const uint32_t s = kc % KST;
              if (!mbar_wait_relaxed(&k_empty[s], ((kc / KST) & 1u) ^ 1u, wctx, SITE_ATTN_KV_EMPTY, 200)) {
                ok = false;
                break;
              }
              mbar_arrive_expect_tx(&k_full[s], L::KV_TILE_BYTES);
              tma_load_3d(smem + L::K_OFFSET + s * L::KV_TILE_BYTES, &tmap_k, &k_full[s], 0, j * PAIR_BN, bh);
              ++kc;
            }
            {
              const uint32_t s = vc % VST;
              if (!mbar_wait_relaxed(&v_empty[s], ((vc / VST) & 1u) ^ 1u, wctx, SITE_ATTN_KV_EMPTY, 200)) {
                ok = false;
                break;
              }
              uint8_t* dst = smem + L::V_OFFSET + s * L::KV_TILE_BYTES;
              mbar_arrive_expect_tx(&v_full[s], L::KV_TILE_BYTES);
              if constexpr (V_KMAJOR) {
                tma_load_3d(dst, &tmap_v, &v_full[s], j * PAIR_BN, 0, bh);  // [D rows, 128 keys]
              } else {
                tma_load_3d(dst, &tmap_v, &v_full[s], 0, j * PAIR_BN, bh);  // [128 keys, D]
              }
              ++vc;
            }
          }
          if (!ok) break;
          unit = next;
        }
        if (!ok) {
          // wait (bounded) for the copies in flight before the CTA may exit
          mbar_drain(&q_full[it & 1u], (it >> 1) & 1u);
          const uint32_t kb = kc < static_cast<uint32_t>(KST) ? kc : static_cast<uint32_t>(KST);
          for (uint32_t i = kc - kb; i < kc; ++i) mbar_drain(&k_full[i % KST], (i / KST) & 1u);
          const uint32_t vb = vc < static_cast<uint32_t>(VST) ? vc : static_cast<uint32_t>(VST);
          for (uint32_t i = vc - vb; i < vc; ++i) mbar_drain(&v_full[i % VST], (i / VST) & 1u);
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      // ------------------------------- the MMA thread --------------------------------------------
      if (lane == 0) {
        constexpr uint32_t idesc_qk = make_idesc_e4m3(PAIR_BM, PAIR_BN, false, false);
        constexpr uint32_t idesc_pv = make_idesc_e4m3(PAIR_BM, D, false, !V_KMAJOR);
        const uint32_t q_addr = smem_u32(smem + L::Q_OFFSET);
        const uint32_t k_addr = smem_u32(smem + L::K_OFFSET);
        const uint32_t v_addr = smem_u32(smem + L::V_OFFSET);
        uint32_t kc = 0, vc = 0;  // K tiles used by a Q K^T pair / V tiles used by a P V pair so far
        uint32_t pg = 0;          // key steps completed so far (phases of p_full / o_ready)
        bool ok = true;
        PAIR_TRACE_DECL(3)

        // S_t = Q_t K^T of one key step into tile t's score columns
        auto issue_qk = [&](int t, uint32_t qb, uint32_t ks) {
          const uint64_t q_desc = make_smem_desc(q_addr + (qb * 2 + t) * L::Q_TILE_BYTES, 16, SBO_QK, SWZ_QK);
          const uint64_t k_desc = make_smem_desc(k_addr + ks * L::KV_TILE_BYTES, 16, SBO_QK, SWZ_QK);
#pragma unroll
          for (int k = 0; k < D / 32; ++k) {
            umma_f8_ss(tmem_base + t * 128, desc_advance(q_desc, k * 32), desc_advance(k_desc, k * 32), idesc_qk,
                       k != 0 ? 1u : 0u);
          }
          umma_commit(&s_full[t]);
        };
        // O_t (+)= P_t V with P read from tensor memory
        auto issue_pv = [&](int t, uint32_t vs, bool first) {
          const uint32_t va = v_addr + vs * L::KV_TILE_BYTES;
          // V [keys, D] with D contiguous: MN-major B, one swizzle-wide block of N, 8 key rows per atom.
          // V [D, keys] with keys contiguous: K-major B with 128-byte rows.
          const uint64_t v_desc = V_KMAJOR ? make_smem_desc(va, 16, 8 * PAIR_BN, SWZ_128B)
                                           : make_smem_desc(va, SBO_QK, SBO_QK, SWZ_QK);
#pragma unroll
          for (int k = 0; k < PAIR_BN / 32; ++k) {
            const uint64_t vd = desc_advance(v_desc, V_KMAJOR ? k * 32 : k * 32 * D);
            umma_f8_ts(tmem_base + 256 + t * D, tmem_base + t * 128 + k * 8, vd, idesc_pv, (!first || k != 0) ? 1u : 0u);
          }
          umma_commit(&pv_done[t]);
        };

        uint32_t it = 0;
        int unit = -1;
        if (mbar_wait(&q_full[0], 0, wctx, SITE_ATTN_Q)) {
          unit = unit_q[0];
        } else {
          ok = false;
        }
        if (ok && unit >= 0) {
          // the first key step of the first unit: both score tiles, nothing to overlap with yet
          const uint32_t ks = kc % KST;
          if (mbar_wait(&k_full[ks], (kc / KST) & 1u, wctx, SITE_ATTN_K_FULL)) {
            tc_fence_after_sync();
            issue_qk(0, 0, ks);
            issue_qk(1, 0, ks);
            umma_commit(&k_empty[ks]);
            if (n_steps == 1) umma_commit(&q_empty[0]);
            ++kc;
          } else {
            ok = false;
          }
        }
        while (ok && unit >= 0) {
          const uint32_t b = it & 1u;
          int next_unit = -1;
          for (int j = 0; j < n_steps; ++j, ++pg) {
            const bool last = j + 1 == n_steps;
            uint32_t qb = b;  // Q buffer of the score tiles issued in this step
            if (last) {
              // the scores issued now are the first key step of the next unit
              qb = b ^ 1u;
              if (!mbar_wait(&q_full[qb], ((it + 1) >> 1) & 1u, wctx, SITE_ATTN_Q)) {
                ok = false;
                break;
              }
              next_unit = unit_q[qb];
            }
            const bool more = !last || next_unit >= 0;
            const int next_j = last ? 0 : j + 1;
            const uint32_t ks = kc % KST;
            const uint32_t vs = vc % VST;
            if ((more && !mbar_wait(&k_full[ks], (kc / KST) & 1u, wctx, SITE_ATTN_K_FULL)) ||
                !mbar_wait(&v_full[vs], (vc / VST) & 1u, wctx, SITE_ATTN_V_FULL)) {
              ok = false;
              break;
            }
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              if (!mbar_wait(&p_full[t], pg & 1u, wctx, SITE_ATTN_P_FULL) ||
                  !mbar_wait(&o_ready[t], pg & 1u, wctx, SITE_ATTN_O_READY)) {
                ok = false;
                break;
              }
              tc_fence_after_sync();
              PAIR_TRACE(it);
              issue_pv(t, vs, j == 0);
              if (t == 1) umma_commit(&v_empty[vs]);
              if (more) {
                issue_qk(t, qb, ks);
                if (t == 1) {
                  umma_commit(&k_empty[ks]);
                  if (next_j + 1 == n_steps) umma_commit(&q_empty[qb]);
                }
              }
              PAIR_TRACE(it);
            }
            if (!ok) break;
            ++vc;
            if (more) ++kc;
          }
          if (!ok) break;
          unit = next_unit;
          ++it;
        }
        if (!ok) {
          umma_commit(drain);
          mbar_drain(drain, 0);
        }
      }
      __syncwarp();
    }
  } else if (warp < 8) {
    // --------------------------------- correction / epilogue -------------------------------------
    reg_set_correction();
    const int row_in_tile = (warp & 3) * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint32_t pg = 0;  // key steps so far (phases of alpha_ready and pv_done, the same for both tiles)
    bool ok = true;
    PAIR_TRACE_DECL(2)
    for (uint32_t it = 0; ok; ++it) {
      const uint32_t b = it & 1u;
      ok = mbar_wait(&q_full[b], (it >> 1) & 1u, wctx, SITE_ATTN_Q);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int unit = unit_q[b];
      mbar_arrive(&q_empty[b]);
      if (unit < 0) break;
      const int bh = unit / pairs;
      const int pr = unit - bh * pairs;
      for (int j = 0; j < n_steps && ok; ++j, ++pg) {
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          ok = mbar_wait(&alpha_ready[t], pg & 1u, wctx, SITE_ATTN_ALPHA);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          PAIR_TRACE(it);
          if (j > 0) {
            const float alpha = alpha_s[t * 128 + row_in_tile];
            if (__any_sync(0xffffffffu, alpha != 1.0f)) {
              // the previous P V of this tile must have landed before O is touched
              ok = mbar_wait(&pv_done[t], (pg - 1u) & 1u, wctx, SITE_ATTN_PV_DONE);
              ok = __all_sync(0xffffffffu, ok);
              if (!ok) break;
              tc_fence_after_sync();
              const uint32_t t_o = tmem_base + 256 + t * D + lane_sel;
#pragma unroll
              for (int c = 0; c < D / 32; ++c) {
                uint32_t o[32];
                tmem_ld_32x32b_x32(t_o + c * 32, o);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                tmem_st_32x32b_x32(t_o + c * 32, o);
              }
              tmem_wait_st();
            }
          }
          tc_fence_before_sync();
          mbar_arrive(&o_ready[t]);  // O of tile t may be accumulated into (overwritten when j == 0)
          PAIR_TRACE(it);
        }
      }
      if (!ok) break;
      // ---- epilogue of the unit: out = O / l for both tiles ---------------------------------------
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        ok = mbar_wait(&l_ready[t], it & 1u, wctx, SITE_ATTN_ALPHA);  // the row sums are final (one phase per unit)
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const float l_i = lfinal_s[(b * 2 + t) * 128 + row_in_tile];
        ok = mbar_wait(&pv_done[t], (pg - 1u) & 1u, wctx, SITE_ATTN_O_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        const int row = (2 * pr + t) * PAIR_BM + row_in_tile;
        const int64_t out_off = static_cast<int64_t>(bh) * out_stride_bh + static_cast<int64_t>(row) * out_stride_s;
        const uint32_t t_o = tmem_base + 256 + t * D + lane_sel;
        // The 8- and 16-bit outputs divide through the correctly rounded reciprocal with one residual
        // correction (div_by_rcp); the fp32 output keeps the IEEE division.
        const float inv_l = __frcp_rn(l_i);
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {  // rolled: runs once per unit, and the roles' hot loops share an instruction cache
          uint32_t o[32];
          tmem_ld_32x32b_x32(t_o + c * 32, o);
          tmem_wait_ld();
          if (row < S) {
            if constexpr (OUT_DT == HB200_DT_E4M3) {
              uint32_t w[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                w[i] = pack_e4m3x4(div_by_rcp(__uint_as_float(o[4 * i]), l_i, inv_l),
                                   div_by_rcp(__uint_as_float(o[4 * i + 1]), l_i, inv_l),
                                   div_by_rcp(__uint_as_float(o[4 * i + 2]), l_i, inv_l),
                                   div_by_rcp(__uint_as_float(o[4 * i + 3]), l_i, inv_l));
              }
              uint8_t* dst = reinterpret_cast<uint8_t*>(out) + out_off + c * 32;
              *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
              *reinterpret_cast<uint4*>(dst + 16) = make_uint4(w[4], w[5], w[6], w[7]);
            } else if constexpr (OUT_DT == HB200_DT_BF16) {
              uint16_t* dst = reinterpret_cast<uint16_t*>(out) + out_off + c * 32;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint32_t w[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                  w[k] = pack_bf16x2(div_by_rcp(__uint_as_float(o[8 * i + 2 * k]), l_i, inv_l),
                                     div_by_rcp(__uint_as_float(o[8 * i + 2 * k + 1]), l_i, inv_l));
                }
                *reinterpret_cast<uint4*>(dst + i * 8) = make_uint4(w[0], w[1], w[2], w[3]);
              }
            } else {
              float* dst = reinterpret_cast<float*>(out) + out_off + c * 32;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                float4 v;
                v.x = __fdiv_rn(__uint_as_float(o[4 * i]), l_i);
                v.y = __fdiv_rn(__uint_as_float(o[4 * i + 1]), l_i);
                v.z = __fdiv_rn(__uint_as_float(o[4 * i + 2]), l_i);
                v.w = __fdiv_rn(__uint_as_float(o[4 * i + 3]), l_i);
                *reinterpret_cast<float4*>(dst + i * 4) = v;
              }
            }
          }
        }
        // O is read: this thread's next arrival on o_ready[t] (first step of the next unit) lets the next
        // P V overwrite it
        tc_fence_before_sync();
      }
    }
  } else {
    // --------------------------------- softmax of tile t ------------------------------------------
    reg_set_softmax();
    const int t = (warp - 8) >> 2;
    const int row_in_tile = (warp & 3) * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem_base + t * 128 + lane_sel;  // scores; P goes into the first 32 of these columns
    uint32_t g = 0;  // key steps so far (phases of s_full[t])
    bool ok = true;
    PAIR_TRACE_DECL(t)
    for (uint32_t it = 0; ok; ++it) {
      const uint32_t b = it & 1u;
      ok = mbar_wait(&q_full[b], (it >> 1) & 1u, wctx, SITE_ATTN_Q);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int unit = unit_q[b];
      mbar_arrive(&q_empty[b]);
      if (unit < 0) break;
      float m_i = -INFINITY;
      float l_i = 0.0f;
      for (int j = 0; j < n_steps; ++j, ++g) {
        ok = mbar_wait(&s_full[t], g & 1u, wctx, SITE_ATTN_S_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        PAIR_TRACE(it);
        uint32_t s[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(t_s + c * 32, s[c]);
        tmem_wait_ld();
        PAIR_TRACE(it);
        const int valid = Sk - j * PAIR_BN;  // keys of this step that exist
        if (valid < PAIR_BN) mask_scores128(s, valid);
        const float mx = row_max128(s);
        // Exact rows follow the running max (examples/fp8_attention.py:76-78).  Lazy rows keep the previous
        // reference point while the max has grown by at most 2^8 (p <= 256 fits e4m3; O and l stay
        // consistent because both use the same reference point).
        const float cand = fmaxf(m_i, mx * scale_log2);
        const bool moved = LAZY ? (cand - m_i > 8.0f) : (cand > m_i);
        const float m_new = (LAZY && !moved) ? m_i : cand;
        const float alpha = moved ? fast_exp2(m_i - m_new) : 1.0f;
        alpha_s[t * 128 + row_in_tile] = alpha;
        mbar_arrive(&alpha_ready[t]);  // the correction warps rescale O while this warp exponentiates
        PAIR_TRACE(it);

        const uint64_t c2 = pack2f(scale_log2, scale_log2);
        const uint64_t negm2 = pack2f(-m_new, -m_new);
        uint64_t sum_a = 0ull, sum_b = 0ull;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t packed[8];
          exp_chunk32<POLY_OF8>(s[c], c, c2, negm2, sum_a, sum_b, packed);
          // word w of a row = keys 4w .. 4w+3 = column w of the row's lane
          tmem_st_32x32b_x8(t_s + c * 8, packed);
        }
        {
          uint32_t sl, sh;
          unpack2(fadd2(sum_a, sum_b), sl, sh);
          l_i = l_i * alpha + (__uint_as_float(sl) + __uint_as_float(sh));
        }
        PAIR_TRACE(it);
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(&p_full[t]);
        PAIR_TRACE(it);
        m_i = m_new;
      }
      if (!ok) break;
      // A barrier of its own: on alpha_ready this arrival could complete a second phase before the
      // correction warps have looked at the last step's, and a parity wait cannot see two phases.
      lfinal_s[(b * 2 + t) * 128 + row_in_tile] = l_i;
      mbar_arrive(&l_ready[t]);
    }
  }

  // ------------------------------- teardown ------------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    __syncwarp();
    tmem_dealloc(tmem_base, PAIR_TMEM_COLS);
  }
}

template <int D, bool V_KMAJOR, int OUT_DT, int POLY_OF8, bool LAZY>
int launch_pair_instance(const AttnArgs& a, DeviceCtx* ctx, const CUtensorMap& tq, const CUtensorMap& tk,
                         const CUtensorMap& tv) {
  using L = PairLayout<D>;
  auto kernel = fp8_attention_pair_kernel<D, V_KMAJOR, OUT_DT, POLY_OF8, LAZY>;
  static std::atomic<uint64_t> smem_attr_done{0};
  HB_CUDA_CHECK(set_max_dynamic_smem_once(smem_attr_done, reinterpret_cast<const void*>(kernel), L::SMEM_BYTES, a.device));
  const int64_t m_tiles = (a.S + PAIR_BM - 1) / PAIR_BM;
  const int64_t num_units = a.BH * ((m_tiles + 1) / 2);
  if (num_units > INT32_MAX / 2) return set_error(HB200_ERR_BAD_SHAPE, "fp8_attention: too many tiles");
  const int grid = static_cast<int>(std::min<int64_t>(num_units, ctx->num_sms));
  kernel<<<grid, PAIR_THREADS, L::SMEM_BYTES, a.stream>>>(tq, tk, tv, a.out, static_cast<int>(a.BH),
                                                          static_cast<int>(a.S), static_cast<int>(a.Sk),
                                                          a.out_strides[0], a.out_strides[1], a.scale_log2,
                                                          ctx->status_dev, a.sched);
  HB_CUDA_CHECK(cudaGetLastError());
  return HB200_OK;
}

template <int D, bool V_KMAJOR, int OUT_DT>
int launch_pair_by_row(const AttnArgs& a, DeviceCtx* ctx, const CUtensorMap& tq, const CUtensorMap& tk,
                       const CUtensorMap& tv, int poly_of8, bool lazy) {
  if (lazy) {
    if (poly_of8 == 4) return launch_pair_instance<D, V_KMAJOR, OUT_DT, 4, true>(a, ctx, tq, tk, tv);
    return set_error(HB200_ERR_BAD_CONFIG, "fp8_attention: config has no kernel instance");
  }
  switch (poly_of8) {
    case 0:
      return launch_pair_instance<D, V_KMAJOR, OUT_DT, 0, false>(a, ctx, tq, tk, tv);
    case 2:
      return launch_pair_instance<D, V_KMAJOR, OUT_DT, 2, false>(a, ctx, tq, tk, tv);
    case 4:
      return launch_pair_instance<D, V_KMAJOR, OUT_DT, 4, false>(a, ctx, tq, tk, tv);
    default:
      return set_error(HB200_ERR_BAD_CONFIG, "fp8_attention: config has no kernel instance");
  }
}

template <int D, bool V_KMAJOR>
int launch_pair_by_dtype(const AttnArgs& a, DeviceCtx* ctx, const CUtensorMap& tq, const CUtensorMap& tk,
                         const CUtensorMap& tv, int poly_of8, bool lazy) {
  switch (a.out_dtype) {
    case HB200_DT_E4M3:
      return launch_pair_by_row<D, V_KMAJOR, HB200_DT_E4M3>(a, ctx, tq, tk, tv, poly_of8, lazy);
    case HB200_DT_BF16:
      return launch_pair_by_row<D, V_KMAJOR, HB200_DT_BF16>(a, ctx, tq, tk, tv, poly_of8, lazy);
    case HB200_DT_FP32:
      return launch_pair_by_row<D, V_KMAJOR, HB200_DT_FP32>(a, ctx, tq, tk, tv, poly_of8, lazy);
    default:
      return set_error(HB200_ERR_BAD_DTYPE, "fp8_attention: unsupported out_dtype");
  }
}

}  // namespace

// Tensor maps as the one-tile kernel builds them for 128-key steps (Q box [128, D], K / V box [128 keys, D] or
// [D, 128 keys]).
int launch_fp8_attention_pair(const AttnArgs& a, DeviceCtx* ctx, const CUtensorMap& tq, const CUtensorMap& tk,
                              const CUtensorMap& tv, bool v_kmajor, int poly_of8, bool lazy) {
  if (a.causal) return set_error(HB200_ERR_BAD_CONFIG, "fp8_attention: the two-tile rows have no causal mask");
  if (a.D == 64) {
    return v_kmajor ? launch_pair_by_dtype<64, true>(a, ctx, tq, tk, tv, poly_of8, lazy)
                    : launch_pair_by_dtype<64, false>(a, ctx, tq, tk, tv, poly_of8, lazy);
  }
  return v_kmajor ? launch_pair_by_dtype<128, true>(a, ctx, tq, tk, tv, poly_of8, lazy)
                  : launch_pair_by_dtype<128, false>(a, ctx, tq, tk, tv, poly_of8, lazy);
}

}  // namespace hb
