// FP8 attention forward for sm_100a with the numerics of pytorch-labs/helion's
// examples/fp8_attention.py:54-105 (non-causal, seq_k = seq_q there; a separate key length and a
// bottom-right-aligned causal mask are extensions, see steps_of / `visible` below):
//   s = (q k^T) * c            e4m3 x e4m3 -> fp32,  c = log2(e)/sqrt(D)
//   m = running row max, p = exp2(s - m), l = l*alpha + rowsum(p)   (fp32, online softmax)
//   acc = acc*alpha + e4m3(p) v                                     (P cast to e4m3 un-normalised)
//   out = cast(acc / l)
//
// One CTA owns one (batch*head, 128-query-row) tile at a time and walks the keys in steps of 128;
// CTAs are persistent, two per SM, so that one CTA's softmax overlaps the other's MMAs.  The
// producer hands out tiles: statically (blockIdx.x, + gridDim.x, ...) or, when the caller passes a
// zeroed counter, from that counter, which evens out the different speeds of co-resident CTAs and
// the last partial round.  Tile ids reach the other roles through a two-entry queue in shared
// memory that rides on the Q barriers; -1 ends the kernel.
//
//   one warp    TMA producer: Q tile, then K/V tiles through one ring of smem slots
//   one warp    MMA thread 1: S = Q K^T into tensor memory; tcgen05.commit publishes S and frees K slots
//   one warp    MMA thread 2: O += P V with P read from shared memory (from tensor memory for head_dim 64
//               with 128-key steps, where 64 columns are spare); tcgen05.commit frees V slots
//               and publishes O.  (Which of warps 0-3 takes which role depends on which of the SM's
//               CTAs this is, so that the MMA threads of co-resident CTAs sit on different schedulers.)
//   warp 2      also allocates and frees the tensor memory
//   warps 4-7   softmax: each thread owns one query row: pulls its 128 scores out of tensor memory
//               into registers (which frees S for the next Q K^T at once), row max, exp2, row sum,
//               e4m3 P into 128B-swizzled smem (or tensor memory), rescales O in tensor memory when the max moved,
//               and writes the normalised output at the end of the tile
//
// V is accepted in both physical layouts of the reference's "[BH, D, S]" argument: D contiguous
// (B operand of P V is MN-major) or S contiguous (K-major).
#include <algorithm>
#include <cmath>
#include <cstdio>

#include "common.cuh"
#include "host.h"

namespace hb {

namespace {

constexpr int ATT_BM = 128;  // query rows per tile (= UMMA M, one row per softmax thread)
// keys per step: template parameter BN (128, or 64 for head_dim 64 where four CTAs fit one SM)
constexpr int ATT_THREADS = 256;
constexpr int ATT_SOFTMAX_THREADS = 128;
// tensor memory: S in columns [0, BN), O in columns [BN, BN + D); allocation = next power of two

template <int D, int BN>
struct AttnLayout {
  static constexpr int CTAS_PER_SM = (D == 64 && BN == 64) ? 4 : 2;
  static constexpr int TMEM_COLS = (BN + D <= 128) ? 128 : 256;
  static constexpr int KV_STAGES = (BN == 64) ? 8 : ((D == 64) ? 8 : 4);
  static constexpr int Q_BYTES = 128 * D;    // the Q tile
  static constexpr int TILE_BYTES = BN * D;  // one K or V tile
  static constexpr int Q_OFFSET = 0;
  static constexpr int P_OFFSET = Q_BYTES;                    // 128 x BN e4m3
  static constexpr int KV_OFFSET = P_OFFSET + ATT_BM * BN;
  static constexpr int BAR_OFFSET = KV_OFFSET + KV_STAGES * TILE_BYTES;
  // q_full q_empty s_full s_free p_full pv_done drain kv_full[ST] kv_empty[ST]
  static constexpr int NUM_BARS = 8 + 2 * KV_STAGES;  // + drain of the second MMA thread, last
  static constexpr int MISC_OFFSET = BAR_OFFSET + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = MISC_OFFSET + 16 + 1024;
  static_assert(SMEM_BYTES <= (CTAS_PER_SM == 4 ? 56 : 113) * 1024, "the CTAs must fit one SM together");
};

// two CTAs per SM: 256 threads x 128 registers at launch -> 128 x 56 + 128 x 200
// four CTAs per SM: 256 threads x 64 registers at launch -> 128 x 24 + 128 x 104
template <int CTAS>
__device__ __forceinline__ void reg_dec_wg0() {
  if constexpr (CTAS == 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 24;");
  else asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
}
template <int CTAS>
__device__ __forceinline__ void reg_inc_softmax() {
  if constexpr (CTAS == 4) asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
  else asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
}

template <int D, int BN, bool V_KMAJOR, int OUT_DT, int POLY_OF8, bool LAZY>
__global__ void __launch_bounds__(ATT_THREADS, (D == 64 && BN == 64) ? 4 : 2)
fp8_attention_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, void* out, int BH, int S, int Sk, int causal_off,
                     int64_t out_stride_bh,
                     int64_t out_stride_s, float scale_log2, uint32_t* status, unsigned int* sched) {
  using L = AttnLayout<D, BN>;
  constexpr int ST = L::KV_STAGES;
  constexpr int ATT_BN = BN;
  constexpr int ATT_O_COL = BN;
  constexpr int ATT_TMEM_COLS = L::TMEM_COLS;
  // P rows are BN bytes long: 128-byte or 64-byte swizzle, 8-row atoms
  // head_dim 64 with 128-key steps leaves 64 of the 256 tensor-memory columns unused: P (128 x 128 e4m3 =
  // 32 columns) lives there and P V reads its A operand from tensor memory -- no smem round trip, no
  // generic-to-async proxy fence, and the P V instructions fetch only V from shared memory.
  constexpr bool P_TMEM = D == 64 && BN == 128;
  constexpr int ATT_P_COL = BN + D;
  constexpr uint32_t SWZ_P = (BN == 128) ? SWZ_128B : SWZ_64B;
  constexpr uint32_t SBO_P = 8 * BN;
  constexpr uint32_t SWZ_QK = (D == 128) ? SWZ_128B : SWZ_64B;  // rows of Q/K/V tiles are D bytes long
  constexpr uint32_t SBO_QK = 8 * D;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* q_full = bars + 0;
  uint64_t* q_empty = bars + 1;
  uint64_t* s_full = bars + 2;
  uint64_t* s_free = bars + 3;
  uint64_t* p_full = bars + 4;
  uint64_t* pv_done = bars + 5;
  uint64_t* drain = bars + 6;
  uint64_t* kv_full = bars + 7;
  uint64_t* kv_empty = bars + 7 + ST;
  uint64_t* drain_pv = bars + 7 + 2 * ST;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::MISC_OFFSET);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::MISC_OFFSET + 4);
  volatile int* tile_q = reinterpret_cast<volatile int*>(smem + L::MISC_OFFSET + 8);  // [2], indexed by tile parity

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = (S + ATT_BM - 1) / ATT_BM;
  // S query rows, Sk keys.  causal_off < 0: no mask.  Otherwise query row i sees keys 0 .. i + causal_off
  // (causal_off = Sk - S: the diagonal ends in the bottom-right corner), a tile only walks the key steps
  // some of its rows can see, and tiles are handed out longest first within a batch*head slice.
  const bool causal = causal_off >= 0;
  const int n_steps_all = (Sk + ATT_BN - 1) / ATT_BN;
  auto steps_of = [&](int mt) -> int {
    if (!causal) return n_steps_all;
    const int last_key = min(Sk - 1, mt * ATT_BM + ATT_BM - 1 + causal_off);
    return last_key / ATT_BN + 1;
  };
  auto row_block_of = [&](int tile, int bh) -> int {
    const int t = tile - bh * m_tiles;
    return causal ? m_tiles - 1 - t : t;
  };
  const int num_tiles = BH * m_tiles;
  const WaitCtx wctx{abort_flag, status};

  if (threadIdx.x == 0) {
    // descriptor fetches overlap the barrier set-up and the tensor-memory allocation
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    mbar_init(q_full, 1);
    // last Q K^T of the tile + every softmax thread and the P V thread have the tile id
    mbar_init(q_empty, 2 + ATT_SOFTMAX_THREADS);
    mbar_init(s_full, 1);
    mbar_init(s_free, ATT_SOFTMAX_THREADS);
    mbar_init(p_full, ATT_SOFTMAX_THREADS);
    mbar_init(pv_done, 1);
    mbar_init(drain, 1);
    mbar_init(drain_pv, 1);
    for (int s = 0; s < ST; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, ATT_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // Which warp plays which role depends on which of the SM's CTAs this is (read off the tensor-memory
  // columns it was given): issuing a tcgen05 instruction occupies its scheduler for tens of cycles, and
  // every scheduler also hosts one softmax warp of each resident CTA, so the two MMA threads of the
  // two CTAs are spread over all four schedulers instead of loading one of them with everything.
  const uint32_t sm_slot = ((tmem_base & 0xffffu) / ATT_TMEM_COLS) & 1u;
  const int w_producer = sm_slot ? 1 : 0;
  const int w_qk = sm_slot ? 2 : 1;
  const int w_pv = sm_slot ? 0 : 3;
  if (warp < 4) {
    reg_dec_wg0<L::CTAS_PER_SM>();
    if (warp == w_producer) {
      // ------------------------------- TMA producer ------------------------------------------
      if (lane == 0) {
        uint32_t slot_it = 0;  // running K/V tile counter (ring position)
        uint32_t tile_iter = 0;
        bool ok = true;
        int tile = blockIdx.x;  // gridDim.x <= num_tiles
        for (;; ++tile_iter) {
          // Q buffer and queue entry of this parity are free once the tile two back is done with them
          if (!mbar_wait_relaxed(q_empty, (tile_iter & 1u) ^ 1u, wctx, SITE_ATTN_Q, 200)) {
            ok = false;
            break;
          }
          tile_q[tile_iter & 1u] = tile;
          if (tile < 0) {
            mbar_arrive(q_full);  // publishes the end marker
            break;
          }
          const int bh = tile / m_tiles;
          const int mt = row_block_of(tile, bh);
          const int n_steps = steps_of(mt);
          mbar_arrive_expect_tx(q_full, L::Q_BYTES);
          tma_load_3d(smem + L::Q_OFFSET, &tmap_q, q_full, 0, mt * ATT_BM, bh);
          // the next tile: asked for now, needed after this tile's loads are issued
          int next = sched != nullptr ? static_cast<int>(gridDim.x + atomicAdd(sched, 1u)) : tile + static_cast<int>(gridDim.x);
          if (next >= num_tiles || next < 0) next = -1;
          for (int j = 0; j < n_steps && ok; ++j) {
#pragma unroll
            for (int kv = 0; kv < 2; ++kv, ++slot_it) {
              const uint32_t s = slot_it % ST;
              const uint32_t ph = (slot_it / ST) & 1u;
              if (!mbar_wait_relaxed(&kv_empty[s], ph ^ 1u, wctx, SITE_ATTN_KV_EMPTY, 200)) {
                ok = false;
                break;
              }
              uint8_t* dst = smem + L::KV_OFFSET + s * L::TILE_BYTES;
              mbar_arrive_expect_tx(&kv_full[s], L::TILE_BYTES);
              if (kv == 0) {
                tma_load_3d(dst, &tmap_k, &kv_full[s], 0, j * ATT_BN, bh);
              } else if constexpr (V_KMAJOR) {
                tma_load_3d(dst, &tmap_v, &kv_full[s], j * ATT_BN, 0, bh);  // [D rows, 128 keys]
              } else {
                tma_load_3d(dst, &tmap_v, &kv_full[s], 0, j * ATT_BN, bh);  // [128 keys, D]
              }
            }
          }
          if (!ok) break;
          tile = next;
        }
        if (!ok) {
          mbar_drain(q_full, tile_iter & 1u);
          const uint32_t back = slot_it < static_cast<uint32_t>(ST) ? slot_it : static_cast<uint32_t>(ST);
          for (uint32_t i = slot_it - back; i < slot_it; ++i) mbar_drain(&kv_full[i % ST], (i / ST) & 1u);
        }
      }
      __syncwarp();
    } else if (warp == w_qk) {
      // ------------------------------- MMA thread 1: S = Q K^T -------------------------------
      if (lane == 0) {
        constexpr uint32_t idesc_qk = make_idesc_e4m3(ATT_BM, ATT_BN, false, false);
        const uint32_t q_addr = smem_u32(smem + L::Q_OFFSET);
        const uint32_t kv_addr = smem_u32(smem + L::KV_OFFSET);
        const uint32_t t_s = tmem_base;
        const uint64_t q_desc = make_smem_desc(q_addr, 16, SBO_QK, SWZ_QK);
        uint32_t g = 0;        // running step counter: phases of s_full / s_free
        uint32_t slot_it = 0;  // ring position of this step's K tile (its V tile is the next one)
        uint32_t tile_iter = 0;
        bool ok = true;
        for (; ok; ++tile_iter) {
          if (!mbar_wait_relaxed(q_full, tile_iter & 1u, wctx, SITE_ATTN_Q, 100)) {
            ok = false;
            break;
          }
          const int tile = tile_q[tile_iter & 1u];
          if (tile < 0) break;  // no more tiles
          const int n_steps = steps_of(row_block_of(tile, tile / m_tiles));
          for (int j = 0; j < n_steps; ++j, ++g, slot_it += 2) {
            // waits for the K tile and for S to be free (the softmax warps have pulled step g-1 out)
            const uint32_t s = slot_it % ST;
            if (!mbar_wait_relaxed(&kv_full[s], (slot_it / ST) & 1u, wctx, SITE_ATTN_K_FULL, 100) ||
                (g > 0 && !mbar_wait_relaxed(s_free, (g - 1u) & 1u, wctx, SITE_ATTN_S_FREE, 100))) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
            const uint64_t k_desc = make_smem_desc(kv_addr + s * L::TILE_BYTES, 16, SBO_QK, SWZ_QK);
#pragma unroll
            for (int k = 0; k < D / 32; ++k) {
              umma_f8_ss(t_s, desc_advance(q_desc, k * 32), desc_advance(k_desc, k * 32), idesc_qk, k != 0 ? 1u : 0u);
            }
            umma_commit(&kv_empty[s]);
            if (j + 1 == n_steps) umma_commit(q_empty);
            umma_commit(s_full);
          }
        }
        if (!ok) {
          umma_commit(drain);
          mbar_drain(drain, 0);
        }
      }
      __syncwarp();
    } else if (warp == w_pv) {
      // ------------------------------- MMA thread 2: O (+)= P V ------------------------------
      // Ordered against thread 1 by the barriers alone: P V of step g starts after p_full(g), which
      // the softmax warps signal after pv_done(g-1); Q K^T of step g+1 only touches S.
      if (lane == 0) {
        constexpr uint32_t idesc_pv = make_idesc_e4m3(ATT_BM, D, false, !V_KMAJOR);
        const uint32_t p_addr = smem_u32(smem + L::P_OFFSET);
        const uint32_t kv_addr = smem_u32(smem + L::KV_OFFSET);
        const uint32_t t_o = tmem_base + ATT_O_COL;
        const uint64_t p_desc = make_smem_desc(p_addr, 16, SBO_P, SWZ_P);
        uint32_t g = 0;        // running step counter: phases of p_full / pv_done
        uint32_t slot_it = 0;  // ring position of this step's K tile; V is slot_it + 1
        uint32_t tile_iter = 0;
        bool ok = true;
        for (; ok; ++tile_iter) {
          if (!mbar_wait_relaxed(q_full, tile_iter & 1u, wctx, SITE_ATTN_Q, 100)) {
            ok = false;
            break;
          }
          const int tile = tile_q[tile_iter & 1u];
          mbar_arrive(q_empty);  // this thread has the id (keeps q_full from running two phases ahead of it)
          if (tile < 0) break;
          const int n_steps = steps_of(row_block_of(tile, tile / m_tiles));
          for (int j = 0; j < n_steps; ++j, ++g, slot_it += 2) {
            const uint32_t vs = (slot_it + 1) % ST;
            if (!mbar_wait_relaxed(&kv_full[vs], ((slot_it + 1) / ST) & 1u, wctx, SITE_ATTN_V_FULL, 100) ||
                !mbar_wait_relaxed(p_full, g & 1u, wctx, SITE_ATTN_P_FULL, 100)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
            const uint32_t v_addr = kv_addr + vs * L::TILE_BYTES;
            // V [keys, D] with D contiguous: MN-major B, one swizzle-wide block of N, 8 key rows per
            // atom.  V [D, keys] with keys contiguous: K-major B with 128-byte rows.
            const uint64_t v_desc = V_KMAJOR ? make_smem_desc(v_addr, 16, SBO_P, SWZ_P)
                                             : make_smem_desc(v_addr, SBO_QK, SBO_QK, SWZ_QK);
#pragma unroll
            for (int k = 0; k < ATT_BN / 32; ++k) {
              const uint64_t pd = desc_advance(p_desc, k * 32);
              const uint64_t vd = desc_advance(v_desc, V_KMAJOR ? k * 32 : k * 32 * D);
              if constexpr (P_TMEM) {
                umma_f8_ts(t_o, tmem_base + ATT_P_COL + k * 8, vd, idesc_pv, (j | k) != 0 ? 1u : 0u);
              } else {
                umma_f8_ss(t_o, pd, vd, idesc_pv, (j | k) != 0 ? 1u : 0u);
              }
            }
            umma_commit(&kv_empty[vs]);
            umma_commit(pv_done);
          }
        }
        if (!ok) {
          umma_commit(drain_pv);
          mbar_drain(drain_pv, 0);
        }
      }
      __syncwarp();
    }
  } else {
    // --------------------------------- softmax / epilogue --------------------------------------
    reg_inc_softmax<L::CTAS_PER_SM>();
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t t_s = tmem_base + lane_sel;
    const uint32_t t_o = tmem_base + ATT_O_COL + lane_sel;
    // P tile: BN-byte rows, 16-byte chunks XOR-swizzled with (row % 8) for 128-byte rows or with
    // ((row >> 1) % 4) for 64-byte rows
    uint8_t* p_row = smem + L::P_OFFSET + row_in_tile * BN;
    const uint32_t p_xor = (BN == 128) ? static_cast<uint32_t>(row_in_tile & 7) : static_cast<uint32_t>((row_in_tile >> 1) & 3);
    uint32_t g = 0;
    bool ok = true;

    for (uint32_t tile_iter = 0; ok; ++tile_iter) {
      ok = mbar_wait(q_full, tile_iter & 1u, wctx, SITE_ATTN_Q);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int tile = tile_q[tile_iter & 1u];
      mbar_arrive(q_empty);  // this thread has the id; the entry may be reused two tiles on
      if (tile < 0) break;
      const int bh = tile / m_tiles;
      const int mt = row_block_of(tile, bh);
      const int n_steps = steps_of(mt);
      // keys this thread's row may see (all of them without a mask)
      const int visible = causal ? mt * ATT_BM + row_in_tile + causal_off + 1 : Sk;
      float m_i = -INFINITY;
      float l_i = 0.0f;
      for (int j = 0; j < n_steps; ++j, ++g) {
        ok = mbar_wait(s_full, g & 1u, wctx, SITE_ATTN_S_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        constexpr int NC = BN / 32;  // 32-column chunks of the score row
        uint32_t s[NC][32];
#pragma unroll
        for (int c = 0; c < NC; ++c) tmem_ld_32x32b_x32(t_s + c * 32, s[c]);
        tmem_wait_ld();
        tc_fence_before_sync();
        mbar_arrive(s_free);  // S may be overwritten by the next Q K^T

        const int valid = min(Sk, visible) - j * ATT_BN;  // keys of this step that exist and that this row may see
        if (valid < ATT_BN) {
#pragma unroll
          for (int c = 0; c < NC; ++c) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (c * 32 + i >= valid) s[c][i] = __float_as_uint(-INFINITY);
            }
          }
        }
        // row max: 3-input max, four independent chains
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            mx0 = fmax3(mx0, __uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
            mx1 = fmax3(mx1, __uint_as_float(s[c][i + 2]), __uint_as_float(s[c][i + 3]));
            mx2 = fmax3(mx2, __uint_as_float(s[c][i + 4]), __uint_as_float(s[c][i + 5]));
            mx3 = fmax3(mx3, __uint_as_float(s[c][i + 6]), __uint_as_float(s[c][i + 7]));
          }
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        // Exact mode follows the running max (examples/fp8_attention.py:76-78).  Lazy mode keeps the
        // previous reference point m_i while the max has grown by at most 2^8: p is then at most
        // 256 (e4m3 holds 448), O and l stay consistent because both use the same m_i, and the
        // tensor-memory round trip that rescales O leaves the critical path of almost every step.
        const float cand = fmaxf(m_i, mx * scale_log2);
        const bool moved = LAZY ? (cand - m_i > 8.0f) : (cand > m_i);
        const float m_new = (LAZY && !moved) ? m_i : cand;
        const float alpha = fast_exp2(m_i - m_new);

        // p = exp2(s*c - m) on packed pairs; POLY_OF8 of every 8 pairs take the FMA-pipe polynomial
        // instead of the MUFU unit.  Row sum from the fp32 values; e4m3 pack (4 per word).
        const uint64_t c2 = pack2f(scale_log2, scale_log2);
        const uint64_t negm2 = pack2f(-m_new, -m_new);
        uint64_t sum_a = 0ull, sum_b = 0ull;  // two (0.0f, 0.0f) pairs
        uint32_t packed[BN / 4];
#pragma unroll
        for (int c = 0; c < NC; ++c) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const int pair0 = (c * 32 + i) / 2;
            const uint64_t t0 = ffma2(pack2(s[c][i], s[c][i + 1]), c2, negm2);
            const uint64_t t1 = ffma2(pack2(s[c][i + 2], s[c][i + 3]), c2, negm2);
            const uint64_t p0 = (pair0 % 8) < POLY_OF8 ? exp2_pair_poly(t0) : exp2_pair_mufu(t0);
            const uint64_t p1 = ((pair0 + 1) % 8) < POLY_OF8 ? exp2_pair_poly(t1) : exp2_pair_mufu(t1);
            sum_a = fadd2(sum_a, p0);
            sum_b = fadd2(sum_b, p1);
            uint32_t a0, a1, b0, b1;
            unpack2(p0, a0, a1);
            unpack2(p1, b0, b1);
            packed[c * 8 + i / 4] =
                pack_e4m3x4(__uint_as_float(a0), __uint_as_float(a1), __uint_as_float(b0), __uint_as_float(b1));
          }
        }
        {
          uint32_t sl, sh;
          unpack2(fadd2(sum_a, sum_b), sl, sh);
          l_i = l_i * alpha + (__uint_as_float(sl) + __uint_as_float(sh));
        }

        // The previous P V must be complete before P (smem) is overwritten or O is rescaled.
        if (g > 0) {
          ok = mbar_wait(pv_done, (g - 1u) & 1u, wctx, SITE_ATTN_PV_DONE);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
        }
        if (j > 0) {
          if (__any_sync(0xffffffffu, moved)) {
            // two 32-column groups in flight per round trip (one with four CTAs per SM: registers)
            constexpr int GROUP = L::CTAS_PER_SM == 4 ? 1 : 2;
#pragma unroll
            for (int c0 = 0; c0 < D / 32; c0 += GROUP) {
              uint32_t o[GROUP][32];
#pragma unroll
              for (int c = 0; c < GROUP; ++c) tmem_ld_32x32b_x32(t_o + (c0 + c) * 32, o[c]);
              tmem_wait_ld();
#pragma unroll
              for (int c = 0; c < GROUP; ++c) {
#pragma unroll
                for (int i = 0; i < 32; ++i) o[c][i] = __float_as_uint(__uint_as_float(o[c][i]) * alpha);
                tmem_st_32x32b_x32(t_o + (c0 + c) * 32, o[c]);
              }
            }
            tmem_wait_st();
          }
        }
        if constexpr (P_TMEM) {
          // word w of a row = keys 4w .. 4w+3 = column w of the row's lane
          tmem_st_32x32b_x32(tmem_base + ATT_P_COL + lane_sel, packed);
          tmem_wait_st();
        } else {
#pragma unroll
          for (int ch = 0; ch < BN / 16; ++ch) {
            *reinterpret_cast<uint4*>(p_row + ((static_cast<uint32_t>(ch) ^ p_xor) << 4)) =
                make_uint4(packed[ch * 4], packed[ch * 4 + 1], packed[ch * 4 + 2], packed[ch * 4 + 3]);
          }
          fence_proxy_async_smem();
        }
        tc_fence_before_sync();
        mbar_arrive(p_full);
        m_i = m_new;
      }
      if (!ok) break;

      // ---- epilogue of the tile: out = O / l --------------------------------------------------
      ok = mbar_wait(pv_done, (g - 1u) & 1u, wctx, SITE_ATTN_O_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int row = mt * ATT_BM + row_in_tile;
      const int64_t out_off = static_cast<int64_t>(bh) * out_stride_bh + static_cast<int64_t>(row) * out_stride_s;
      // The 8- and 16-bit outputs divide through the correctly rounded reciprocal with one residual
      // correction (div_by_rcp): an IEEE division costs ~30 instructions per element, 64-128 of them per
      // row; the fp32 output keeps the IEEE division.
      const float inv_l = __frcp_rn(l_i);
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
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
            uint32_t w[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              w[i] = pack_bf16x2(div_by_rcp(__uint_as_float(o[2 * i]), l_i, inv_l),
                                 div_by_rcp(__uint_as_float(o[2 * i + 1]), l_i, inv_l));
            }
            uint16_t* dst = reinterpret_cast<uint16_t*>(out) + out_off + c * 32;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              *reinterpret_cast<uint4*>(dst + i * 8) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
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
      // O is read; the next tile's first P V (which overwrites it) is ordered after this thread's
      // next arrival on p_full.
      tc_fence_before_sync();
    }
  }

  // ------------------------------- teardown ------------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    __syncwarp();
    tmem_dealloc(tmem_base, ATT_TMEM_COLS);
  }
}

struct AttnConfig {
  int poly_of8;  // of every 8 pairs of exponentials, how many use an FMA-pipe polynomial
  bool lazy;     // rescale O only when a row max grew by more than 2^8
  int bn;        // keys per step; 64 exists for head_dim 64 only (head_dim 128 then runs 128-key steps)
  bool pair;     // two query tiles per CTA (fp8_attention_pair.cu); problems it does not take run the row's one-tile form
  const char* note;
};
const AttnConfig kAttnConfigs[] = {
    {0, false, 128, false, "exact running max (rescale whenever a row max moves), all exp2 on the MUFU unit"},
    {0, true, 128, false, "lazy rescale (only when a row max grew by more than 2^8), all exp2 on the MUFU unit"},
    {2, true, 128, false, "lazy rescale, 2 of 8 exp2 pairs on the FMA pipes (degree-3 polynomial)"},
    {4, true, 128, false, "lazy rescale, 4 of 8 exp2 pairs on the FMA pipes"},
    {0, false, 64, false, "exact running max, 64-key steps with four CTAs per SM for head_dim 64 (128-key steps otherwise)"},
    {0, true, 64, false, "lazy rescale, 64-key steps with four CTAs per SM for head_dim 64 (128-key steps otherwise)"},
    {0, false, 128, true, "two query tiles per CTA, exact running max, all exp2 on the MUFU unit"},
    {2, false, 128, true, "two query tiles per CTA, exact running max, 2 of 8 exp2 pairs on the FMA pipes (degree-5 polynomial)"},
    {4, false, 128, true, "two query tiles per CTA, exact running max, 4 of 8 exp2 pairs on the FMA pipes (degree-5 polynomial)"},
    {4, true, 128, true, "two query tiles per CTA, lazy rescale, 4 of 8 exp2 pairs on the FMA pipes (degree-5 polynomial)"},
};
constexpr int kNumAttnConfigs = 10;
constexpr int kDefaultAttnConfig = 0;

// The two-tile kernel takes unmasked problems with at least two row blocks per slice and at least two key
// steps; everything else runs the one-tile kernel.
bool attn_pair_applies(const AttnArgs& a) { return !a.causal && a.S > ATT_BM && a.Sk > 128; }

// The row used for cfg_id = -1: always an exact-running-max row.  Measured on B200 (cold L2, exact rows only):
//   B8 H32 S4096 D64:   row 6 (two tiles per CTA) 1501 us, row 0 1536 us, row 4 (64-key steps) 1548 us
//   B4 H48 S1024 D64:   row 0 92 us, rows 4 and 6 98 us
//   B8 H32 S4096 D128:  rows 0 and 6 1718-1720 us;  B4 H48 S1024 D128: row 0 107 us, row 6 115 us
// so the two-tile kernel is taken for head_dim 64 from 2048 keys up where it applies (no mask, at least two row
// blocks), the 64-key-step row for the other head_dim 64 problems of that length, and row 0 everywhere else.
int attn_select_config(const AttnArgs& a) {
  if (a.D == 64 && a.Sk >= 2048) return attn_pair_applies(a) ? 6 : 4;
  return kDefaultAttnConfig;
}

// keys per step that a table row means for a head dimension
int attn_block_n(int cfg_id, int64_t d) {
  const int cfg = cfg_id < 0 ? kDefaultAttnConfig : cfg_id;
  return (kAttnConfigs[cfg].bn == 64 && d == 64) ? 64 : 128;
}

template <int D, int BN, bool V_KMAJOR, int OUT_DT, int POLY_OF8, bool LAZY>
int launch_attn_poly(const AttnArgs& a, DeviceCtx* ctx, const CUtensorMap& tq, const CUtensorMap& tk,
                     const CUtensorMap& tv) {
  using L = AttnLayout<D, BN>;
  auto kernel = fp8_attention_kernel<D, BN, V_KMAJOR, OUT_DT, POLY_OF8, LAZY>;
  static std::atomic<uint64_t> smem_attr_done{0};
  HB_CUDA_CHECK(set_max_dynamic_smem_once(smem_attr_done, reinterpret_cast<const void*>(kernel), L::SMEM_BYTES, a.device));
  const int64_t m_tiles = (a.S + ATT_BM - 1) / ATT_BM;
  const int64_t num_tiles = a.BH * m_tiles;
  if (num_tiles > INT32_MAX) return set_error(HB200_ERR_BAD_SHAPE, "fp8_attention: too many tiles");
  const int grid = static_cast<int>(std::min<int64_t>(num_tiles, L::CTAS_PER_SM * ctx->num_sms));
  kernel<<<grid, ATT_THREADS, L::SMEM_BYTES, a.stream>>>(tq, tk, tv, a.out, static_cast<int>(a.BH),
                                                         static_cast<int>(a.S), static_cast<int>(a.Sk),
                                                         a.causal ? static_cast<int>(a.Sk - a.S) : -1, a.out_strides[0],
                                                         a.out_strides[1],
                                                         a.scale_log2, ctx->status_dev, a.sched);
  HB_CUDA_CHECK(cudaGetLastError());
  return HB200_OK;
}

template <int D, bool V_KMAJOR, int OUT_DT>
int launch_attn_instance(const AttnArgs& a, DeviceCtx* ctx, const CUtensorMap& tq, const CUtensorMap& tk,
                         const CUtensorMap& tv) {
  const int cfg = a.cfg_id < 0 ? kDefaultAttnConfig : a.cfg_id;
  const AttnConfig& c = kAttnConfigs[cfg];
  if constexpr (D == 64) {
    if (c.bn == 64) {
      return c.lazy ? launch_attn_poly<D, 64, V_KMAJOR, OUT_DT, 0, true>(a, ctx, tq, tk, tv)
                    : launch_attn_poly<D, 64, V_KMAJOR, OUT_DT, 0, false>(a, ctx, tq, tk, tv);
    }
  }
  if (!c.lazy) return launch_attn_poly<D, 128, V_KMAJOR, OUT_DT, 0, false>(a, ctx, tq, tk, tv);
  switch (c.poly_of8) {
    case 0:
      return launch_attn_poly<D, 128, V_KMAJOR, OUT_DT, 0, true>(a, ctx, tq, tk, tv);
    case 2:
      return launch_attn_poly<D, 128, V_KMAJOR, OUT_DT, 2, true>(a, ctx, tq, tk, tv);
    case 4:
      return launch_attn_poly<D, 128, V_KMAJOR, OUT_DT, 4, true>(a, ctx, tq, tk, tv);
    default:
      return set_error(HB200_ERR_BAD_CONFIG, "fp8_attention: config has no kernel instance");
  }
}

template <int D, bool V_KMAJOR>
int launch_attn_by_dtype(const AttnArgs& a, DeviceCtx* ctx, const CUtensorMap& tq, const CUtensorMap& tk,
                         const CUtensorMap& tv) {
  switch (a.out_dtype) {
    case HB200_DT_E4M3:
      return launch_attn_instance<D, V_KMAJOR, HB200_DT_E4M3>(a, ctx, tq, tk, tv);
    case HB200_DT_BF16:
      return launch_attn_instance<D, V_KMAJOR, HB200_DT_BF16>(a, ctx, tq, tk, tv);
    case HB200_DT_FP32:
      return launch_attn_instance<D, V_KMAJOR, HB200_DT_FP32>(a, ctx, tq, tk, tv);
    default:
      return set_error(HB200_ERR_BAD_DTYPE, "fp8_attention: unsupported out_dtype");
  }
}

}  // namespace

int attn_num_configs() { return kNumAttnConfigs; }

int attn_describe_config(int cfg_id, char* buf, int buf_len) {
  if (cfg_id < 0 || cfg_id >= kNumAttnConfigs) return set_error(HB200_ERR_BAD_CONFIG, "fp8_attention: no such config");
  return std::snprintf(buf, buf_len, "attention cfg %d: %s", cfg_id, kAttnConfigs[cfg_id].note);
}

int launch_fp8_attention(const AttnArgs& args, DeviceCtx* ctx) {
  if (args.cfg_id >= kNumAttnConfigs) return set_error(HB200_ERR_BAD_CONFIG, "fp8_attention: no such config");
  AttnArgs a = args;
  if (a.cfg_id < 0) a.cfg_id = attn_select_config(a);
  const bool v_kmajor = a.v_strides[2] == 1 && a.v_strides[1] != 1;  // keys contiguous
  const uint32_t d = static_cast<uint32_t>(a.D);
  const CUtensorMapSwizzle swz_d = a.D == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  const uint32_t bn = static_cast<uint32_t>(attn_block_n(a.cfg_id, a.D));
  CUtensorMap tq, tk, tv;
  int rc;
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(a.D), static_cast<uint64_t>(a.S), static_cast<uint64_t>(a.BH)};
    const uint64_t kdims[3] = {static_cast<uint64_t>(a.D), static_cast<uint64_t>(a.Sk), static_cast<uint64_t>(a.BH)};
    const uint32_t box[3] = {d, 128, 1};
    const uint32_t kvbox[3] = {d, bn, 1};
    const uint64_t qs[2] = {static_cast<uint64_t>(a.q_strides[1]), static_cast<uint64_t>(a.q_strides[0])};
    rc = encode_tmap_u8(&tq, a.q, 3, dims, qs, box, swz_d);
    if (rc != HB200_OK) return rc;
    const uint64_t ks[2] = {static_cast<uint64_t>(a.k_strides[1]), static_cast<uint64_t>(a.k_strides[0])};
    rc = encode_tmap_u8(&tk, a.k, 3, kdims, ks, kvbox, swz_d);
    if (rc != HB200_OK) return rc;
    if (!v_kmajor) {
      // physical [BH, S, D]: logical strides {bh, d, s} = {v_strides[0], 1, v_strides[2]}
      const uint64_t vs[2] = {static_cast<uint64_t>(a.v_strides[2]), static_cast<uint64_t>(a.v_strides[0])};
      rc = encode_tmap_u8(&tv, a.v, 3, kdims, vs, kvbox, swz_d);
      if (rc != HB200_OK) return rc;
    } else {
      const uint64_t vdims[3] = {static_cast<uint64_t>(a.Sk), static_cast<uint64_t>(a.D), static_cast<uint64_t>(a.BH)};
      const uint32_t vbox[3] = {bn, d, 1};
      const uint64_t vs[2] = {static_cast<uint64_t>(a.v_strides[1]), static_cast<uint64_t>(a.v_strides[0])};
      rc = encode_tmap_u8(&tv, a.v, 3, vdims, vs, vbox,
                          bn == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
      if (rc != HB200_OK) return rc;
    }
  }
  if (kAttnConfigs[a.cfg_id].pair) {
    if (attn_pair_applies(a)) {
      return launch_fp8_attention_pair(a, ctx, tq, tk, tv, v_kmajor, kAttnConfigs[a.cfg_id].poly_of8, kAttnConfigs[a.cfg_id].lazy);
    }
    a.cfg_id = kAttnConfigs[a.cfg_id].lazy ? 1 : 0;  // the row's one-tile form (same tensor maps: 128-key steps)
  }
  if (a.D == 64) {
    return v_kmajor ? launch_attn_by_dtype<64, true>(a, ctx, tq, tk, tv)
                    : launch_attn_by_dtype<64, false>(a, ctx, tq, tk, tv);
  }
  return v_kmajor ? launch_attn_by_dtype<128, true>(a, ctx, tq, tk, tv)
                  : launch_attn_by_dtype<128, false>(a, ctx, tq, tk, tv);
}

}  // namespace hb
