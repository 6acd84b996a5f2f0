// fp16 / bf16 attention forward (non-causal) for sm_100a with the numerics of pytorch-labs/helion's
// examples/attention.py:29-84 in ref-eager mode:
//   qk  = cast16(q k^T)                       torch.bmm of 16-bit tensors returns 16 bits   (:66)
//   t   = cast16(qk * c)                      16-bit tensor times a Python scalar, c = log2(e)/sqrt(D)   (:67-68)
//   m   = max(m, rowmax(t));  p = exp2(t - m);  l = l*alpha + rowsum(p)       fp32   (:67-72)
//   acc = acc*alpha + cast16(p) v             fp32 accumulation   (:73-76)
//   out = cast16(acc / l)                     (:78-80)
// k and v may hold a different number of rows than q (examples/attention.py:51-58).
//
// The pipeline is the one of the e4m3 kernel (fp8_attention.cu): persistent CTAs, two per SM, a TMA
// producer warp, one MMA thread for S = Q K^T and one for O += P V (kind::f16 instructions), four
// softmax warps with one query row per thread, tiles handed out through the shared-memory tile
// queue.  What differs is the geometry: rows are 2*D bytes long, so a Q / K / V tile is stored as one
// or two column blocks of 128-byte rows (head_dim 64 / 128), keys are walked in steps of 128 (head_dim
// 64) or 64 (head_dim 128), and P, as 16-bit values, never touches shared memory: it is written to the
// tensor-memory columns that S and O leave free (S: BN, O: D, P: BN/2 of the 256 columns) and P V reads
// its A operand from there.
#include <algorithm>
#include <cmath>
#include <cstdio>

#include "common.cuh"
#include "host.h"

namespace hb {

namespace {

constexpr int A16_BM = 128;  // query rows per tile
constexpr int A16_THREADS = 256;
constexpr int A16_SOFTMAX_THREADS = 128;

template <int D>
struct Attn16Layout {
  static constexpr int BN = D == 64 ? 128 : 64;        // keys per step
  static constexpr int ROW_BYTES = D * 2;
  static constexpr int BLOCKS = ROW_BYTES / 128;       // 128-byte column blocks per row
  static constexpr int Q_BYTES = A16_BM * ROW_BYTES;   // BLOCKS x [128 rows x 128 B]
  static constexpr int TILE_BYTES = BN * ROW_BYTES;    // one K or V tile: BLOCKS x [BN rows x 128 B], 16 KB
  static constexpr int KV_STAGES = D == 64 ? 5 : 4;
  // tensor memory: S in [0, BN), O in [BN, BN + D), P (two values per column) in [BN + D, BN + D + BN/2)
  static constexpr int O_COL = BN;
  static constexpr int P_COL = BN + D;
  static constexpr int TMEM_COLS = 256;
  static_assert(P_COL + BN / 2 <= TMEM_COLS, "S, O and P must fit the CTA's tensor memory");
  static constexpr int Q_OFFSET = 0;
  static constexpr int KV_OFFSET = Q_BYTES;
  static constexpr int BAR_OFFSET = KV_OFFSET + KV_STAGES * TILE_BYTES;
  // q_full q_empty s_full s_free p_full pv_done drain drain_pv kv_full[ST] kv_empty[ST]
  static constexpr int NUM_BARS = 8 + 2 * KV_STAGES;
  static constexpr int MISC_OFFSET = BAR_OFFSET + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = MISC_OFFSET + 16 + 1024;
  static_assert(SMEM_BYTES <= 112 * 1024, "two CTAs must fit one SM");
};

// Two fp32 values -> rounded to the 16-bit type -> back to fp32, with one packed conversion.
template <int KIND>
__device__ __forceinline__ void round16_pair(float& a, float& b) {
  if constexpr (KIND == KIND_F16) {
    const float2 f = __half22float2(__floats2half2_rn(a, b));
    a = f.x;
    b = f.y;
  } else {
    const uint32_t w = pack_bf16x2(a, b);  // a in the low half
    a = __uint_as_float(w << 16);
    b = __uint_as_float(w & 0xffff0000u);
  }
}

template <int KIND>
__device__ __forceinline__ uint32_t pack16x2(float lo, float hi) {
  if constexpr (KIND == KIND_F16) return pack_f16x2(lo, hi);
  else return pack_bf16x2(lo, hi);
}

template <int D, int KIND, int OUT_DT>
__global__ void __launch_bounds__(A16_THREADS, 2)
attention16_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, void* out, int BH, int S, int Sk, int64_t out_stride_bh,
                   int64_t out_stride_s, float scale_log2, uint32_t* status, unsigned int* sched) {
  using L = Attn16Layout<D>;
  constexpr int ST = L::KV_STAGES;
  constexpr int NB = L::BLOCKS;
  constexpr int A16_BN = L::BN;

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
  uint64_t* drain_pv = bars + 7;
  uint64_t* kv_full = bars + 8;
  uint64_t* kv_empty = bars + 8 + ST;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::MISC_OFFSET);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::MISC_OFFSET + 4);
  volatile int* tile_q = reinterpret_cast<volatile int*>(smem + L::MISC_OFFSET + 8);  // [2], indexed by tile parity

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = (S + A16_BM - 1) / A16_BM;
  const int n_steps = (Sk + A16_BN - 1) / A16_BN;
  const int num_tiles = BH * m_tiles;
  const WaitCtx wctx{abort_flag, status};

  if (threadIdx.x == 0) {
    // descriptor fetches overlap the barrier set-up and the tensor-memory allocation
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    mbar_init(q_full, 1);
    mbar_init(q_empty, 2 + A16_SOFTMAX_THREADS);  // last Q K^T + every softmax thread and the P V thread hold the tile id
    mbar_init(s_full, 1);
    mbar_init(s_free, A16_SOFTMAX_THREADS);
    mbar_init(p_full, A16_SOFTMAX_THREADS);
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
    tmem_alloc(tmem_slot, L::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // roles by SM slot, as in the e4m3 kernel: the MMA threads of co-resident CTAs sit on different schedulers
  const uint32_t sm_slot = ((tmem_base & 0xffffu) / L::TMEM_COLS) & 1u;
  const int w_producer = sm_slot ? 1 : 0;
  const int w_qk = sm_slot ? 2 : 1;
  const int w_pv = sm_slot ? 0 : 3;

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == w_producer) {
      // ------------------------------- TMA producer ------------------------------------------
      if (lane == 0) {
        uint32_t slot_it = 0;
        uint32_t tile_iter = 0;
        bool ok = true;
        int tile = blockIdx.x;  // gridDim.x <= num_tiles
        for (;; ++tile_iter) {
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
          const int mt = tile - bh * m_tiles;
          mbar_arrive_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            tma_load_3d(smem + L::Q_OFFSET + b * (A16_BM * 128), &tmap_q, q_full, b * 128, mt * A16_BM, bh);
          }
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
              // K and V tiles have the same geometry: 64 rows (keys) of 2*D bytes, in 128-byte column blocks
#pragma unroll
              for (int b = 0; b < NB; ++b) {
                tma_load_3d(dst + b * (A16_BN * 128), kv == 0 ? &tmap_k : &tmap_v, &kv_full[s], b * 128, j * A16_BN, bh);
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
        constexpr uint32_t idesc_qk = make_idesc<KIND>(A16_BM, A16_BN, false, false);
        const uint32_t q_addr = smem_u32(smem + L::Q_OFFSET);
        const uint32_t kv_addr = smem_u32(smem + L::KV_OFFSET);
        const uint32_t t_s = tmem_base;
        uint32_t g = 0;
        uint32_t slot_it = 0;
        uint32_t tile_iter = 0;
        bool ok = true;
        for (; ok; ++tile_iter) {
          if (!mbar_wait_relaxed(q_full, tile_iter & 1u, wctx, SITE_ATTN_Q, 100)) {
            ok = false;
            break;
          }
          if (tile_q[tile_iter & 1u] < 0) break;
          for (int j = 0; j < n_steps; ++j, ++g, slot_it += 2) {
            const uint32_t s = slot_it % ST;
            if (!mbar_wait_relaxed(&kv_full[s], (slot_it / ST) & 1u, wctx, SITE_ATTN_K_FULL, 100) ||
                (g > 0 && !mbar_wait_relaxed(s_free, (g - 1u) & 1u, wctx, SITE_ATTN_S_FREE, 100))) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
            const uint32_t k_addr = kv_addr + s * L::TILE_BYTES;
            // contraction over head_dim: 32 bytes (16 elements) per instruction, 4 per 128-byte column block
#pragma unroll
            for (int k = 0; k < L::ROW_BYTES / 32; ++k) {
              const int blk = k / 4;
              const uint64_t q_desc = make_smem_desc(q_addr + blk * (A16_BM * 128), 16, 1024, SWZ_128B);
              const uint64_t k_desc = make_smem_desc(k_addr + blk * (A16_BN * 128), 16, 1024, SWZ_128B);
              umma_f16_ss(t_s, desc_advance(q_desc, (k % 4) * 32), desc_advance(k_desc, (k % 4) * 32), idesc_qk,
                          k != 0 ? 1u : 0u);
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
      if (lane == 0) {
        constexpr uint32_t idesc_pv = make_idesc<KIND>(A16_BM, D, false, true);
        const uint32_t kv_addr = smem_u32(smem + L::KV_OFFSET);
        const uint32_t t_o = tmem_base + L::O_COL;
        const uint32_t t_p = tmem_base + L::P_COL;
        uint32_t g = 0;
        uint32_t slot_it = 0;
        uint32_t tile_iter = 0;
        bool ok = true;
        for (; ok; ++tile_iter) {
          if (!mbar_wait_relaxed(q_full, tile_iter & 1u, wctx, SITE_ATTN_Q, 100)) {
            ok = false;
            break;
          }
          const int tile = tile_q[tile_iter & 1u];
          mbar_arrive(q_empty);
          if (tile < 0) break;
          for (int j = 0; j < n_steps; ++j, ++g, slot_it += 2) {
            const uint32_t vs = (slot_it + 1) % ST;
            if (!mbar_wait_relaxed(&kv_full[vs], ((slot_it + 1) / ST) & 1u, wctx, SITE_ATTN_V_FULL, 100) ||
                !mbar_wait_relaxed(p_full, g & 1u, wctx, SITE_ATTN_P_FULL, 100)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
            // V [BN keys, D] with D contiguous: MN-major B; column blocks of 64 elements (128 B) lie
            // BN x 128 bytes apart, 8 key rows per atom (1024 B), 16 keys (2048 B) per instruction.
            // A = P from tensor memory: 16 keys = 8 columns per instruction.
            const uint64_t v_desc = make_smem_desc(kv_addr + vs * L::TILE_BYTES, A16_BN * 128, 1024, SWZ_128B);
#pragma unroll
            for (int k = 0; k < A16_BN / 16; ++k) {
              umma_f16_ts(t_o, t_p + k * 8, desc_advance(v_desc, k * 16 * 128), idesc_pv, (j | k) != 0 ? 1u : 0u);
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
    asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t t_s = tmem_base + lane_sel;
    const uint32_t t_o = tmem_base + L::O_COL + lane_sel;
    const uint32_t t_p = tmem_base + L::P_COL + lane_sel;
    constexpr int NC = A16_BN / 32;  // 32-column chunks of the score row
    uint32_t g = 0;
    bool ok = true;

    for (uint32_t tile_iter = 0; ok; ++tile_iter) {
      ok = mbar_wait(q_full, tile_iter & 1u, wctx, SITE_ATTN_Q);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int tile = tile_q[tile_iter & 1u];
      mbar_arrive(q_empty);
      if (tile < 0) break;
      const int bh = tile / m_tiles;
      const int mt = tile - bh * m_tiles;
      float m_i = -INFINITY;
      float l_i = 0.0f;
      for (int j = 0; j < n_steps; ++j, ++g) {
        ok = mbar_wait(s_full, g & 1u, wctx, SITE_ATTN_S_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        uint32_t s[NC][32];
#pragma unroll
        for (int c = 0; c < NC; ++c) tmem_ld_32x32b_x32(t_s + c * 32, s[c]);
        tmem_wait_ld();
        tc_fence_before_sync();
        mbar_arrive(s_free);

        // keys beyond seq_k count as -inf (ragged last step only; -inf survives the roundings and the scale)
        const int valid = Sk - j * A16_BN;
        if (valid < A16_BN) {
#pragma unroll
          for (int c = 0; c < NC; ++c) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (c * 32 + i >= valid) s[c][i] = __float_as_uint(-INFINITY);
            }
          }
        }
        // t = cast16(cast16(qk) * c): the two 16-bit roundings of the reference's tensors, on packed pairs
        const uint64_t c2 = pack2f(scale_log2, scale_log2);
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;  // independent chains
#pragma unroll
        for (int c = 0; c < NC; ++c) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              float t0 = __uint_as_float(s[c][i + 2 * h]), t1 = __uint_as_float(s[c][i + 2 * h + 1]);
              round16_pair<KIND>(t0, t1);
              uint32_t u0, u1;
              unpack2(fmul2(pack2f(t0, t1), c2), u0, u1);
              t0 = __uint_as_float(u0);
              t1 = __uint_as_float(u1);
              round16_pair<KIND>(t0, t1);
              s[c][i + 2 * h] = __float_as_uint(t0);
              s[c][i + 2 * h + 1] = __float_as_uint(t1);
              if (h == 0) mx0 = fmax3(mx0, t0, t1);
              if (h == 1) mx1 = fmax3(mx1, t0, t1);
              if (h == 2) mx2 = fmax3(mx2, t0, t1);
              if (h == 3) mx3 = fmax3(mx3, t0, t1);
            }
          }
        }
        const float m_new = fmaxf(m_i, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)));
        const bool moved = m_new > m_i;
        const float alpha = fast_exp2(m_i - m_new);
        // p = exp2(t - m) on packed pairs; the even and the odd keys are summed separately, as before
        const uint64_t negm2 = pack2f(-m_new, -m_new);
        uint64_t sum2 = 0ull;  // (0.0f, 0.0f)
        uint32_t packed[NC][16];
#pragma unroll
        for (int c = 0; c < NC; ++c) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const uint64_t p2 = exp2_pair_mufu(fadd2(pack2(s[c][i], s[c][i + 1]), negm2));
            sum2 = fadd2(sum2, p2);
            uint32_t p0, p1;
            unpack2(p2, p0, p1);
            packed[c][i / 2] = pack16x2<KIND>(__uint_as_float(p0), __uint_as_float(p1));
          }
        }
        float sum0, sum1;
        {
          uint32_t u0, u1;
          unpack2(sum2, u0, u1);
          sum0 = __uint_as_float(u0);
          sum1 = __uint_as_float(u1);
        }
        l_i = l_i * alpha + (sum0 + sum1);

        if (g > 0) {
          ok = mbar_wait(pv_done, (g - 1u) & 1u, wctx, SITE_ATTN_PV_DONE);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
        }
        if (j > 0 && __any_sync(0xffffffffu, moved)) {
#pragma unroll
          for (int c0 = 0; c0 < D / 32; c0 += 2) {  // two 32-column groups per round trip
            uint32_t o[2][32];
#pragma unroll
            for (int c = 0; c < 2; ++c) tmem_ld_32x32b_x32(t_o + (c0 + c) * 32, o[c]);
            tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < 2; ++c) {
#pragma unroll
              for (int i = 0; i < 32; ++i) o[c][i] = __float_as_uint(__uint_as_float(o[c][i]) * alpha);
              tmem_st_32x32b_x32(t_o + (c0 + c) * 32, o[c]);
            }
          }
        }
        // P: column w of this row's lane = keys 2w (low half) and 2w + 1
#pragma unroll
        for (int c = 0; c < NC; ++c) tmem_st_32x32b_x16(t_p + c * 16, packed[c]);
        tmem_wait_st();
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
      const int row = mt * A16_BM + row_in_tile;
      const int64_t out_off = static_cast<int64_t>(bh) * out_stride_bh + static_cast<int64_t>(row) * out_stride_s;
      const float inv_l = __frcp_rn(l_i);
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(t_o + c * 32, o);
        tmem_wait_ld();
        if (row < S) {
          if constexpr (OUT_DT == HB200_DT_FP32) {
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
          } else {
            uint32_t w[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              // through the rounded reciprocal with one residual correction instead of an IEEE division
              const float lo = div_by_rcp(__uint_as_float(o[2 * i]), l_i, inv_l);
              const float hi = div_by_rcp(__uint_as_float(o[2 * i + 1]), l_i, inv_l);
              w[i] = OUT_DT == HB200_DT_FP16 ? pack_f16x2(lo, hi) : pack_bf16x2(lo, hi);
            }
            uint16_t* dst = reinterpret_cast<uint16_t*>(out) + out_off + c * 32;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              *reinterpret_cast<uint4*>(dst + i * 8) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
            }
          }
        }
      }
      tc_fence_before_sync();
    }
  }

  // ------------------------------- teardown ------------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    __syncwarp();
    tmem_dealloc(tmem_base, L::TMEM_COLS);
  }
}

template <int D, int KIND, int OUT_DT>
int launch_attn16(const AttnArgs& a, DeviceCtx* ctx, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv) {
  using L = Attn16Layout<D>;
  auto kernel = attention16_kernel<D, KIND, OUT_DT>;
  static std::atomic<uint64_t> smem_attr_done{0};
  HB_CUDA_CHECK(set_max_dynamic_smem_once(smem_attr_done, reinterpret_cast<const void*>(kernel), L::SMEM_BYTES, a.device));
  const int64_t m_tiles = (a.S + A16_BM - 1) / A16_BM;
  const int64_t num_tiles = a.BH * m_tiles;
  if (num_tiles > INT32_MAX) return set_error(HB200_ERR_BAD_SHAPE, "attention_16bit: too many tiles");
  const int grid = static_cast<int>(std::min<int64_t>(num_tiles, 2 * ctx->num_sms));
  kernel<<<grid, A16_THREADS, L::SMEM_BYTES, a.stream>>>(tq, tk, tv, a.out, static_cast<int>(a.BH), static_cast<int>(a.S),
                                                         static_cast<int>(a.Sk), a.out_strides[0], a.out_strides[1],
                                                         a.scale_log2, ctx->status_dev, a.sched);
  HB_CUDA_CHECK(cudaGetLastError());
  return HB200_OK;
}

template <int D, int KIND>
int launch_attn16_out(const AttnArgs& a, DeviceCtx* ctx, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv) {
  constexpr int SAME = KIND == KIND_F16 ? HB200_DT_FP16 : HB200_DT_BF16;
  if (a.out_dtype == SAME) return launch_attn16<D, KIND, SAME>(a, ctx, tq, tk, tv);
  if (a.out_dtype == HB200_DT_FP32) return launch_attn16<D, KIND, HB200_DT_FP32>(a, ctx, tq, tk, tv);
  return set_error(HB200_ERR_BAD_DTYPE, "attention_16bit: out_dtype must be the operands' dtype or FP32");
}

}  // namespace

// q [BH, S, D], k and v [BH, Sk, D] (head_dim contiguous) in fp16 / bf16 (args.kind); strides in elements.
int launch_attention_16bit(const AttnArgs& a, DeviceCtx* ctx) {
  CUtensorMap tq, tk, tv;
  // maps over bytes: 128-byte column blocks of rows that are 2*D bytes long
  const uint32_t qbox[3] = {128, A16_BM, 1};
  const uint32_t kvbox[3] = {128, static_cast<uint32_t>(a.D == 64 ? Attn16Layout<64>::BN : Attn16Layout<128>::BN), 1};
  const uint64_t qdims[3] = {static_cast<uint64_t>(a.D * 2), static_cast<uint64_t>(a.S), static_cast<uint64_t>(a.BH)};
  const uint64_t kdims[3] = {static_cast<uint64_t>(a.D * 2), static_cast<uint64_t>(a.Sk), static_cast<uint64_t>(a.BH)};
  const uint64_t qs[2] = {static_cast<uint64_t>(a.q_strides[1] * 2), static_cast<uint64_t>(a.q_strides[0] * 2)};
  const uint64_t ks[2] = {static_cast<uint64_t>(a.k_strides[1] * 2), static_cast<uint64_t>(a.k_strides[0] * 2)};
  const uint64_t vs[2] = {static_cast<uint64_t>(a.v_strides[1] * 2), static_cast<uint64_t>(a.v_strides[0] * 2)};
  int rc = encode_tmap_u8(&tq, a.q, 3, qdims, qs, qbox, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != HB200_OK) return rc;
  rc = encode_tmap_u8(&tk, a.k, 3, kdims, ks, kvbox, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != HB200_OK) return rc;
  rc = encode_tmap_u8(&tv, a.v, 3, kdims, vs, kvbox, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != HB200_OK) return rc;
  if (a.kind == KIND_F16) {
    return a.D == 64 ? launch_attn16_out<64, KIND_F16>(a, ctx, tq, tk, tv) : launch_attn16_out<128, KIND_F16>(a, ctx, tq, tk, tv);
  }
  return a.D == 64 ? launch_attn16_out<64, KIND_BF16>(a, ctx, tq, tk, tv) : launch_attn16_out<128, KIND_BF16>(a, ctx, tq, tk, tv);
}

}  // namespace hb
