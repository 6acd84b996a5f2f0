// Device-side building blocks shared by the sm_100a kernels: mbarrier, TMA, tcgen05 (UMMA +
// tensor memory) wrappers written as inline PTX, the shared-memory / instruction descriptor
// encoders, and the bounded-wait scheme.
//
// Every wait in these kernels is bounded: a wait that does not complete within
// HB_WAIT_LIMIT_NS raises a CTA-wide abort flag and records where it gave up in a status word
// that the host can read; all roles then leave their loops, in-flight copies and MMAs are
// drained (again with a limit), tensor memory is released and the kernel returns.  Nothing here
// traps, asserts or spins without a limit.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hb {

// ------------------------------------------------------------------------------------------
// status word layout (one 32-bit word per device, in mapped pinned host memory):
//   0                      : no device-side problem recorded
//   (site << 16) | blockIdx: first wait that ran out, `site` identifies the wait in the source
// ------------------------------------------------------------------------------------------
constexpr unsigned long long HB_WAIT_LIMIT_NS = 2000000000ull;  // 2 s per wait
constexpr unsigned long long HB_DRAIN_LIMIT_NS = 200000000ull;  // 0.2 s per drain wait

// Operand kinds of the GEMM kernels: e4m3 (kind::f8f6f4) or 16-bit floats (kind::f16).  All of them
// move 32 bytes of K per instruction, so the byte-oriented pipelines are shared.
enum OperandKind : int { KIND_E4M3 = 0, KIND_F16 = 1, KIND_BF16 = 2 };

enum WaitSite : uint32_t {
  SITE_GEMM_EMPTY = 1,
  SITE_GEMM_FULL = 2,
  SITE_GEMM_ACC_EMPTY = 3,
  SITE_GEMM_ACC_FULL = 4,
  SITE_ATTN_Q = 10,
  SITE_ATTN_KV_EMPTY = 11,
  SITE_ATTN_K_FULL = 12,
  SITE_ATTN_V_FULL = 13,
  SITE_ATTN_S_FULL = 14,
  SITE_ATTN_S_FREE = 15,
  SITE_ATTN_P_FULL = 16,
  SITE_ATTN_PV_DONE = 17,
  SITE_ATTN_O_FULL = 18,
  SITE_ATTN_ALPHA = 19,
  SITE_ATTN_O_READY = 20,
  SITE_SELFTEST = 40,
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ------------------------------------------------------------------------------------------
// mbarrier
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Make generic-proxy writes to shared memory visible to the async proxy (TMA, UMMA operands).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Shared state of the bounded-wait scheme, one per CTA.
struct WaitCtx {
  volatile uint32_t* abort_flag;  // shared memory, set by the first wait that runs out
  uint32_t* status;               // mapped host word (may be null)
};

__device__ __forceinline__ void record_timeout(const WaitCtx& ctx, uint32_t site) {
  *ctx.abort_flag = 1u;
  if (ctx.status != nullptr) {
    // Plain accesses on purpose: the word lives in mapped host memory, and "first writer wins"
    // does not need to be exact.
    volatile uint32_t* w = ctx.status;
    if (*w == 0u) *w = (site << 16) | (blockIdx.x & 0xffffu);
  }
}

// Wait for the phase with the given parity to complete.  Returns false when the CTA is
// aborting (this wait or another one ran out); the caller must then leave its loop.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& ctx, uint32_t site) {
  if (mbar_try_wait(bar, parity)) return true;
  // The global timer is slow to read, so the clock of the limit only starts at the first check
  // (256 failed polls in); a wait that is satisfied quickly never touches it.
  unsigned long long t0 = 0ull;
  uint32_t spins = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (((++spins) & 0xffu) == 0u) {
      if (*ctx.abort_flag) return false;
      const unsigned long long now = global_timer_ns();
      if (t0 == 0ull) {
        t0 = now;
      } else if (now - t0 > HB_WAIT_LIMIT_NS) {
        record_timeout(ctx, site);
        return false;
      }
    }
  }
}

// mbar_wait with an explicit limit (used by the wait self-test, which waits on a barrier that
// nothing will ever complete in order to exercise the give-up path).
__device__ __forceinline__ bool mbar_wait_limited(uint64_t* bar, uint32_t parity, const WaitCtx& ctx, uint32_t site,
                                                  unsigned long long limit_ns) {
  const unsigned long long t0 = global_timer_ns();
  uint32_t spins = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (((++spins) & 0xffu) == 0u) {
      if (*ctx.abort_flag) return false;
      if (global_timer_ns() - t0 > limit_ns) {
        record_timeout(ctx, site);
        return false;
      }
    }
  }
}

// Same contract as mbar_wait for waits that are not latency-critical (a producer waiting for a free
// slot, an MMA issuer waiting for operands that are needed much later): sleeps between polls so that
// the polling thread does not take issue slots from the warps that share its scheduler.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, const WaitCtx& ctx, uint32_t site,
                                                  uint32_t sleep_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = 0ull;  // set at the first check, see mbar_wait
  uint32_t spins = 0;
  for (;;) {
    __nanosleep(sleep_ns);
    if (mbar_try_wait(bar, parity)) return true;
    if (((++spins) & 0x3fu) == 0u) {
      if (*ctx.abort_flag) return false;
      const unsigned long long now = global_timer_ns();
      if (t0 == 0ull) {
        t0 = now;
      } else if (now - t0 > HB_WAIT_LIMIT_NS) {
        record_timeout(ctx, site);
        return false;
      }
    }
  }
}

// Used only on the abort path: wait, with a short limit and no further bookkeeping.
__device__ __forceinline__ void mbar_drain(uint64_t* bar, uint32_t parity) {
  const unsigned long long t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (((++spins) & 0xffu) == 0u && global_timer_ns() - t0 > HB_DRAIN_LIMIT_NS) return;
  }
}

// ------------------------------------------------------------------------------------------
// TMA (tiled bulk tensor copies, global -> shared, completion on an mbarrier).  Only the plain
// single-CTA form is used anywhere in this library.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y,
                                            int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ------------------------------------------------------------------------------------------
// tensor memory + UMMA
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem], e4m3/e5m2 operands, issued by one thread.
__device__ __forceinline__ void umma_f8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]: A (M = 128 rows on the 128 lanes, K-major, four e4m3 per 32-bit
// column, 8 columns per instruction) is read from tensor memory.
__device__ __forceinline__ void umma_f8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem] for 16-bit operands: two elements per 32-bit column of A, 8 columns
// (K = 16) per instruction.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Same for 16-bit operands (f16 or bf16 per the instruction descriptor), K = 16 elements.
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int KIND>
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  if constexpr (KIND == KIND_E4M3) umma_f8_ss(d_tmem, a_desc, b_desc, idesc, accumulate);
  else umma_f16_ss(d_tmem, a_desc, b_desc, idesc, accumulate);
}

// Programmatic dependent launch.  A kernel launched with launch_pdl() (host.h) may be scheduled while the
// kernel before it in the stream is still running: everything up to pdl_wait() -- barrier set-up,
// tensor-memory allocation, descriptor prefetch -- then overlaps that kernel's tail.  pdl_wait() returns
// once the previous kernel has completed and its writes are visible, so no global memory is touched
// before it.  pdl_launch_dependents() lets the NEXT kernel's CTAs be scheduled as soon as every CTA of
// this grid has called it (they take an SM's resources as this grid's CTAs leave and park in their own
// pdl_wait()).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Arrive on an mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Each thread of the warp reads 32 consecutive 32-bit columns of its own lane.
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ void tmem_st_32x32b_x8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// ------------------------------------------------------------------------------------------
// CTA pairs (cluster of two CTAs on one TPC driving one 256-row UMMA, "cta_group::2").
// The even CTA of the pair is the leader: it issues the MMAs, which read the A rows and one half
// of the B columns from each CTA's shared memory and write each CTA's own 128 accumulator lanes.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// shared::cluster address of `smem_addr` (a shared::cta address) in the CTA with the given rank
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}

// arrive on an mbarrier given by its shared::cluster address (own or peer CTA)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// TMA load into this CTA's shared memory whose completion bytes are counted on an mbarrier that
// may live in the peer CTA (given by its shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// D[tmem of both CTAs] (+)= A[smem of both CTAs] * B[smem halves of both CTAs], M = 256.
__device__ __forceinline__ void umma_f8_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int KIND>
__device__ __forceinline__ void umma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  if constexpr (KIND == KIND_E4M3) umma_f8_ss_pair(d_tmem, a_desc, b_desc, idesc, accumulate);
  else umma_f16_ss_pair(d_tmem, a_desc, b_desc, idesc, accumulate);
}

// Arrive (once) on the mbarrier at a shared::cluster address when all MMAs issued so far by this
// thread have completed.  Used twice in a row to signal the same event to both CTAs of a pair.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}

// ------------------------------------------------------------------------------------------
// descriptors
// ------------------------------------------------------------------------------------------
enum SwizzleMode : uint32_t { SWZ_NONE = 0, SWZ_128B = 2, SWZ_64B = 4, SWZ_32B = 6 };

// 64-bit shared-memory matrix descriptor of tcgen05.mma.
//   bits [ 0,14) start address >> 4         bits [16,30) leading-dimension byte offset >> 4
//   bits [32,46) stride-dimension byte offset >> 4      bits [46,48) descriptor version (1)
//   bits [49,52) base offset (0: tiles are aligned to their swizzle period)
//   bits [61,64) swizzle mode
// K-major operand with a swizzle: rows are `swizzle` bytes long, eight rows form one atom,
//   SBO = distance between 8-row groups, LBO is not used (encoded as 1).
// MN-major operand with a swizzle: `swizzle` bytes are contiguous along M/N, eight K rows form
//   one atom, SBO = distance between 8-row K groups, LBO = distance between consecutive
//   `swizzle`-byte blocks along M/N.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t swizzle) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(swizzle & 7u) << 61;
  return d;
}

// Advance the start address of a descriptor by a byte offset (offset must be a multiple of 16
// and must not carry out of the 14-bit field).
__device__ __forceinline__ uint64_t desc_advance(uint64_t desc, uint32_t bytes) { return desc + (bytes >> 4); }

// 32-bit instruction descriptor for kind::f8f6f4 with e4m3 operands and an fp32 accumulator.
//   bits [4,6) accumulator format (1 = f32)   bits [7,10) A format (0 = e4m3)   bits [10,13) B format
//   bit 15 A major (0 = K, 1 = MN)   bit 16 B major   bits [17,23) N >> 3   bits [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc_e4m3(uint32_t m, uint32_t n, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | (0u << 7) | (0u << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Instruction descriptor for any of the kinds above (fp32 accumulator).  kind::f16 encodes f16 as
// format 0 and bf16 as format 1 in the same A / B format fields.
template <int KIND>
__host__ __device__ constexpr uint32_t make_idesc(uint32_t m, uint32_t n, bool a_mn_major, bool b_mn_major) {
  constexpr uint32_t fmt = KIND == KIND_BF16 ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ------------------------------------------------------------------------------------------
// small numeric helpers
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// a / b from the correctly rounded reciprocal r = 1/b in three instructions: one residual correction of
// the product a*r.  The result is within a small fraction of an ulp of the rounded quotient (it equals
// it except in rare double-rounding cases), at a tenth of the instructions of an IEEE division.
__device__ __forceinline__ float div_by_rcp(float a, float b, float r) {
  const float q = a * r;
  const float e = fmaf(-q, b, a);
  return fmaf(e, r, q);
}

// Two floats -> two e4m3 bytes (lo in bits 0-7), round-to-nearest-even, saturating to +-448.
__device__ __forceinline__ uint16_t pack_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(r) : "f"(lo), "f"(hi));
  return r;
}

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  return static_cast<uint32_t>(pack_e4m3x2(a, b)) | (static_cast<uint32_t>(pack_e4m3x2(c, d)) << 16);
}

// ---- packed fp32 pairs (one 64-bit register = two floats; sm_100 issues these as one instruction)
__device__ __forceinline__ uint64_t pack2(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ uint64_t pack2f(float lo, float hi) { return pack2(__float_as_uint(lo), __float_as_uint(hi)); }
__device__ __forceinline__ void unpack2(uint64_t v, uint32_t& lo, uint32_t& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t fmul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^x for a pair of x <= 0 through the MUFU unit.
__device__ __forceinline__ uint64_t exp2_pair_mufu(uint64_t x2) {
  uint32_t lo, hi;
  unpack2(x2, lo, hi);
  return pack2f(fast_exp2(__uint_as_float(lo)), fast_exp2(__uint_as_float(hi)));
}

// 2^x for a pair of x <= 0 on the FMA / ALU pipes only (no MUFU): round-to-nearest split
// x = n + f with |f| <= 0.5 by the 1.5*2^23 trick, degree-3 minimax polynomial for 2^f
// (relative error 7.5e-5), then n is added into the exponent field.  x is clamped at -126 so that
// the exponent arithmetic cannot wrap (2^-126 rounds to zero in every use here).
__device__ __forceinline__ uint64_t exp2_pair_poly(uint64_t x2) {
  uint32_t xl, xh;
  unpack2(x2, xl, xh);
  const float xcl = fmaxf(__uint_as_float(xl), -126.0f);
  const float xch = fmaxf(__uint_as_float(xh), -126.0f);
  const uint64_t x = pack2f(xcl, xch);
  const uint64_t magic = pack2f(12582912.0f, 12582912.0f);
  const uint64_t neg_magic = pack2f(-12582912.0f, -12582912.0f);
  const uint64_t neg_one = pack2f(-1.0f, -1.0f);
  const uint64_t xr = fadd2(x, magic);        // low mantissa bits now hold round(x)
  const uint64_t nf = fadd2(xr, neg_magic);   // round(x) as a float
  const uint64_t f = ffma2(nf, neg_one, x);   // x - round(x), in [-0.5, 0.5]
  uint64_t p = ffma2(pack2f(0.055171605f, 0.055171605f), f, pack2f(0.24261111f, 0.24261111f));
  p = ffma2(p, f, pack2f(0.69326097f, 0.69326097f));
  p = ffma2(p, f, pack2f(0.99992806f, 0.99992806f));
  uint32_t pl, ph, rl, rh;
  unpack2(p, pl, ph);
  unpack2(xr, rl, rh);
  pl += rl << 23;  // exponent += round(x); the bits above the exponent wrap away
  ph += rh << 23;
  return pack2(pl, ph);
}

// Same split as exp2_pair_poly with a degree-5 polynomial (relative error 2.4e-7, the size of
// ex2.approx's own error): a value computed this way rounds to the same e4m3 code as the MUFU result
// except where either lies within that distance of a rounding boundary, so rows of the attention table
// that follow the reference's running max bit for bit may use it for part of their exponentials.
__device__ __forceinline__ uint64_t exp2_pair_poly5(uint64_t x2) {
  uint32_t xl, xh;
  unpack2(x2, xl, xh);
  const float xcl = fmaxf(__uint_as_float(xl), -126.0f);
  const float xch = fmaxf(__uint_as_float(xh), -126.0f);
  const uint64_t x = pack2f(xcl, xch);
  const uint64_t magic = pack2f(12582912.0f, 12582912.0f);
  const uint64_t neg_magic = pack2f(-12582912.0f, -12582912.0f);
  const uint64_t neg_one = pack2f(-1.0f, -1.0f);
  const uint64_t xr = fadd2(x, magic);       // low mantissa bits now hold round(x)
  const uint64_t nf = fadd2(xr, neg_magic);  // round(x) as a float
  const uint64_t f = ffma2(nf, neg_one, x);  // x - round(x), in [-0.5, 0.5]
  uint64_t p = ffma2(pack2f(0.001327647129073739f, 0.001327647129073739f), f,
                     pack2f(0.009675540961325169f, 0.009675540961325169f));
  p = ffma2(p, f, pack2f(0.05550713092088699f, 0.05550713092088699f));
  p = ffma2(p, f, pack2f(0.24022120237350464f, 0.24022120237350464f));
  p = ffma2(p, f, pack2f(0.6931469440460205f, 0.6931469440460205f));
  p = ffma2(p, f, pack2f(1.0000001192092896f, 1.0000001192092896f));
  uint32_t pl, ph, rl, rh;
  unpack2(p, pl, ph);
  unpack2(xr, rl, rh);
  pl += rl << 23;  // exponent += round(x); the bits above the exponent wrap away
  ph += rh << 23;
  return pack2(pl, ph);
}

}  // namespace hb
