// Host-side plumbing shared by the launchers: per-device context, error text, tensor-map
// encoding.  Nothing here is visible outside the shared library.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <string>

#include "../../include/helion_b200.h"

namespace hb {

struct DeviceCtx {
  bool initialised = false;
  int init_error = 0;         // HB200_ERR_* if initialisation failed
  int num_sms = 0;
  int cc_major = 0;
  int cc_minor = 0;
  uint32_t* status_host = nullptr;  // mapped pinned word written by kernels whose waits ran out
  uint32_t* status_dev = nullptr;   // device-side alias of status_host
};

// Lazily initialised, mutex-protected; returns nullptr (and sets the error text) on failure.
DeviceCtx* get_device_ctx(int device);

// Error code to return when get_device_ctx() gave nullptr.
int device_init_error(int device);

int set_error(int code, const std::string& text);
const char* last_error_text();

#define HB_CUDA_CHECK(expr)                                                                         \
  do {                                                                                              \
    cudaError_t _e = (expr);                                                                        \
    if (_e != cudaSuccess) {                                                                        \
      return ::hb::set_error(HB200_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(_e)); \
    }                                                                                               \
  } while (0)

// Raises a kernel's dynamic shared-memory limit once per device.  `done` is a bit mask of devices (one static
// per kernel instance at the call site); concurrent first calls may both set the attribute, which is harmless.
inline cudaError_t set_max_dynamic_smem_once(std::atomic<uint64_t>& done, const void* kernel, int bytes, int device) {
  const uint64_t bit = 1ull << (static_cast<unsigned>(device) & 63u);
  if (done.load(std::memory_order_acquire) & bit) return cudaSuccess;
  const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) done.fetch_or(bit, std::memory_order_release);
  return e;
}

// Switches the current device for the duration of a launch and restores it afterwards.  ok() is false when
// the device could not be made current; the caller must then return an error instead of launching on
// whatever device happens to be current.
struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  bool good = false;
  explicit DeviceGuard(int device) {
    if (cudaGetDevice(&prev) != cudaSuccess) return;
    if (prev == device) {
      good = true;
      return;
    }
    switched = cudaSetDevice(device) == cudaSuccess;
    good = switched;
  }
  bool ok() const { return good; }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(prev);
  }
};
#define HB_DEVICE_GUARD(device)   \
  ::hb::DeviceGuard guard(device); \
  if (!guard.ok()) return ::hb::set_error(HB200_ERR_CUDA, "cannot make device " + std::to_string(device) + " current")

// The device-side alias of a device's status word if its context already exists, else nullptr.  Never creates
// the context (so it allocates nothing); used by the entry point that must not allocate.
uint32_t* peek_status_dev(int device);

// Encode a tiled tensor map over bytes.  dims/strides innermost first; strides[i] is the byte
// stride of dimension i+1 (dimension 0 is contiguous).  Returns HB200_OK or an error code.
int encode_tmap_u8(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides,
                   const uint32_t* box, CUtensorMapSwizzle swizzle);

// Same for 2- and 4-byte elements (used by the TMA-store epilogues).
int encode_tmap(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, int rank, const uint64_t* dims,
                const uint64_t* strides, const uint32_t* box, CUtensorMapSwizzle swizzle);

// ---- launchers (one per .cu file) -----------------------------------------------------------
struct GemmArgs {
  const void* x;
  const void* y;
  void* out;
  int64_t M, N, K;
  int64_t lda;       // x row stride (elements)
  int64_t ldb;       // y leading stride: column stride if column-major, row stride if row-major
  bool y_colmajor;
  int64_t ldc;       // out row stride (elements)
  int out_dtype;
  int cfg_id;
  void* workspace;
  size_t workspace_bytes;
  int device;
  cudaStream_t stream;
  // optional output scales (hb200_fp8_gemm_scaled): HB200_SCALE_NONE / _TENSOR / _ROWWISE
  const float* scale_a = nullptr;
  const float* scale_b = nullptr;
  int scale_mode = 0;
  // 16-bit operands (hb200_gemm_16bit): 0 = e4m3, 1 = fp16, 2 = bf16; optional bias / ReLU epilogue
  int kind = 0;
  const float* bias = nullptr;
  int relu = 0;
};

int launch_fp8_gemm(const GemmArgs& args, DeviceCtx* ctx);
// Same kernels with fp16 / bf16 operands (args.kind); M, N, K and strides in elements.
int launch_gemm_16bit(const GemmArgs& args, DeviceCtx* ctx);
int gemm_num_configs();
int gemm_describe_config(int cfg_id, char* buf, int buf_len);
int gemm_select_config(int64_t M, int64_t N, int64_t K, bool y_colmajor, int out_dtype, int num_sms);
size_t gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int out_dtype, int cfg_id);

// The operand-swapped kernel for M <= 64 and column-major y (fp8_gemm_skinny.cu); splits > 1 writes
// fp32 partial sums to args.workspace and runs the ordered reduction.
bool gemm_skinny_supported(int64_t M, bool y_colmajor);
int launch_fp8_gemm_skinny(const GemmArgs& args, DeviceCtx* ctx, int splits, int mode);
// out = cast(sum over splits of workspace[split][M][N]), in split order.
int launch_splitk_reduce(const GemmArgs& args, int splits);

// Split-K launch whose partial sums live in the library's static device array (no allocation).
int launch_fp8_gemm_static_scratch(const GemmArgs& args, int splits);
// Makes the tensor-map encoder available without creating a device context (no allocation).
int ensure_tmap_encoder();

struct AttnArgs {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  int64_t BH, S, D;        // S = query rows per slice
  int64_t Sk = 0;          // keys per slice (= S for the reference's square problem)
  int causal = 0;          // hide key j from query i when j > i + (Sk - S)
  int kind = 0;            // 0 = e4m3; 1 = fp16, 2 = bf16 (attention_16bit.cu: v is then [BH, Sk, D], strides {bh, s, d})
  int64_t q_strides[3];
  int64_t k_strides[3];
  int64_t v_strides[3];    // logical [BH, D, S]
  int64_t out_strides[3];  // [BH, S, D]
  float scale_log2;
  int out_dtype;
  int cfg_id;
  int device;
  cudaStream_t stream;
  unsigned int* sched;  // zeroed tile counter in device memory, or null for the static tile order
};

int launch_fp8_attention(const AttnArgs& args, DeviceCtx* ctx);
// fp16 / bf16 attention (attention_16bit.cu); args.kind, args.Sk and args.sched are honoured, args.cfg_id is not.
int launch_attention_16bit(const AttnArgs& args, DeviceCtx* ctx);
// q, k, v (fp16 / bf16 / fp32, `count` elements each) -> e4m3fn with torch's cast rule (quantize.cu).
int launch_attention_preprocess(const void* q, const void* k, const void* v, void* q8, void* k8, void* v8, int64_t count,
                                int src_dtype, DeviceCtx* ctx, cudaStream_t stream);
// The two-tile attention kernel (fp8_attention_pair.cu) on tensor maps built for 128-key steps; non-causal only.
int launch_fp8_attention_pair(const AttnArgs& args, DeviceCtx* ctx, const CUtensorMap& tq, const CUtensorMap& tk,
                              const CUtensorMap& tv, bool v_kmajor, int poly_of8, bool lazy);
// Softmax-only ceiling kernel (softmax_ceiling.cu): `cycles` receives one SM-clock count per CTA.
int launch_softmax_ceiling(int wgs, int ctas_per_sm, int poly_of8, int mode, int steps, unsigned long long* cycles,
                           DeviceCtx* ctx, cudaStream_t stream);
int attn_num_configs();
int attn_describe_config(int cfg_id, char* buf, int buf_len);

// Launch with programmatic stream serialization allowed: the kernel may start while its predecessor in
// the stream drains, and must call pdl_wait() (common.cuh) before it touches global memory.  After a
// predecessor that never triggers early (any ordinary kernel or copy) this is a plain in-order launch.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem_bytes, cudaStream_t stream,
                       Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(block, 1, 1);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
#ifdef HB_NO_PDL  // development builds only: plain in-order launches, to measure what the early launch is worth
  cfg.numAttrs = 0;
#else
  cfg.numAttrs = 1;
#endif
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace hb
