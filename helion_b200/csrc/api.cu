// C ABI of the library (declared in include/helion_b200.h): argument validation, per-device
// context, error text.  The kernels and their launchers live in fp8_gemm.cu / fp8_attention.cu.
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "host.h"

namespace hb {

namespace {
constexpr int kMaxDevices = 64;
DeviceCtx g_ctx[kMaxDevices];
std::mutex g_ctx_mutex;
thread_local std::string g_last_error;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode_tiled = nullptr;
}  // namespace

int set_error(int code, const std::string& text) {
  g_last_error = text;
  return code;
}

const char* last_error_text() { return g_last_error.c_str(); }

DeviceCtx* get_device_ctx(int device) {
  if (device < 0 || device >= kMaxDevices) {
    set_error(HB200_ERR_CUDA, "device index out of range");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_ctx_mutex);
  DeviceCtx& c = g_ctx[device];
  if (c.initialised) {
    if (c.init_error != 0) {
      set_error(c.init_error, "device initialisation failed earlier (not an sm_100 GPU, or a CUDA error)");
      return nullptr;
    }
    return &c;
  }
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || device >= count) {
    // Not cached: a later call may find a GPU.
    set_error(HB200_ERR_CUDA, std::string("no such CUDA device: ") + (e != cudaSuccess ? cudaGetErrorString(e) : "index beyond device count"));
    return nullptr;
  }
  DeviceGuard guard(device);
  if (!guard.ok()) {
    set_error(HB200_ERR_CUDA, "cannot make device " + std::to_string(device) + " current");
    return nullptr;  // not cached: a later call may succeed
  }
  c.initialised = true;
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) {
    c.init_error = HB200_ERR_CUDA;
    set_error(HB200_ERR_CUDA, std::string("cudaGetDeviceProperties: ") + cudaGetErrorString(e));
    return nullptr;
  }
  c.num_sms = prop.multiProcessorCount;
  c.cc_major = prop.major;
  c.cc_minor = prop.minor;
  if (prop.major != 10) {
    c.init_error = HB200_ERR_UNSUPPORTED_ARCH;
    set_error(HB200_ERR_UNSUPPORTED_ARCH, "this library holds sm_100a code only; device is sm_" +
                                              std::to_string(prop.major) + std::to_string(prop.minor));
    return nullptr;
  }
  e = cudaHostAlloc(reinterpret_cast<void**>(&c.status_host), 64, cudaHostAllocMapped);
  if (e == cudaSuccess) {
    std::memset(c.status_host, 0, 64);
    e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&c.status_dev), c.status_host, 0);
  }
  if (e != cudaSuccess) {
    c.init_error = HB200_ERR_CUDA;
    set_error(HB200_ERR_CUDA, std::string("status word allocation: ") + cudaGetErrorString(e));
    return nullptr;
  }
  if (g_encode_tiled == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || fn == nullptr || qres != cudaDriverEntryPointSuccess) {
      c.init_error = HB200_ERR_CUDA;
      set_error(HB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
      return nullptr;
    }
    g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
  }
  return &c;
}

uint32_t* peek_status_dev(int device) {
  if (device < 0 || device >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_ctx_mutex);
  const DeviceCtx& c = g_ctx[device];
  return (c.initialised && c.init_error == 0) ? c.status_dev : nullptr;
}

int ensure_tmap_encoder() {
  std::lock_guard<std::mutex> lock(g_ctx_mutex);
  if (g_encode_tiled != nullptr) return HB200_OK;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || fn == nullptr || qres != cudaDriverEntryPointSuccess) {
    return set_error(HB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  }
  g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
  return HB200_OK;
}

int device_init_error(int device) {
  if (device >= 0 && device < kMaxDevices && g_ctx[device].init_error != 0) return g_ctx[device].init_error;
  return HB200_ERR_CUDA;
}

namespace {
// Encoded tensor maps of this thread's recent launches: a serving loop launches the same few (pointer, shape,
// strides, box) combinations over and over, and an encode is a driver call.  Thread-local, so re-entrant without a
// lock; a map depends on nothing but its key (the driver encodes it on the host from these values alone).
struct TmapKey {
  const void* base;
  uint64_t dims[3];
  uint64_t strides[2];
  uint32_t box[3];
  int rank, dtype, swizzle;
  bool operator==(const TmapKey& o) const { return std::memcmp(this, &o, sizeof(TmapKey)) == 0; }
};
struct TmapCache {
  static constexpr int kEntries = 16;
  TmapKey keys[kEntries];
  CUtensorMap maps[kEntries];
  int used = 0, next = 0;
};
thread_local TmapCache t_tmap_cache;
}  // namespace

int encode_tmap(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, int rank, const uint64_t* dims,
                const uint64_t* strides, const uint32_t* box, CUtensorMapSwizzle swizzle) {
  if (g_encode_tiled == nullptr) return set_error(HB200_ERR_CUDA, "tensor-map encoder not initialised");
  TmapKey key;
  std::memset(&key, 0, sizeof(key));  // padding too: keys are compared as bytes
  const bool cacheable = rank >= 1 && rank <= 3;
  if (cacheable) {
    key.base = base;
    key.rank = rank;
    key.dtype = static_cast<int>(dtype);
    key.swizzle = static_cast<int>(swizzle);
    for (int i = 0; i < rank; ++i) {
      key.dims[i] = dims[i];
      key.box[i] = box[i];
      if (i + 1 < rank) key.strides[i] = strides[i];
    }
    TmapCache& c = t_tmap_cache;
    for (int i = 0; i < c.used; ++i) {
      if (c.keys[i] == key) {
        *map = c.maps[i];
        return HB200_OK;
      }
    }
  }
  cuuint64_t gdims[5];
  cuuint64_t gstrides[5];
  cuuint32_t gbox[5];
  cuuint32_t gelem[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    gelem[i] = 1;
    if (i + 1 < rank) gstrides[i] = strides[i];
  }
  CUresult r = g_encode_tiled(map, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdims, gstrides,
                              gbox, gelem, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[256];
    std::snprintf(buf, sizeof(buf),
                  "cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dims %llu x %llu, stride0 %llu, box %u x %u)",
                  static_cast<int>(r), rank, (unsigned long long)dims[0], (unsigned long long)(rank > 1 ? dims[1] : 0),
                  (unsigned long long)(rank > 1 ? strides[0] : 0), box[0], rank > 1 ? box[1] : 0);
    return set_error(HB200_ERR_CUDA, buf);
  }
  if (cacheable) {
    TmapCache& c = t_tmap_cache;
    const int slot = c.used < TmapCache::kEntries ? c.used++ : (c.next++ % TmapCache::kEntries);
    c.keys[slot] = key;
    c.maps[slot] = *map;
  }
  return HB200_OK;
}

int encode_tmap_u8(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides,
                   const uint32_t* box, CUtensorMapSwizzle swizzle) {
  return encode_tmap(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, base, rank, dims, strides, box, swizzle);
}

}  // namespace hb

namespace hb {
namespace selftest {
// One CTA waits on an mbarrier that nothing arrives on; the bounded wait gives up after `limit_ns`,
// records SITE_SELFTEST in the status word and the kernel returns normally.
__global__ void wait_selftest_kernel(uint32_t* status, unsigned long long limit_ns, int* gave_up) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  const WaitCtx wctx{&abort_flag, status};
  const bool completed = mbar_wait_limited(&bar, 0, wctx, SITE_SELFTEST, limit_ns);
  if (threadIdx.x == 0 && gave_up != nullptr) *gave_up = completed ? 0 : 1;
}
}  // namespace selftest
}  // namespace hb

using namespace hb;

static int ctx_error_code(int device) {
  return hb::device_init_error(device);
}

extern "C" {

int hb200_version(void) { return HB200_VERSION; }

const char* hb200_last_error(void) { return last_error_text(); }

int hb200_num_sms(int device) {
  DeviceCtx* ctx = get_device_ctx(device);
  return ctx == nullptr ? HB200_ERR_CUDA : ctx->num_sms;
}

int hb200_read_status(int device, uint32_t* site) {
  DeviceCtx* ctx = get_device_ctx(device);
  if (ctx == nullptr) return HB200_ERR_CUDA;
  uint32_t v = *reinterpret_cast<volatile uint32_t*>(ctx->status_host);
  if (site != nullptr) *site = v;
  if (v != 0) {
    char buf[128];
    std::snprintf(buf, sizeof(buf), "a device-side wait ran out: site %u, block %u", v >> 16, v & 0xffffu);
    return set_error(HB200_ERR_TIMEOUT, buf);
  }
  return HB200_OK;
}

int hb200_reset_status(int device) {
  DeviceCtx* ctx = get_device_ctx(device);
  if (ctx == nullptr) return HB200_ERR_CUDA;
  *reinterpret_cast<volatile uint32_t*>(ctx->status_host) = 0;
  return HB200_OK;
}

int hb200_debug_wait_selftest(int device, int limit_ms, void* stream) {
  if (limit_ms < 1 || limit_ms > 1000) return set_error(HB200_ERR_BAD_CONFIG, "wait self-test: limit must be 1..1000 ms");
  DeviceCtx* ctx = get_device_ctx(device);
  if (ctx == nullptr) return device_init_error(device);
  HB_DEVICE_GUARD(device);
  selftest::wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      ctx->status_dev, static_cast<unsigned long long>(limit_ms) * 1000000ull, nullptr);
  HB_CUDA_CHECK(cudaGetLastError());
  return HB200_OK;
}

int hb200_debug_softmax_ceiling(int wgs, int ctas_per_sm, int poly_of8, int mode, int steps, void* cycles, int device,
                                void* stream) {
  if (wgs < 1 || wgs > 2 || ctas_per_sm < 1 || ctas_per_sm > 2 || (wgs == 2 && ctas_per_sm != 1)) {
    return set_error(HB200_ERR_BAD_CONFIG, "softmax_ceiling: 1 or 2 warpgroups per CTA; 2 CTAs per SM only with 1 warpgroup");
  }
  const bool noise_mode = mode == 17 || mode == 18 || mode == 20 || mode == 24 || mode == 31;
  if (!((mode >= 0 && mode <= 3) || noise_mode) || steps < 1 || steps > (1 << 20)) {
    return set_error(HB200_ERR_BAD_CONFIG, "softmax_ceiling: mode must be 0..3 or 16 + a noise mask of 1, 2, 4, 8, 15; steps 1..2^20");
  }
  if (noise_mode && (wgs != 2 || poly_of8 != 0)) {
    return set_error(HB200_ERR_BAD_CONFIG, "softmax_ceiling: the noise modes run two warpgroups with all exp2 on the MUFU unit");
  }
  if (cycles == nullptr || (reinterpret_cast<uintptr_t>(cycles) & 7u)) {
    return set_error(HB200_ERR_ALIGN, "softmax_ceiling: cycles must be an 8-byte aligned device pointer");
  }
  DeviceCtx* ctx = get_device_ctx(device);
  if (ctx == nullptr) return ctx_error_code(device);
  HB_DEVICE_GUARD(device);
  return launch_softmax_ceiling(wgs, ctas_per_sm, poly_of8, mode, steps, static_cast<unsigned long long*>(cycles), ctx,
                                static_cast<cudaStream_t>(stream));
}

int hb200_num_configs(int op) {
  if (op == HB200_OP_GEMM) return gemm_num_configs();
  if (op == HB200_OP_ATTENTION) return attn_num_configs();
  return set_error(HB200_ERR_BAD_CONFIG, "unknown op");
}

int hb200_describe_config(int op, int cfg_id, char* buf, int buf_len) {
  if (buf == nullptr || buf_len <= 0) return set_error(HB200_ERR_BAD_CONFIG, "no buffer");
  if (op == HB200_OP_GEMM) return gemm_describe_config(cfg_id, buf, buf_len);
  if (op == HB200_OP_ATTENTION) return attn_describe_config(cfg_id, buf, buf_len);
  return set_error(HB200_ERR_BAD_CONFIG, "unknown op");
}

size_t hb200_fp8_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int out_dtype, int cfg_id) {
  return gemm_workspace_bytes(M, N, K, out_dtype, cfg_id);
}

// SM count the table choice is made for: that of the current device when one can be asked without creating
// anything, else 148 (B200).  The launch itself always uses the count of the device it runs on.
static int query_num_sms() {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) == cudaSuccess &&
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0) {
    return sms;
  }
  cudaGetLastError();  // no device: not an error of this call
  return 148;
}

int hb200_fp8_gemm_select_config(int64_t M, int64_t N, int64_t K, int y_is_colmajor, int out_dtype) {
  return gemm_select_config(M, N, K, y_is_colmajor != 0, out_dtype, query_num_sms());
}

// Validation and launch shared by hb200_fp8_gemm (scale_mode 0) and hb200_fp8_gemm_scaled.
static int fp8_gemm_impl(const void* x, const void* y, void* out, int64_t M, int64_t N, int64_t K, int64_t x_rs,
                         int64_t x_cs, int64_t y_rs, int64_t y_cs, int64_t out_rs, int out_dtype, const float* scale_a,
                         const float* scale_b, int scale_mode, int cfg_id, void* workspace, size_t workspace_bytes,
                         int device, void* stream) {
  if (scale_mode != HB200_SCALE_NONE && scale_mode != HB200_SCALE_TENSOR && scale_mode != HB200_SCALE_ROWWISE) {
    return set_error(HB200_ERR_BAD_CONFIG, "fp8_gemm_scaled: scale_mode must be HB200_SCALE_TENSOR or HB200_SCALE_ROWWISE");
  }
  if (scale_mode != HB200_SCALE_NONE) {
    if (scale_a == nullptr || scale_b == nullptr) return set_error(HB200_ERR_ALIGN, "fp8_gemm_scaled: null scale pointer");
    if ((reinterpret_cast<uintptr_t>(scale_a) | reinterpret_cast<uintptr_t>(scale_b)) & 3u) {
      return set_error(HB200_ERR_ALIGN, "fp8_gemm_scaled: scale pointers must be 4-byte aligned");
    }
  }
  if (out_dtype != HB200_DT_FP16 && out_dtype != HB200_DT_BF16 && out_dtype != HB200_DT_FP32) {
    return set_error(HB200_ERR_BAD_DTYPE, "fp8_gemm: out_dtype must be FP16, BF16 or FP32");
  }
  if (M < 1 || N < 1 || K < 1 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) {
    return set_error(HB200_ERR_BAD_SHAPE, "fp8_gemm: M, N, K must be in [1, 2^31)");
  }
  if (K % 16 != 0) return set_error(HB200_ERR_BAD_SHAPE, "fp8_gemm: K must be a multiple of 16");
  if (N % 8 != 0) return set_error(HB200_ERR_BAD_SHAPE, "fp8_gemm: N must be a multiple of 8");
  if (x == nullptr || y == nullptr || out == nullptr) return set_error(HB200_ERR_ALIGN, "fp8_gemm: null pointer");
  if (x_cs != 1) return set_error(HB200_ERR_BAD_STRIDE, "fp8_gemm: x must be row-major (column stride 1)");
  if (x_rs < K || x_rs % 16 != 0) {
    return set_error(HB200_ERR_BAD_STRIDE, "fp8_gemm: x row stride must be >= K and a multiple of 16");
  }
  bool y_colmajor;
  int64_t ldb;
  if (y_rs == 1 && (K == 1 || y_cs >= K)) {
    y_colmajor = true;
    ldb = y_cs;
  } else if (y_cs == 1 && y_rs >= N) {
    y_colmajor = false;
    ldb = y_rs;
    if (N % 16 != 0) return set_error(HB200_ERR_BAD_SHAPE, "fp8_gemm: row-major y needs N to be a multiple of 16");
  } else {
    return set_error(HB200_ERR_BAD_STRIDE, "fp8_gemm: y must be column-major (row stride 1) or row-major (column stride 1)");
  }
  if (ldb % 16 != 0) return set_error(HB200_ERR_BAD_STRIDE, "fp8_gemm: y leading stride must be a multiple of 16");
  const int64_t out_elem = out_dtype == HB200_DT_FP32 ? 4 : 2;
  if (out_rs < N || (out_rs * out_elem) % 16 != 0) {
    return set_error(HB200_ERR_BAD_STRIDE, "fp8_gemm: out row stride must be >= N and give 16-byte aligned rows");
  }
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out)) & 15u) {
    return set_error(HB200_ERR_ALIGN, "fp8_gemm: x, y and out must be 16-byte aligned");
  }
  DeviceCtx* ctx = get_device_ctx(device);
  if (ctx == nullptr) return ctx_error_code(device);
  GemmArgs a;
  a.x = x;
  a.y = y;
  a.out = out;
  a.M = M;
  a.N = N;
  a.K = K;
  a.lda = x_rs;
  a.ldb = ldb;
  a.y_colmajor = y_colmajor;
  a.ldc = out_rs;
  a.out_dtype = out_dtype;
  a.cfg_id = cfg_id;
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  a.device = device;
  a.stream = static_cast<cudaStream_t>(stream);
  a.scale_a = scale_a;
  a.scale_b = scale_b;
  a.scale_mode = scale_mode;
  HB_DEVICE_GUARD(device);
  return launch_fp8_gemm(a, ctx);
}

int hb200_fp8_gemm(const void* x, const void* y, void* out, int64_t M, int64_t N, int64_t K, int64_t x_rs,
                   int64_t x_cs, int64_t y_rs, int64_t y_cs, int64_t out_rs, int out_dtype, int cfg_id,
                   void* workspace, size_t workspace_bytes, int device, void* stream) {
  return fp8_gemm_impl(x, y, out, M, N, K, x_rs, x_cs, y_rs, y_cs, out_rs, out_dtype, nullptr, nullptr,
                       HB200_SCALE_NONE, cfg_id, workspace, workspace_bytes, device, stream);
}

int hb200_fp8_gemm_scaled(const void* x, const void* y, void* out, int64_t M, int64_t N, int64_t K, int64_t x_rs,
                          int64_t x_cs, int64_t y_rs, int64_t y_cs, int64_t out_rs, int out_dtype,
                          const float* scale_a, const float* scale_b, int scale_mode, int cfg_id, void* workspace,
                          size_t workspace_bytes, int device, void* stream) {
  if (scale_mode == HB200_SCALE_NONE) {
    return set_error(HB200_ERR_BAD_CONFIG, "fp8_gemm_scaled: scale_mode must be HB200_SCALE_TENSOR or HB200_SCALE_ROWWISE");
  }
  return fp8_gemm_impl(x, y, out, M, N, K, x_rs, x_cs, y_rs, y_cs, out_rs, out_dtype, scale_a, scale_b, scale_mode,
                       cfg_id, workspace, workspace_bytes, device, stream);
}

int hb200_gemm_16bit(const void* x, const void* y, void* out, int64_t M, int64_t N, int64_t K, int64_t x_rs, int64_t x_cs,
                     int64_t y_rs, int64_t y_cs, int64_t out_rs, int in_dtype, int out_dtype, const float* bias, int relu,
                     int cfg_id, int device, void* stream) {
  if (in_dtype != HB200_DT_FP16 && in_dtype != HB200_DT_BF16) {
    return set_error(HB200_ERR_BAD_DTYPE, "gemm_16bit: in_dtype must be FP16 or BF16");
  }
  if (out_dtype != in_dtype && out_dtype != HB200_DT_FP32) {
    return set_error(HB200_ERR_BAD_DTYPE, "gemm_16bit: out_dtype must be the operands' dtype or FP32");
  }
  if (M < 1 || N < 1 || K < 1 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX / 2) {
    return set_error(HB200_ERR_BAD_SHAPE, "gemm_16bit: M, N must be in [1, 2^31) and K in [1, 2^30)");
  }
  if (K % 8 != 0) return set_error(HB200_ERR_BAD_SHAPE, "gemm_16bit: K must be a multiple of 8");
  if (N % 8 != 0) return set_error(HB200_ERR_BAD_SHAPE, "gemm_16bit: N must be a multiple of 8");
  if (x == nullptr || y == nullptr || out == nullptr) return set_error(HB200_ERR_ALIGN, "gemm_16bit: null pointer");
  if (x_cs != 1) return set_error(HB200_ERR_BAD_STRIDE, "gemm_16bit: x must be row-major (column stride 1)");
  if (x_rs < K || x_rs % 8 != 0) {
    return set_error(HB200_ERR_BAD_STRIDE, "gemm_16bit: x row stride must be >= K and a multiple of 8");
  }
  bool y_colmajor;
  int64_t ldb;
  if (y_rs == 1 && (K == 1 || y_cs >= K)) {
    y_colmajor = true;
    ldb = y_cs;
  } else if (y_cs == 1 && y_rs >= N) {
    y_colmajor = false;
    ldb = y_rs;
  } else {
    return set_error(HB200_ERR_BAD_STRIDE, "gemm_16bit: y must be column-major (row stride 1) or row-major (column stride 1)");
  }
  if (ldb % 8 != 0) return set_error(HB200_ERR_BAD_STRIDE, "gemm_16bit: y leading stride must be a multiple of 8");
  const int64_t out_elem = out_dtype == HB200_DT_FP32 ? 4 : 2;
  if (out_rs < N || (out_rs * out_elem) % 16 != 0) {
    return set_error(HB200_ERR_BAD_STRIDE, "gemm_16bit: out row stride must be >= N and give 16-byte aligned rows");
  }
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out)) & 15u) {
    return set_error(HB200_ERR_ALIGN, "gemm_16bit: x, y and out must be 16-byte aligned");
  }
  if (bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 3u)) {
    return set_error(HB200_ERR_ALIGN, "gemm_16bit: bias must be 4-byte aligned");
  }
  DeviceCtx* ctx = get_device_ctx(device);
  if (ctx == nullptr) return ctx_error_code(device);
  GemmArgs a;
  a.x = x;
  a.y = y;
  a.out = out;
  a.M = M;
  a.N = N;
  a.K = K;
  a.lda = x_rs;
  a.ldb = ldb;
  a.y_colmajor = y_colmajor;
  a.ldc = out_rs;
  a.out_dtype = out_dtype;
  a.cfg_id = cfg_id;
  a.workspace = nullptr;
  a.workspace_bytes = 0;
  a.device = device;
  a.stream = static_cast<cudaStream_t>(stream);
  a.kind = in_dtype == HB200_DT_FP16 ? 1 : 2;
  a.bias = bias;
  a.relu = relu != 0 ? 1 : 0;
  HB_DEVICE_GUARD(device);
  return launch_gemm_16bit(a, ctx);
}

int hb200_fp8_gemm_splitk_static(const void* x, const void* y, void* out, int64_t M, int64_t N, int64_t K,
                                 int64_t x_rs, int64_t x_cs, int64_t y_rs, int64_t y_cs, int64_t out_rs, int out_dtype,
                                 int splits, int device, void* stream) {
  // Same argument contract as hb200_fp8_gemm, checked here again so that this entry point shares no
  // code path with it before the launch.
  if (out_dtype != HB200_DT_FP16 && out_dtype != HB200_DT_BF16 && out_dtype != HB200_DT_FP32) {
    return set_error(HB200_ERR_BAD_DTYPE, "fp8_gemm_splitk_static: out_dtype must be FP16, BF16 or FP32");
  }
  if (M < 1 || N < 1 || K < 1 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) {
    return set_error(HB200_ERR_BAD_SHAPE, "fp8_gemm_splitk_static: M, N, K must be in [1, 2^31)");
  }
  if (K % 16 != 0 || N % 8 != 0) {
    return set_error(HB200_ERR_BAD_SHAPE, "fp8_gemm_splitk_static: K must be a multiple of 16 and N of 8");
  }
  if (splits < 2 || splits > 8) return set_error(HB200_ERR_BAD_CONFIG, "fp8_gemm_splitk_static: splits must be 2..8");
  if (x == nullptr || y == nullptr || out == nullptr) {
    return set_error(HB200_ERR_ALIGN, "fp8_gemm_splitk_static: null pointer");
  }
  if (x_cs != 1 || x_rs < K || x_rs % 16 != 0) {
    return set_error(HB200_ERR_BAD_STRIDE, "fp8_gemm_splitk_static: x must be row-major with a row stride >= K, multiple of 16");
  }
  bool y_colmajor;
  int64_t ldb;
  if (y_rs == 1 && (K == 1 || y_cs >= K)) {
    y_colmajor = true;
    ldb = y_cs;
  } else if (y_cs == 1 && y_rs >= N && N % 16 == 0) {
    y_colmajor = false;
    ldb = y_rs;
  } else {
    return set_error(HB200_ERR_BAD_STRIDE,
                     "fp8_gemm_splitk_static: y must be column-major, or row-major with N a multiple of 16");
  }
  if (ldb % 16 != 0) {
    return set_error(HB200_ERR_BAD_STRIDE, "fp8_gemm_splitk_static: y leading stride must be a multiple of 16");
  }
  const int64_t out_elem = out_dtype == HB200_DT_FP32 ? 4 : 2;
  if (out_rs < N || (out_rs * out_elem) % 16 != 0) {
    return set_error(HB200_ERR_BAD_STRIDE, "fp8_gemm_splitk_static: out rows must be >= N long and 16-byte aligned");
  }
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out)) & 15u) {
    return set_error(HB200_ERR_ALIGN, "fp8_gemm_splitk_static: x, y and out must be 16-byte aligned");
  }
  if (device < 0 || device >= kMaxDevices) return set_error(HB200_ERR_CUDA, "device index out of range");
  {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device >= count) {
      cudaGetLastError();
      return set_error(HB200_ERR_CUDA, "fp8_gemm_splitk_static: no such CUDA device");
    }
  }
  GemmArgs a;
  a.x = x;
  a.y = y;
  a.out = out;
  a.M = M;
  a.N = N;
  a.K = K;
  a.lda = x_rs;
  a.ldb = ldb;
  a.y_colmajor = y_colmajor;
  a.ldc = out_rs;
  a.out_dtype = out_dtype;
  a.cfg_id = -1;
  a.workspace = nullptr;  // filled in by the launcher with the static array's address
  a.workspace_bytes = 0;
  a.device = device;
  a.stream = static_cast<cudaStream_t>(stream);
  HB_DEVICE_GUARD(device);
  return launch_fp8_gemm_static_scratch(a, splits);
}

// Validation and launch shared by the two attention entry points; workspace == nullptr selects
// the static tile order.
static int fp8_attention_impl(const void* q, const void* k, const void* v, void* out, int64_t BH, int64_t S, int64_t Sk,
                              int causal, int64_t D, const int64_t q_strides[3], const int64_t k_strides[3],
                              const int64_t v_strides[3], const int64_t out_strides[3], float scale_log2,
                              int out_dtype, int cfg_id, void* workspace, size_t workspace_bytes, int device,
                              void* stream) {
  if (out_dtype != HB200_DT_E4M3 && out_dtype != HB200_DT_BF16 && out_dtype != HB200_DT_FP32) {
    return set_error(HB200_ERR_BAD_DTYPE, "fp8_attention: out_dtype must be E4M3, BF16 or FP32");
  }
  if (D != 64 && D != 128) return set_error(HB200_ERR_BAD_SHAPE, "fp8_attention: head_dim must be 64 or 128");
  if (BH < 1 || S < 1 || BH > INT32_MAX || S > INT32_MAX) {
    return set_error(HB200_ERR_BAD_SHAPE, "fp8_attention: batch*heads and seq must be in [1, 2^31)");
  }
  if (Sk < 1 || Sk > INT32_MAX) return set_error(HB200_ERR_BAD_SHAPE, "fp8_attention: seq_k must be in [1, 2^31)");
  if (causal != 0 && Sk < S) {
    return set_error(HB200_ERR_BAD_SHAPE, "fp8_attention: the causal mask needs seq_k >= seq_q (every query must see a key)");
  }
  if (q == nullptr || k == nullptr || v == nullptr || out == nullptr || q_strides == nullptr ||
      k_strides == nullptr || v_strides == nullptr || out_strides == nullptr) {
    return set_error(HB200_ERR_ALIGN, "fp8_attention: null pointer");
  }
  if (q_strides[2] != 1 || k_strides[2] != 1 || out_strides[2] != 1) {
    return set_error(HB200_ERR_BAD_STRIDE, "fp8_attention: q, k and out need a unit head_dim stride");
  }
  if (q_strides[1] % 16 != 0 || k_strides[1] % 16 != 0 || q_strides[0] % 16 != 0 || k_strides[0] % 16 != 0 ||
      q_strides[1] < D || k_strides[1] < D) {
    return set_error(HB200_ERR_BAD_STRIDE, "fp8_attention: q/k row and slice strides must be multiples of 16 and >= D");
  }
  if (!((v_strides[1] == 1 && v_strides[2] >= D) || (v_strides[2] == 1 && v_strides[1] >= Sk))) {
    return set_error(HB200_ERR_BAD_STRIDE,
                     "fp8_attention: v (logical [BH, D, S]) must have a unit stride along D or along S");
  }
  if (v_strides[0] % 16 != 0 || (v_strides[1] == 1 ? v_strides[2] : v_strides[1]) % 16 != 0) {
    return set_error(HB200_ERR_BAD_STRIDE, "fp8_attention: v strides must be multiples of 16");
  }
  const int64_t out_elem = out_dtype == HB200_DT_FP32 ? 4 : (out_dtype == HB200_DT_BF16 ? 2 : 1);
  if (out_strides[1] < D || (out_strides[1] * out_elem) % 16 != 0 || (out_strides[0] * out_elem) % 16 != 0) {
    return set_error(HB200_ERR_BAD_STRIDE, "fp8_attention: out rows must be 16-byte aligned");
  }
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(out)) & 15u) {
    return set_error(HB200_ERR_ALIGN, "fp8_attention: q, k, v and out must be 16-byte aligned");
  }
  DeviceCtx* ctx = get_device_ctx(device);
  if (ctx == nullptr) return ctx_error_code(device);
  AttnArgs a;
  a.q = q;
  a.k = k;
  a.v = v;
  a.out = out;
  a.BH = BH;
  a.S = S;
  a.Sk = Sk;
  a.causal = causal != 0 ? 1 : 0;
  a.D = D;
  for (int i = 0; i < 3; ++i) {
    a.q_strides[i] = q_strides[i];
    a.k_strides[i] = k_strides[i];
    a.v_strides[i] = v_strides[i];
    a.out_strides[i] = out_strides[i];
  }
  a.scale_log2 = scale_log2;
  a.out_dtype = out_dtype;
  a.cfg_id = cfg_id;
  a.device = device;
  a.stream = static_cast<cudaStream_t>(stream);
  a.sched = nullptr;
  HB_DEVICE_GUARD(device);
  if (workspace != nullptr) {
    if (workspace_bytes < HB200_ATTN_WORKSPACE_BYTES) {
      return set_error(HB200_ERR_WORKSPACE, "fp8_attention: workspace smaller than HB200_ATTN_WORKSPACE_BYTES");
    }
    if (reinterpret_cast<uintptr_t>(workspace) & 15u) {
      return set_error(HB200_ERR_ALIGN, "fp8_attention: workspace must be 16-byte aligned");
    }
    // the tile counter starts at zero for every launch; the clear is ordered before the kernel on
    // the same stream and allocates nothing
    HB_CUDA_CHECK(cudaMemsetAsync(workspace, 0, HB200_ATTN_WORKSPACE_BYTES, a.stream));
    a.sched = static_cast<unsigned int*>(workspace);
  }
  return launch_fp8_attention(a, ctx);
}

int hb200_fp8_attention(const void* q, const void* k, const void* v, void* out, int64_t BH, int64_t S, int64_t D,
                        const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                        const int64_t out_strides[3], float scale_log2, int out_dtype, int cfg_id, int device,
                        void* stream) {
  return fp8_attention_impl(q, k, v, out, BH, S, S, 0, D, q_strides, k_strides, v_strides, out_strides, scale_log2,
                            out_dtype, cfg_id, nullptr, 0, device, stream);
}

int hb200_attention_16bit(const void* q, const void* k, const void* v, void* out, int64_t BH, int64_t S_q, int64_t S_k,
                          int64_t D, const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                          const int64_t out_strides[3], float scale_log2, int in_dtype, int out_dtype, void* workspace,
                          size_t workspace_bytes, int device, void* stream) {
  if (in_dtype != HB200_DT_FP16 && in_dtype != HB200_DT_BF16) {
    return set_error(HB200_ERR_BAD_DTYPE, "attention_16bit: in_dtype must be FP16 or BF16");
  }
  if (out_dtype != in_dtype && out_dtype != HB200_DT_FP32) {
    return set_error(HB200_ERR_BAD_DTYPE, "attention_16bit: out_dtype must be the operands' dtype or FP32");
  }
  if (D != 64 && D != 128) return set_error(HB200_ERR_BAD_SHAPE, "attention_16bit: head_dim must be 64 or 128");
  if (BH < 1 || S_q < 1 || S_k < 1 || BH > INT32_MAX || S_q > INT32_MAX || S_k > INT32_MAX) {
    return set_error(HB200_ERR_BAD_SHAPE, "attention_16bit: batch*heads, seq_q and seq_k must be in [1, 2^31)");
  }
  if (q == nullptr || k == nullptr || v == nullptr || out == nullptr || q_strides == nullptr || k_strides == nullptr ||
      v_strides == nullptr || out_strides == nullptr) {
    return set_error(HB200_ERR_ALIGN, "attention_16bit: null pointer");
  }
  if (q_strides[2] != 1 || k_strides[2] != 1 || v_strides[2] != 1 || out_strides[2] != 1) {
    return set_error(HB200_ERR_BAD_STRIDE, "attention_16bit: q, k, v and out need a unit head_dim stride");
  }
  const int64_t* in_strides[3] = {q_strides, k_strides, v_strides};
  for (const int64_t* st : in_strides) {
    if (st[1] < D || st[1] % 8 != 0 || st[0] % 8 != 0) {
      return set_error(HB200_ERR_BAD_STRIDE, "attention_16bit: row and slice strides must be multiples of 8 and rows >= D");
    }
  }
  const int64_t out_elem = out_dtype == HB200_DT_FP32 ? 4 : 2;
  if (out_strides[1] < D || (out_strides[1] * out_elem) % 16 != 0 || (out_strides[0] * out_elem) % 16 != 0) {
    return set_error(HB200_ERR_BAD_STRIDE, "attention_16bit: out rows must be 16-byte aligned");
  }
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(out)) & 15u) {
    return set_error(HB200_ERR_ALIGN, "attention_16bit: q, k, v and out must be 16-byte aligned");
  }
  DeviceCtx* ctx = get_device_ctx(device);
  if (ctx == nullptr) return ctx_error_code(device);
  AttnArgs a;
  a.q = q;
  a.k = k;
  a.v = v;
  a.out = out;
  a.BH = BH;
  a.S = S_q;
  a.Sk = S_k;
  a.D = D;
  for (int i = 0; i < 3; ++i) {
    a.q_strides[i] = q_strides[i];
    a.k_strides[i] = k_strides[i];
    a.v_strides[i] = v_strides[i];
    a.out_strides[i] = out_strides[i];
  }
  a.scale_log2 = scale_log2;
  a.out_dtype = out_dtype;
  a.cfg_id = -1;
  a.device = device;
  a.stream = static_cast<cudaStream_t>(stream);
  a.sched = nullptr;
  a.kind = in_dtype == HB200_DT_FP16 ? 1 : 2;
  HB_DEVICE_GUARD(device);
  if (workspace != nullptr) {
    if (workspace_bytes < HB200_ATTN_WORKSPACE_BYTES || (reinterpret_cast<uintptr_t>(workspace) & 15u)) {
      return set_error(HB200_ERR_WORKSPACE, "attention_16bit: workspace must be 16-byte aligned and hold HB200_ATTN_WORKSPACE_BYTES");
    }
    HB_CUDA_CHECK(cudaMemsetAsync(workspace, 0, HB200_ATTN_WORKSPACE_BYTES, a.stream));
    a.sched = static_cast<unsigned int*>(workspace);
  }
  return launch_attention_16bit(a, ctx);
}

int hb200_fp8_attention_preprocess(const void* q, const void* k, const void* v, void* q8, void* k8, void* v8,
                                   int64_t count, int src_dtype, int device, void* stream) {
  if (src_dtype != HB200_DT_FP16 && src_dtype != HB200_DT_BF16 && src_dtype != HB200_DT_FP32) {
    return set_error(HB200_ERR_BAD_DTYPE, "fp8_attention_preprocess: source dtype must be FP16, BF16 or FP32");
  }
  if (count < 1 || count % 16 != 0) {
    return set_error(HB200_ERR_BAD_SHAPE, "fp8_attention_preprocess: the element count must be a positive multiple of 16");
  }
  if (q == nullptr || k == nullptr || v == nullptr || q8 == nullptr || k8 == nullptr || v8 == nullptr) {
    return set_error(HB200_ERR_ALIGN, "fp8_attention_preprocess: null pointer");
  }
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(q8) | reinterpret_cast<uintptr_t>(k8) | reinterpret_cast<uintptr_t>(v8)) & 15u) {
    return set_error(HB200_ERR_ALIGN, "fp8_attention_preprocess: all six tensors must be 16-byte aligned");
  }
  DeviceCtx* ctx = get_device_ctx(device);
  if (ctx == nullptr) return ctx_error_code(device);
  HB_DEVICE_GUARD(device);
  return launch_attention_preprocess(q, k, v, q8, k8, v8, count, src_dtype, ctx, static_cast<cudaStream_t>(stream));
}

int hb200_fp8_attention_ws(const void* q, const void* k, const void* v, void* out, int64_t BH, int64_t S, int64_t D,
                           const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                           const int64_t out_strides[3], float scale_log2, int out_dtype, int cfg_id, void* workspace,
                           size_t workspace_bytes, int device, void* stream) {
  if (workspace == nullptr) return set_error(HB200_ERR_WORKSPACE, "fp8_attention_ws: workspace is null");
  return fp8_attention_impl(q, k, v, out, BH, S, S, 0, D, q_strides, k_strides, v_strides, out_strides, scale_log2,
                            out_dtype, cfg_id, workspace, workspace_bytes, device, stream);
}

int hb200_fp8_attention_ex(const void* q, const void* k, const void* v, void* out, int64_t BH, int64_t S_q, int64_t S_k,
                           int64_t D, const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                           const int64_t out_strides[3], float scale_log2, int causal, int out_dtype, int cfg_id,
                           void* workspace, size_t workspace_bytes, int device, void* stream) {
  return fp8_attention_impl(q, k, v, out, BH, S_q, S_k, causal, D, q_strides, k_strides, v_strides, out_strides,
                            scale_log2, out_dtype, cfg_id, workspace, workspace_bytes, device, stream);
}

}  // extern "C"
