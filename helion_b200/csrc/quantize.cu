// Input preparation for the FP8 attention kernel: q, k and v ([batch, heads, seq, head_dim] in
// fp16, bf16 or fp32) -> float8_e4m3fn, all three tensors in one launch.
//
// This is the arithmetic of preprocess_fp8_attention_inputs (examples/fp8_attention.py:110-133 of
// pytorch-labs/helion): three `.to(torch.float8_e4m3fn)` casts; the function's permute and reshapes
// only change strides (v stays physically [batch*heads, seq, head_dim]), so no data is re-laid out.
// The cast is torch's: round to nearest even, and -- unlike a saturating conversion -- a value that
// rounds beyond +-448 becomes NaN (0x7f / 0xff), because e4m3fn has no infinity.
//
// The kernel is bound by HBM traffic (2 or 4 bytes in, 1 byte out per element): every thread
// converts 16 consecutive elements per step with 16-byte loads and one 16-byte store, and the grid
// is a few CTAs per SM striding over the tensors.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "common.cuh"
#include "host.h"

namespace hb {

namespace {

struct QuantArgs {
  const void* src[3];
  void* dst[3];
  int64_t groups;  // 16-element groups per tensor
};

// Two floats -> two e4m3fn bytes with torch's overflow rule.  The hardware conversion saturates to
// +-448; 464 is the midpoint between 448 and the next (non-existent) value and ties go to the even
// mantissa, 448, so exactly the magnitudes above 464 (and infinities) turn into NaN, as does a NaN.
__device__ __forceinline__ uint32_t cast2_e4m3fn(float lo, float hi) {
  uint32_t r = pack_e4m3x2(lo, hi);
  if (!(fabsf(lo) <= 464.0f)) r |= 0x007fu;  // written so that NaN takes the branch too
  if (!(fabsf(hi) <= 464.0f)) r |= 0x7f00u;
  return r;
}

__device__ __forceinline__ uint32_t cast4_e4m3fn(float a, float b, float c, float d) {
  return cast2_e4m3fn(a, b) | (cast2_e4m3fn(c, d) << 16);
}

template <int SRC_DT>
__device__ __forceinline__ void load16(const void* src, int64_t group, float (&v)[16]) {
  if constexpr (SRC_DT == HB200_DT_FP32) {
    const float4* p = reinterpret_cast<const float4*>(src) + group * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 f = __ldcs(p + i);
      v[4 * i] = f.x;
      v[4 * i + 1] = f.y;
      v[4 * i + 2] = f.z;
      v[4 * i + 3] = f.w;
    }
  } else {
    const uint4* p = reinterpret_cast<const uint4*>(src) + group * 2;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint4 u = __ldcs(p + i);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f;
        if constexpr (SRC_DT == HB200_DT_FP16) {
          f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
        } else {
          f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
        }
        v[8 * i + 2 * j] = f.x;
        v[8 * i + 2 * j + 1] = f.y;
      }
    }
  }
}

template <int SRC_DT>
__global__ void __launch_bounds__(256) qkv_to_e4m3_kernel(QuantArgs a) {
  const void* src = a.src[blockIdx.y];
  uint4* dst = reinterpret_cast<uint4*>(a.dst[blockIdx.y]);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < a.groups; g += stride) {
    float v[16];
    load16<SRC_DT>(src, g, v);
    uint4 o;
    o.x = cast4_e4m3fn(v[0], v[1], v[2], v[3]);
    o.y = cast4_e4m3fn(v[4], v[5], v[6], v[7]);
    o.z = cast4_e4m3fn(v[8], v[9], v[10], v[11]);
    o.w = cast4_e4m3fn(v[12], v[13], v[14], v[15]);
    __stcs(dst + g, o);
  }
}

}  // namespace

int launch_attention_preprocess(const void* q, const void* k, const void* v, void* q8, void* k8, void* v8, int64_t count,
                                int src_dtype, DeviceCtx* ctx, cudaStream_t stream) {
  QuantArgs a;
  a.src[0] = q;
  a.src[1] = k;
  a.src[2] = v;
  a.dst[0] = q8;
  a.dst[1] = k8;
  a.dst[2] = v8;
  a.groups = count / 16;
  const int64_t want_blocks = (a.groups + 255) / 256;
  const dim3 grid(static_cast<unsigned>(std::min<int64_t>(want_blocks, static_cast<int64_t>(ctx->num_sms) * 8)), 3, 1);
  switch (src_dtype) {
    case HB200_DT_FP16:
      qkv_to_e4m3_kernel<HB200_DT_FP16><<<grid, 256, 0, stream>>>(a);
      break;
    case HB200_DT_BF16:
      qkv_to_e4m3_kernel<HB200_DT_BF16><<<grid, 256, 0, stream>>>(a);
      break;
    case HB200_DT_FP32:
      qkv_to_e4m3_kernel<HB200_DT_FP32><<<grid, 256, 0, stream>>>(a);
      break;
    default:
      return set_error(HB200_ERR_BAD_DTYPE, "fp8_attention_preprocess: source dtype must be FP16, BF16 or FP32");
  }
  HB_CUDA_CHECK(cudaGetLastError());
  return HB200_OK;
}

}  // namespace hb
