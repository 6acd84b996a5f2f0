/* helion_b200.h -- C ABI of the B200 (sm_100a) FP8 GEMM / FP8 attention library.
 *
 * The library replaces, for two kernels of pytorch-labs/helion, everything below the Python
 * call `fp8_gemm(x, y)` / `fp8_attention_kernel(q, k, v, batch, heads)`: Helion's generated
 * Triton kernel and its launcher (helion/runtime/__init__.py:55-65, `default_launcher`, which is
 * what the generated host function calls, test/test_examples.expected:836-840 and :786-790).
 * Helion has no FFI of its own (it is pure Python), so these entry points are the boundary a
 * maintainer binds with ctypes from the two example modules.
 *
 * Conventions
 *   - plain pointers and sizes only; all pointers are DEVICE pointers unless stated otherwise;
 *   - every launch is asynchronous on the given stream (a `cudaStream_t`, passed as void*) and
 *     performs no allocation and no synchronisation once the device has been initialised
 *     (first call on a device creates a small per-device context);
 *   - return value 0 = launched, negative = HB200_ERR_*; `hb200_last_error()` gives the text;
 *   - strides are in ELEMENTS;
 *   - fp8 means float8_e4m3fn bit patterns (1 byte per element).
 */
#ifndef HELION_B200_H
#define HELION_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HB200_VERSION 1

#if defined(__GNUC__)
#define HB200_API __attribute__((visibility("default")))
#else
#define HB200_API
#endif

/* error codes */
#define HB200_OK 0
#define HB200_ERR_BAD_DTYPE (-1)
#define HB200_ERR_BAD_SHAPE (-2)
#define HB200_ERR_BAD_STRIDE (-3)
#define HB200_ERR_ALIGN (-4)
#define HB200_ERR_UNSUPPORTED_ARCH (-5)
#define HB200_ERR_CUDA (-6)
#define HB200_ERR_TIMEOUT (-7)
#define HB200_ERR_BAD_CONFIG (-8)
#define HB200_ERR_WORKSPACE (-9)

/* output element types */
#define HB200_DT_FP16 0
#define HB200_DT_BF16 1
#define HB200_DT_FP32 2
#define HB200_DT_E4M3 3

/* operations (for the tile-config queries) */
#define HB200_OP_GEMM 0
#define HB200_OP_ATTENTION 1

/* out[M,N] = cast(x[M,K] @ y[K,N]), e4m3 operands, fp32 accumulation.
 * Replaces the device kernel of examples/fp8_gemm.py:29-57 (`fp8_gemm`) and its launch.
 *   x: fp8, x_cs must be 1 (row-major), x_rs % 16 == 0, pointer 16-byte aligned.
 *   y: fp8, either column-major (y_rs == 1, y_cs % 16 == 0) or row-major (y_cs == 1,
 *      y_rs % 16 == 0), pointer 16-byte aligned.
 *   out: row-major, out_rs in elements, rows 16-byte aligned; out_dtype one of FP16/BF16/FP32
 *      (FP16 is what the reference produces).
 *   K % 16 == 0, N % 8 == 0, M >= 1.
 *   cfg_id: index into the tile-config table, or -1 to let the library choose from the table.
 *      Every row computes the same product in stream order, with one exception that is never chosen
 *      automatically: row 23 (few rows of x, for chains of launches) starts reading y before the kernel
 *      that precedes it on the stream has ended.  Choosing it states that that kernel does not write y
 *      (y is a weight); x is read, and out written, only after the predecessor has ended.
 *   workspace: scratch for split-K configurations (fp32 partial sums), may be NULL when
 *      hb200_fp8_gemm_workspace_bytes() returns 0 for the configuration.
 */
HB200_API int hb200_fp8_gemm(const void* x, const void* y, void* out, int64_t M, int64_t N, int64_t K, int64_t x_rs,
                   int64_t x_cs, int64_t y_rs, int64_t y_cs, int64_t out_rs, int out_dtype, int cfg_id,
                   void* workspace, size_t workspace_bytes, int device, void* stream);

/* hb200_fp8_gemm with output scales: out = cast(((x @ y) * scale_a) * scale_b), the two
 * multiplications in fp32 on the fp32 accumulator, in that order, before the cast.  The reference
 * hard-codes unit scales (examples/fp8_gemm.py:74-75 and helion/language/matmul_ops.py:232-233 pass
 * torch.tensor(1.0) as scale_a and scale_b of torch._scaled_mm); callers with real FP8 tensors carry
 * scales, and this entry point takes the two forms torch._scaled_mm takes:
 *   HB200_SCALE_TENSOR:  scale_a and scale_b point to ONE float each (per-tensor scales);
 *   HB200_SCALE_ROWWISE: scale_a points to M floats (one per row of x / out), scale_b to N floats
 *                        (one per column of y / out).
 * The scales are device pointers to fp32, read when the kernel runs.  All other arguments and
 * limits are those of hb200_fp8_gemm; with unit scales the result equals hb200_fp8_gemm's bit for
 * bit. */
#define HB200_SCALE_NONE 0
#define HB200_SCALE_TENSOR 1
#define HB200_SCALE_ROWWISE 2
HB200_API int hb200_fp8_gemm_scaled(const void* x, const void* y, void* out, int64_t M, int64_t N, int64_t K,
                          int64_t x_rs, int64_t x_cs, int64_t y_rs, int64_t y_cs, int64_t out_rs, int out_dtype,
                          const float* scale_a, const float* scale_b, int scale_mode, int cfg_id, void* workspace,
                          size_t workspace_bytes, int device, void* stream);

/* out = cast(epilogue(x @ y)) for fp16 or bf16 x [M,K] and y [K,N] with fp32 accumulation: the same
 * kernels with kind::f16 tensor-core instructions.  Replaces the device kernel of the reference's
 * examples/matmul.py:26-56 (`matmul(x, y, epilogue)`; zero-initialised fp32 accumulator, torch.addmm
 * per K tile, epilogue applied to the fp32 accumulator, cast to promote_types(x, y) on store).  The
 * reference's epilogue is an arbitrary Python closure; here it is one of the three the reference's
 * own checks use (examples/matmul.py:92-117): identity, `acc + bias[column]`, `relu(acc + bias[column])`.
 *   in_dtype: HB200_DT_FP16 or HB200_DT_BF16 (both operands); out_dtype: the same, or HB200_DT_FP32.
 *   x row-major; y row-major (what the reference passes) or column-major; strides in elements.
 *   K % 8 == 0, N % 8 == 0, strides multiples of 8, pointers 16-byte aligned.
 *   bias: NULL, or N floats (fp32; an fp16 / bf16 bias converts exactly); relu: 0 or 1.
 *   cfg_id: a row of the GEMM table built for 16-bit operands (0, 1, 3-10, 14-17), or -1. */
HB200_API int hb200_gemm_16bit(const void* x, const void* y, void* out, int64_t M, int64_t N, int64_t K, int64_t x_rs,
                     int64_t x_cs, int64_t y_rs, int64_t y_cs, int64_t out_rs, int in_dtype, int out_dtype,
                     const float* bias, int relu, int cfg_id, int device, void* stream);

/* Bytes of workspace hb200_fp8_gemm needs for this problem and configuration (0 for most). */
HB200_API size_t hb200_fp8_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int out_dtype, int cfg_id);

/* The configuration the library would choose for this problem when cfg_id == -1. */
HB200_API int hb200_fp8_gemm_select_config(int64_t M, int64_t N, int64_t K, int y_is_colmajor, int out_dtype);

/* out[bh, s, :] = cast( softmax(q k^T * scale) v ), per batch*head slice, non-causal, with the
 * reference's numerics: scores and softmax in fp32 with exp2, P cast to e4m3 UN-normalised
 * before P@V, the row sum taken from the fp32 P, division by the row sum at the end.
 * Replaces the device kernel of examples/fp8_attention.py:22-106 (`fp8_attention_kernel`).
 *   q, k: fp8 [BH, S, D], innermost stride 1, row stride D... given as {bh, s, d} strides.
 *   v: fp8 with LOGICAL shape [BH, D, S] (the reference's "pre-transposed" argument); strides
 *      {bh, d, s}.  Both physical layouts occur: stride_d == 1 (what
 *      preprocess_fp8_attention_inputs really produces, examples/fp8_attention.py:127-132) and
 *      stride_s == 1 (a genuinely contiguous [BH, D, S]).
 *   out: [BH, S, D] with strides {bh, s, d}, d stride 1; FP8 (reference), or BF16 / FP32.
 *   D in {64, 128}; any S >= 1 (every stride except the unit one a multiple of 16 bytes, so a
 *   [BH, D, S] tensor with S contiguous needs S % 16 == 0); scale_log2 = log2(e)/sqrt(D) for the reference's
 *   scale (examples/fp8_attention.py:50-52).
 */
HB200_API int hb200_fp8_attention(const void* q, const void* k, const void* v, void* out, int64_t BH, int64_t S, int64_t D,
                        const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                        const int64_t out_strides[3], float scale_log2, int out_dtype, int cfg_id, int device,
                        void* stream);

/* hb200_fp8_attention with a balanced tile order.  Same computation, arguments and results
 * (bit-identical: each output tile is computed by the same code whichever CTA takes it); the only
 * difference is which CTA computes which 128-row tile.  hb200_fp8_attention hands tiles out in a
 * fixed round-robin, so the kernel ends when the slowest CTA has finished its share; co-resident
 * CTAs run at different speeds and the last round is usually partial.  Here the CTAs draw tiles
 * from a counter in `workspace`, which shortens the kernel by roughly a tenth.  The Helion kernel
 * it replaces is examples/fp8_attention.py:22-106, as for hb200_fp8_attention; the reference has no
 * workspace argument (its grid is one program per batch*head, fp8_attention.py:54).
 *   workspace: HB200_ATTN_WORKSPACE_BYTES of device memory, 16-byte aligned, owned by the caller.
 *      The call clears it on `stream` before the kernel (no allocation); it must not be shared by
 *      calls that can overlap in time (other streams), and may be reused by the next call on the
 *      same stream.
 */
#define HB200_ATTN_WORKSPACE_BYTES 16u
HB200_API int hb200_fp8_attention_ws(const void* q, const void* k, const void* v, void* out, int64_t BH, int64_t S,
                           int64_t D, const int64_t q_strides[3], const int64_t k_strides[3],
                           const int64_t v_strides[3], const int64_t out_strides[3], float scale_log2,
                           int out_dtype, int cfg_id, void* workspace, size_t workspace_bytes, int device,
                           void* stream);

/* hb200_fp8_attention_ws with two extensions the reference's fp8 kernel does not have (its bf16 sibling
 * examples/attention.py:51-58 takes seq_k != seq_q; neither has a mask): k and v may hold S_k keys while q
 * holds S_q rows per slice, and causal != 0 hides key j from query i when j > i + (S_k - S_q) -- the
 * diagonal ends in the bottom-right corner, every query sees at least key 0, S_k >= S_q is required.
 * A hidden score counts as -inf before the row max, like the padding of a ragged key tile; tiles skip
 * the key steps none of their rows can see and are handed out longest first.
 *   q [BH, S_q, D], k [BH, S_k, D], v logical [BH, D, S_k], out [BH, S_q, D]; strides as for
 *   hb200_fp8_attention.
 *   workspace: NULL (fixed tile order) or HB200_ATTN_WORKSPACE_BYTES as for hb200_fp8_attention_ws
 *   (recommended with a mask: the tiles of a slice differ in length). */
HB200_API int hb200_fp8_attention_ex(const void* q, const void* k, const void* v, void* out, int64_t BH, int64_t S_q,
                           int64_t S_k, int64_t D, const int64_t q_strides[3], const int64_t k_strides[3],
                           const int64_t v_strides[3], const int64_t out_strides[3], float scale_log2, int causal,
                           int out_dtype, int cfg_id, void* workspace, size_t workspace_bytes, int device,
                           void* stream);

/* out[bh] = cast(softmax(q[bh] k[bh]^T / sqrt(D)) v[bh]) for fp16 or bf16 q [BH, S_q, D], k and v [BH, S_k, D]
 * (head_dim contiguous; strides {bh, s, d} in elements), out [BH, S_q, D], non-causal.  Replaces the device
 * kernel of the reference's examples/attention.py:29-84 (`attention(q_in, k_in, v_in)`) with its ref-eager
 * numerics: q k^T rounded to the operands' 16-bit type (torch.bmm of 16-bit tensors), times
 * scale_log2 = log2(e)/sqrt(D) rounded to 16 bits again, running max / exp2 / row sum in fp32, P cast to 16
 * bits for P V, fp32 accumulation, division by the row sum, cast to the operands' type.
 *   in_dtype: HB200_DT_FP16 or HB200_DT_BF16; out_dtype: the same, or HB200_DT_FP32.
 *   D in {64, 128}; S_q, S_k >= 1 (any: ragged tiles are zero-filled and masked); strides multiples of 8.
 *   workspace: NULL (fixed tile order) or HB200_ATTN_WORKSPACE_BYTES for the balanced tile order, as for
 *   hb200_fp8_attention_ws. */
HB200_API int hb200_attention_16bit(const void* q, const void* k, const void* v, void* out, int64_t BH, int64_t S_q,
                          int64_t S_k, int64_t D, const int64_t q_strides[3], const int64_t k_strides[3],
                          const int64_t v_strides[3], const int64_t out_strides[3], float scale_log2, int in_dtype,
                          int out_dtype, void* workspace, size_t workspace_bytes, int device, void* stream);

/* q, k, v -> float8_e4m3fn in one launch: the three casts of preprocess_fp8_attention_inputs
 * (examples/fp8_attention.py:125-128; the permute and reshapes of :127-132 only change strides, so
 * the caller does them as views).  Each of q, k, v holds `count` contiguous elements of src_dtype
 * (HB200_DT_FP16, HB200_DT_BF16 or HB200_DT_FP32); q8, k8, v8 receive `count` bytes each, element
 * i of the output being the cast of element i of the input.  The cast is torch's
 * Tensor.to(torch.float8_e4m3fn): round to nearest even; a value that rounds beyond +-448, an
 * infinity or a NaN becomes the NaN pattern (no saturation).  count % 16 == 0; all pointers are
 * 16-byte aligned device pointers. */
HB200_API int hb200_fp8_attention_preprocess(const void* q, const void* k, const void* v, void* q8, void* k8, void* v8,
                                   int64_t count, int src_dtype, int device, void* stream);

/* Split-K FP8 GEMM that allocates nothing: same computation and arguments as hb200_fp8_gemm with a
 * split-K row of the table, but the fp32 partial sums live in a fixed array compiled into the
 * library instead of a caller-provided workspace.  It has no counterpart in the reference; it
 * exists for callers that must not call cudaMalloc / cudaFree (or torch's allocator) around a GEMM:
 * a serving loop whose device memory was handed out completely at start-up, an operator hook that
 * runs inside another runtime which owns the allocator, or a host callback where the device-wide
 * synchronisation that an allocation can cause would stall unrelated streams.
 *   - scratch: HB200_STATIC_SCRATCH_BYTES of device memory per GPU that loads the library, held
 *     until the process exits; a call needs splits * M * N * 4 bytes of it and is rejected with
 *     HB200_ERR_WORKSPACE when that exceeds the array (use hb200_fp8_gemm with a workspace then);
 *   - splits: 2..8 (the K range is cut into that many parts; every part of every output element is
 *     written before it is read, so the array needs no clearing between calls);
 *   - the first call on a device looks up the array's device address, and the first call for each
 *     (out_dtype, layout of y) on a device raises that kernel instance's shared-memory limit and lets
 *     the driver load it (no allocation by this library); make one warm-up call per (out_dtype, layout)
 *     you will use before starting any stream capture or entering a section that must not allocate;
 *   - a device-side wait that runs out (hb200_read_status) is reported for this entry point only once
 *     the device's context exists, i.e. after any other entry point of this library has run on the
 *     device; before that such a wait still ends the kernel early, but nothing records it, because
 *     creating the context allocates;
 *   - all calls on a device share the one array: two calls whose kernels can overlap on the GPU
 *     (different streams, no dependency between them) race on it and give wrong results -- order them;
 *   - calls neither cudaMalloc nor cudaFree nor any allocating library routine; launches two kernels
 *     (partial products, then the ordered sum and conversion) on the given stream.
 * x, y, out, sizes, strides, out_dtype and the return codes are those of hb200_fp8_gemm (plus
 * HB200_ERR_CUDA when `device` does not exist or cannot be made current). */
#define HB200_STATIC_SCRATCH_BYTES (4u << 20)
HB200_API int hb200_fp8_gemm_splitk_static(const void* x, const void* y, void* out, int64_t M, int64_t N, int64_t K,
                                           int64_t x_rs, int64_t x_cs, int64_t y_rs, int64_t y_cs, int64_t out_rs,
                                           int out_dtype, int splits, int device, void* stream);

/* Tile-config table introspection (the table replaces Helion's autotuner,
 * helion/autotuner/differential_evolution.py:20-101). */
HB200_API int hb200_num_configs(int op);
/* Writes a NUL-terminated description into buf (at most buf_len bytes); returns its length. */
HB200_API int hb200_describe_config(int op, int cfg_id, char* buf, int buf_len);

/* Device-side status word of the bounded waits: returns 0 if no wait ran out on this device
 * since the last reset, else HB200_ERR_TIMEOUT with *site = (wait site << 16) | block index.
 * Reads mapped host memory; does not synchronise.  hb200_reset_status clears it. */
HB200_API int hb200_read_status(int device, uint32_t* site);
HB200_API int hb200_reset_status(int device);

/* Self-test of the bounded-wait scheme: launches one small CTA that waits on a barrier nothing will
 * complete; after limit_ms (1..1000) the wait gives up, the kernel returns normally and the status
 * word reports HB200_ERR_TIMEOUT with wait site 40.  The context stays usable.  (No counterpart in the
 * reference: Helion's only timeout handling is around Triton compilation,
 * helion/autotuner/base_search.py:155-200.) */
HB200_API int hb200_debug_wait_selftest(int device, int limit_ms, void* stream);

/* Softmax-only ceiling of the attention kernels: runs nothing but the per-score work of
 * examples/fp8_attention.py:74-94 (row max, exp2, row sum, cast of P to e4m3, with the scores read from and
 * P written to tensor memory) for `steps` 128x128 steps per softmax warpgroup, on every SM.
 *   wgs: softmax warpgroups per CTA (1 or 2); ctas_per_sm: 1 or 2 (2 only with wgs = 1);
 *   poly_of8: of every 8 pairs of exponentials, how many run as a polynomial on the FMA pipes (0, 2, 3, 4);
 *   mode: 0 full step, 1 without the row max, 2 without the exponentials, 3 tensor-memory traffic only;
 *      16 + mask (wgs = 2, poly_of8 = 0): the full step next to other roles of an attention kernel, mask bit
 *      1 = four warps polling a barrier, 2 = one thread issuing tensor-core instructions back to back,
 *      4 = four warps rescaling tensor memory, 8 = the softmax threads' own barrier traffic; masks 1, 2, 4, 8, 15;
 *   cycles: device pointer to num_sms * ctas_per_sm uint64: SM clocks the slowest warp of each CTA took.
 * Cycles per step per SM = cycles / (steps * wgs * ctas_per_sm): the floor for any pipeline built around this
 * arithmetic.  A measurement aid; the reference has no counterpart. */
HB200_API int hb200_debug_softmax_ceiling(int wgs, int ctas_per_sm, int poly_of8, int mode, int steps, void* cycles,
                                          int device, void* stream);

/* Number of SMs the persistent kernels size their grids with (cudaDevAttrMultiProcessorCount;
 * the role of helion/runtime/__init__.py:41-52 `get_num_sm`). */
HB200_API int hb200_num_sms(int device);

/* Thread-local text of the last error returned on this thread. */
HB200_API const char* hb200_last_error(void);

HB200_API int hb200_version(void);

#ifdef __cplusplus
}
#endif

#endif /* HELION_B200_H */
