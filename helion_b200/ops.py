"""Host-side operators: torch tensors in, one C-ABI launch, torch tensor out.

These functions do what the generated host functions of the reference do around their Triton
launch (allocate the output with ``torch.empty`` on the inputs' device, launch on the current
stream, return the output; pytorch-labs/helion ``examples/fp8_gemm.py:42-57``,
``examples/fp8_attention.py:43-106``).  torch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from . import _lib

_OUT_DT = {
    torch.float16: _lib.DT_FP16,
    torch.bfloat16: _lib.DT_BF16,
    torch.float32: _lib.DT_FP32,
    torch.float8_e4m3fn: _lib.DT_E4M3,
}


def _require_cuda(*tensors: torch.Tensor) -> int:
    dev = tensors[0].device
    if dev.type != "cuda":
        raise RuntimeError(
            f"helion_b200 runs on CUDA (sm_100a) tensors only, got a tensor on {dev}; there is no CPU fallback"
        )
    for t in tensors[1:]:
        if t.device != dev:
            raise RuntimeError(f"all tensors must be on the same device, got {dev} and {t.device}")
    return dev.index if dev.index is not None else torch.cuda.current_device()


def _stream_ptr(device_index: int) -> int:
    return torch.cuda.current_stream(device_index).cuda_stream


def _round_up(v: int, mult: int) -> int:
    return (v + mult - 1) // mult * mult


def _pad_gemm_operands(x: torch.Tensor, y: torch.Tensor, kp: int, np_: int):
    """Zero-padded copies of ``x [M,K]`` -> ``[M,kp]`` and ``y [K,N]`` -> ``[kp,np_]`` (y keeps its layout).

    The C ABI takes TMA-legal operands only (16-byte aligned rows); the reference accepts any M, N, K
    (masked tiles, helion/_compiler/inductor_lowering.py:825-831).  Zero rows / columns add nothing to
    the products, so the odd shapes go through the same kernels on padded device copies and the
    caller gets the ``[:, :N]`` part back.
    """
    m, k = x.shape
    n = y.shape[1]
    if kp != k:
        xp = x.new_zeros((m, kp))
        xp[:, :k].copy_(x)
        x = xp
    if kp != k or np_ != n:
        if y.stride(0) == 1 and y.stride(1) != 1:  # column-major: pad the [N, K] storage
            yt = y.new_zeros((np_, kp))
            yt[:n, :k].copy_(y.t())
            y = yt.t()
        else:
            yp = y.new_zeros((kp, np_))
            yp[:k, :n].copy_(y)
            y = yp
    return x, y


def _pad_vector(v: Optional[torch.Tensor], n: int, np_: int, fill: float) -> Optional[torch.Tensor]:
    if v is None or v.numel() != n or np_ == n:
        return v
    out = v.new_full((np_,), fill)
    out[:n].copy_(v.reshape(n))
    return out


def fp8_gemm(
    x: torch.Tensor,
    y: torch.Tensor,
    *,
    out_dtype: torch.dtype = torch.float16,
    config: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
    scale_a: Optional[torch.Tensor] = None,
    scale_b: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """``out = (x @ y).to(out_dtype)`` for float8_e4m3fn ``x [M,K]`` and ``y [K,N]``, fp32 accumulation.

    Same contract as the reference's ``fp8_gemm(x, y)`` (examples/fp8_gemm.py:29-57): fp16 output by
    default.  ``y`` may be row-major or column-major (a transposed view); ``x`` must be row-major.
    ``out_dtype`` (fp16 / bf16 / fp32), ``config`` (tile-config id, None = table choice) and ``out``
    are keyword-only extensions.

    ``scale_a`` / ``scale_b`` (fp32 CUDA tensors, both or neither) give
    ``out = (((x @ y) * scale_a) * scale_b).to(out_dtype)`` with the shapes ``torch._scaled_mm``
    accepts: one element each (per-tensor), or ``[M, 1]`` / ``[M]`` and ``[1, N]`` / ``[N]``
    (row-wise).  The reference fixes both at 1.0 (examples/fp8_gemm.py:74-75).
    """
    if x.dtype != torch.float8_e4m3fn or y.dtype != torch.float8_e4m3fn:
        raise TypeError(f"fp8_gemm expects float8_e4m3fn inputs, got {x.dtype} and {y.dtype}")
    if x.dim() != 2 or y.dim() != 2:
        raise ValueError(f"fp8_gemm expects 2-D inputs, got {tuple(x.shape)} and {tuple(y.shape)}")
    m, k = x.shape
    k2, n = y.shape
    assert k == k2, f"size mismatch {k} != {k2}"  # same check and text as examples/fp8_gemm.py:44
    if out_dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise TypeError(f"fp8_gemm out_dtype must be float16, bfloat16 or float32, got {out_dtype}")
    dev = _require_cuda(x, y)
    if x.stride(1) != 1:
        x = x.contiguous()
    if y.stride(0) != 1 and y.stride(1) != 1:
        y = y.contiguous()
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    else:
        if out.dtype != out_dtype or tuple(out.shape) != (m, n) or out.stride(1) != 1 or out.device != x.device:
            raise ValueError("fp8_gemm: `out` must be a row-major [M, N] tensor of out_dtype on the inputs' device")
    if m == 0 or n == 0:
        return out
    if k == 0:
        return out.zero_()
    kp, np_ = _round_up(k, 16), _round_up(n, 16)
    if kp != k or np_ != n:  # odd K or N: same kernels on zero-padded copies (see _pad_gemm_operands)
        xp, yp = _pad_gemm_operands(x, y, kp, np_)
        if scale_b is not None and scale_b.numel() != 1:
            _check_scales(scale_a, scale_b, m, n, x.device)
            scale_b = _pad_vector(scale_b, n, np_, 1.0)
        res = fp8_gemm(xp, yp, out_dtype=out_dtype, config=config, scale_a=scale_a, scale_b=scale_b)
        out.copy_(res[:, :n])
        return out
    if x.stride(0) % 16 != 0:
        x = x.contiguous()
    lib = _lib.load()
    cfg = -1 if config is None else int(config)
    # Split-K rows of the tile table need scratch for their fp32 partial sums; like `out` it comes
    # from torch's caching allocator and is only used by this call's two kernels on this stream.
    ws_bytes = lib.hb200_fp8_gemm_workspace_bytes(m, n, k, _OUT_DT[out_dtype], cfg)
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device) if ws_bytes else None
    ws_ptr = workspace.data_ptr() if workspace is not None else None
    if scale_a is None and scale_b is None:
        code = lib.hb200_fp8_gemm(
            x.data_ptr(), y.data_ptr(), out.data_ptr(), m, n, k,
            x.stride(0), x.stride(1), y.stride(0), y.stride(1), out.stride(0),
            _OUT_DT[out_dtype], cfg, ws_ptr, ws_bytes, dev, _stream_ptr(dev),
        )
    else:
        sa, sb, mode = _check_scales(scale_a, scale_b, m, n, x.device)
        code = lib.hb200_fp8_gemm_scaled(
            x.data_ptr(), y.data_ptr(), out.data_ptr(), m, n, k,
            x.stride(0), x.stride(1), y.stride(0), y.stride(1), out.stride(0),
            _OUT_DT[out_dtype], sa.data_ptr(), sb.data_ptr(), mode, cfg, ws_ptr, ws_bytes, dev, _stream_ptr(dev),
        )
    _lib.raise_for(code, "fp8_gemm")
    return out


def _check_scales(scale_a, scale_b, m: int, n: int, device):
    """Validate the two scale tensors; returns contiguous fp32 tensors and the C-ABI scale mode."""
    if scale_a is None or scale_b is None:
        raise ValueError("fp8_gemm: pass both scale_a and scale_b or neither")
    for name, t in (("scale_a", scale_a), ("scale_b", scale_b)):
        if not isinstance(t, torch.Tensor) or t.dtype != torch.float32:
            raise TypeError(f"fp8_gemm: {name} must be a float32 tensor")
        if t.device != device:
            raise ValueError(f"fp8_gemm: {name} must live on the inputs' device")
    if scale_a.numel() == 1 and scale_b.numel() == 1:
        return scale_a.reshape(1).contiguous(), scale_b.reshape(1).contiguous(), _lib.SCALE_TENSOR
    if tuple(scale_a.shape) in ((m, 1), (m,)) and tuple(scale_b.shape) in ((1, n), (n,)):
        return scale_a.reshape(m).contiguous(), scale_b.reshape(n).contiguous(), _lib.SCALE_ROWWISE
    raise ValueError(
        f"fp8_gemm: scales must be one element each, or [M,1]/[M] and [1,N]/[N]; got {tuple(scale_a.shape)} and "
        f"{tuple(scale_b.shape)} for M={m}, N={n}"
    )


def _kernel_head_dim(d: int, what: str) -> int:
    """The head_dim the kernels run a logical head_dim at: 64 or 128 (zero-padded columns in between)."""
    if d < 1 or d > 128:
        raise ValueError(f"{what}: head_dim must be in [1, 128] (kernels exist for 64 and 128; smaller ones are zero-padded), got {d}")
    return 64 if d <= 64 else 128


def _pad_last(t: torch.Tensor, dp: int) -> torch.Tensor:
    out = t.new_zeros((*t.shape[:-1], dp))
    out[..., : t.shape[-1]].copy_(t)
    return out


def fp8_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    batch: int,
    heads: int,
    *,
    out_dtype: torch.dtype = torch.float8_e4m3fn,
    config: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
    balanced: Optional[bool] = None,
    causal: bool = False,
) -> torch.Tensor:
    """FP8 attention forward with the reference's numerics (non-causal unless ``causal=True``).

    Same contract as the reference's ``fp8_attention_kernel(q, k, v, batch, heads)``
    (examples/fp8_attention.py:22-106): ``q``, ``k`` are ``[batch*heads, seq, dim]`` e4m3, ``v`` is
    the "pre-transposed" ``[batch*heads, dim, seq]`` e4m3 tensor (either physical layout), the
    result is ``[batch, heads, seq, dim]`` e4m3.  ``out_dtype`` (e4m3 / bf16 / fp32), ``config``,
    ``out`` and ``balanced`` (see :func:`attention_into`) are keyword-only extensions.  Two more go
    beyond the reference's kernel: ``k`` / ``v`` may hold a different number of keys than ``q`` has
    rows, and ``causal=True`` hides key j from query i when ``j > i + (seq_k - seq_q)``.
    """
    for name, t in (("q", q), ("k", k), ("v", v)):
        if t.dtype != torch.float8_e4m3fn:
            raise TypeError(f"fp8_attention expects float8_e4m3fn inputs, {name} is {t.dtype}")
        if t.dim() != 3:
            raise ValueError(f"fp8_attention expects 3-D inputs, {name} has shape {tuple(t.shape)}")
    bh, s, d = q.shape
    sk = k.shape[1]
    if tuple(k.shape) != (bh, sk, d) or tuple(v.shape) != (bh, d, sk):
        raise ValueError(
            f"fp8_attention shape mismatch: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)} "
            "(expected [BH,S,D], [BH,S,D], [BH,D,S])"
        )
    if bh != batch * heads:
        raise ValueError(f"fp8_attention: q.size(0)={bh} != batch*heads={batch * heads}")
    if out_dtype not in (torch.float8_e4m3fn, torch.bfloat16, torch.float32):
        raise TypeError(f"fp8_attention out_dtype must be float8_e4m3fn, bfloat16 or float32, got {out_dtype}")
    dev = _require_cuda(q, k, v)
    dp = _kernel_head_dim(d, "fp8_attention")
    if dp != d and bh > 0 and s > 0:
        # The kernels exist for head_dim 64 and 128; the reference pads any head_dim to a power of two
        # and masks (examples/fp8_attention.py:31-33).  Zero columns add nothing to q k^T and give
        # zero output columns, so the same kernel runs on padded copies with the scale of the real D.
        qp, kp = (_pad_last(t, dp) for t in (q, k))
        vp = _pad_last(v.transpose(1, 2), dp).transpose(1, 2)
        res = torch.empty((batch, heads, s, dp), dtype=out_dtype, device=q.device)
        attention_into(qp, kp, vp, res.view(bh, s, dp), config=config, balanced=balanced, causal=causal, head_dim=d)
        if out is None:
            return res[..., :d].contiguous()
        if out.dtype != out_dtype or tuple(out.shape) != (batch, heads, s, d):
            raise ValueError("fp8_attention: `out` must be a [batch, heads, seq, dim] tensor of out_dtype")
        out.copy_(res[..., :d])
        return out
    if q.stride(2) != 1:
        q = q.contiguous()
    if k.stride(2) != 1:
        k = k.contiguous()
    if v.stride(1) != 1 and v.stride(2) != 1:
        v = v.contiguous()
    if v.stride(2) == 1 and v.stride(1) != 1 and (v.stride(1) % 16 != 0 or v.stride(0) % 16 != 0):
        # keys contiguous with rows that are not 16-byte aligned (seq_k % 16 != 0): take the other
        # physical layout of the same logical tensor (head_dim contiguous), which any seq_k fits
        v = v.transpose(1, 2).contiguous().transpose(1, 2)
    if out is None:
        out = torch.empty((batch, heads, s, d), dtype=out_dtype, device=q.device)
    elif out.dtype != out_dtype or tuple(out.shape) != (batch, heads, s, d) or not out.is_contiguous():
        raise ValueError("fp8_attention: `out` must be a contiguous [batch, heads, seq, dim] tensor of out_dtype")
    if bh == 0 or s == 0:
        return out
    attention_into(q, k, v, out.view(bh, s, d), config=config, balanced=balanced, causal=causal)
    return out


def attention_into(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out3: torch.Tensor, *, config: Optional[int] = None,
    balanced: Optional[bool] = None, causal: bool = False, head_dim: Optional[int] = None,
) -> None:
    """Launch the attention kernel on ``[BH,S,D]`` / ``[BH,D,S]`` tensors, writing ``out3 [BH,S,D]``.

    The batch*head slices are independent, so a shard of them (a slice along dim 0 of every
    tensor) is a valid call; the multi-GPU driver uses exactly that.

    ``balanced=True`` lets the CTAs draw tiles from a counter in a 16-byte workspace that this
    wrapper takes from torch's caching allocator per call (stream-ordered, so overlapping calls on
    other streams never share it); ``balanced=False`` is the fixed round-robin of
    ``hb200_fp8_attention``.  Results are bit-identical either way.  The default (``None``) uses the
    counter from 2048 keys up: measured on B200 it shortens the kernel by 4-10 % at seq 4096 and
    gains nothing at seq 1024, where clearing the counter costs what the better balance saves.
    """
    bh, s, d = q.shape
    dev = _require_cuda(q, k, v, out3)
    # The kernel scales by log2(e)/sqrt(D) and uses exp2, like examples/fp8_attention.py:50-52
    # (head_dim: the logical D when the tensors carry zero-padded columns).
    scale_log2 = (1.0 / math.sqrt(float(d if head_dim is None else head_dim))) * 1.44269504
    arr = ctypes.c_int64 * 3
    lib = _lib.load()
    cfg = -1 if config is None else int(config)
    sk = k.shape[1]
    if balanced is None:
        balanced = sk >= 2048 or (causal and sk >= 512)  # masked tiles differ in length: balance earlier
    if causal or sk != s:
        ws = torch.empty(_lib.ATTN_WORKSPACE_BYTES, dtype=torch.uint8, device=q.device) if balanced else None
        code = lib.hb200_fp8_attention_ex(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out3.data_ptr(), bh, s, sk, d,
            arr(*q.stride()), arr(*k.stride()), arr(*v.stride()), arr(*out3.stride()),
            scale_log2, int(bool(causal)), _OUT_DT[out3.dtype], cfg,
            ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, dev, _stream_ptr(dev),
        )
    elif balanced:
        ws = torch.empty(_lib.ATTN_WORKSPACE_BYTES, dtype=torch.uint8, device=q.device)
        code = lib.hb200_fp8_attention_ws(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out3.data_ptr(), bh, s, d,
            arr(*q.stride()), arr(*k.stride()), arr(*v.stride()), arr(*out3.stride()),
            scale_log2, _OUT_DT[out3.dtype], cfg, ws.data_ptr(), ws.numel(), dev, _stream_ptr(dev),
        )
    else:
        code = lib.hb200_fp8_attention(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out3.data_ptr(), bh, s, d,
            arr(*q.stride()), arr(*k.stride()), arr(*v.stride()), arr(*out3.stride()),
            scale_log2, _OUT_DT[out3.dtype], cfg, dev, _stream_ptr(dev),
        )
    _lib.raise_for(code, "fp8_attention")


def preprocess_fp8_attention_inputs(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``[B,H,S,D]`` fp16 / bf16 / fp32 tensors -> e4m3 ``q [BH,S,D]``, ``k [BH,S,D]``, ``v [BH,D,S]``.

    Same results, shapes and strides as the reference's function of this name
    (examples/fp8_attention.py:110-133), whose three ``.to(float8_e4m3fn)`` casts run here as one
    CUDA kernel; ``v`` comes back as the reference's pre-transposed view of memory that is physically
    ``[BH, S, D]``.  Inputs that are already e4m3 are only reshaped.
    """
    if q.dim() != 4 or q.shape != k.shape or q.shape != v.shape:
        raise ValueError(f"expected three [B,H,S,D] tensors, got {tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    batch, heads, seq, dim = q.shape
    bh = batch * heads
    if q.dtype == k.dtype == v.dtype == torch.float8_e4m3fn:
        q8, k8, v8 = q.contiguous(), k.contiguous(), v.contiguous()
    else:
        if not (q.dtype == k.dtype == v.dtype) or q.dtype not in _OUT_DT or q.dtype == torch.float8_e4m3fn:
            raise TypeError(f"q, k, v must share one dtype of float16, bfloat16, float32; got {q.dtype}, {k.dtype}, {v.dtype}")
        dev = _require_cuda(q, k, v)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        q8, k8, v8 = (torch.empty(t.shape, dtype=torch.float8_e4m3fn, device=t.device) for t in (q, k, v))
        count = q.numel()
        if count:
            code = _lib.load().hb200_fp8_attention_preprocess(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), q8.data_ptr(), k8.data_ptr(), v8.data_ptr(), count,
                _OUT_DT[q.dtype], dev, _stream_ptr(dev),
            )
            _lib.raise_for(code, "preprocess_fp8_attention_inputs")
    return q8.reshape(bh, seq, dim), k8.reshape(bh, seq, dim), v8.reshape(bh, seq, dim).permute(0, 2, 1)


def matmul(
    x: torch.Tensor,
    y: torch.Tensor,
    *,
    bias: Optional[torch.Tensor] = None,
    relu: bool = False,
    out_dtype: Optional[torch.dtype] = None,
    config: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """``out = epilogue(x @ y).to(out_dtype)`` for fp16 or bf16 ``x [M,K]``, ``y [K,N]``, fp32 accumulation.

    The computation of the reference's ``matmul(x, y, epilogue)`` (examples/matmul.py:26-56) with the
    epilogues its own checks use: identity, ``acc + bias[column]`` (``bias`` of N elements), and
    ``relu(acc + bias[column])``.  The result has the operands' dtype (the reference's
    ``promote_types``) unless ``out_dtype=torch.float32``.
    """
    if x.dtype != y.dtype or x.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError(f"matmul expects two float16 or two bfloat16 operands, got {x.dtype} and {y.dtype}")
    if x.dim() != 2 or y.dim() != 2:
        raise ValueError(f"matmul expects 2-D inputs, got {tuple(x.shape)} and {tuple(y.shape)}")
    m, k = x.shape
    k2, n = y.shape
    assert k == k2, f"size mismatch {k} != {k2}"  # same check and text as examples/matmul.py:47
    out_dtype = x.dtype if out_dtype is None else out_dtype
    if out_dtype not in (x.dtype, torch.float32):
        raise TypeError(f"matmul out_dtype must be {x.dtype} or float32, got {out_dtype}")
    dev = _require_cuda(x, y)
    if x.stride(1) != 1:
        x = x.contiguous()
    if y.stride(0) != 1 and y.stride(1) != 1:
        y = y.contiguous()
    bias32 = None
    if bias is not None:
        if bias.dim() != 1 or bias.shape[0] != n or bias.device != x.device:
            raise ValueError(f"matmul: bias must be a vector of N={n} elements on the inputs' device")
        bias32 = bias.to(torch.float32).contiguous()
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    elif out.dtype != out_dtype or tuple(out.shape) != (m, n) or out.stride(1) != 1 or out.device != x.device:
        raise ValueError("matmul: `out` must be a row-major [M, N] tensor of out_dtype on the inputs' device")
    if m == 0 or n == 0:
        return out
    if k == 0:
        out.zero_()
        if bias32 is not None:
            out += bias32.to(out_dtype)
        return out.relu_() if relu else out
    kp, np_ = _round_up(k, 8), _round_up(n, 8)
    if kp != k or np_ != n:  # odd K or N: same kernels on zero-padded copies (see _pad_gemm_operands)
        xp, yp = _pad_gemm_operands(x, y, kp, np_)
        res = matmul(xp, yp, bias=_pad_vector(bias32, n, np_, 0.0), relu=relu, out_dtype=out_dtype, config=config)
        out.copy_(res[:, :n])
        return out
    if x.stride(0) % 8 != 0:
        x = x.contiguous()
    code = _lib.load().hb200_gemm_16bit(
        x.data_ptr(), y.data_ptr(), out.data_ptr(), m, n, k,
        x.stride(0), x.stride(1), y.stride(0), y.stride(1), out.stride(0),
        _OUT_DT[x.dtype], _OUT_DT[out_dtype], bias32.data_ptr() if bias32 is not None else None, int(bool(relu)),
        -1 if config is None else int(config), dev, _stream_ptr(dev),
    )
    _lib.raise_for(code, "matmul")
    return out


def attention(
    q_in: torch.Tensor,
    k_in: torch.Tensor,
    v_in: torch.Tensor,
    *,
    out_dtype: Optional[torch.dtype] = None,
    balanced: Optional[bool] = None,
) -> torch.Tensor:
    """``softmax(q k^T / sqrt(D)) v`` for fp16 or bf16 ``q [..., Sq, D]``, ``k``, ``v [..., Sk, D]``.

    Same contract as the reference's ``attention(q_in, k_in, v_in)`` (examples/attention.py:29-84): leading
    dimensions are flattened into independent slices, the result has ``q_in``'s shape and dtype (fp32 with
    ``out_dtype=torch.float32``), and the intermediate roundings are those of the reference's 16-bit tensors.
    """
    if not (q_in.dtype == k_in.dtype == v_in.dtype) or q_in.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError(f"attention expects three float16 or three bfloat16 tensors, got {q_in.dtype}, {k_in.dtype}, {v_in.dtype}")
    if q_in.dim() < 2 or k_in.dim() != q_in.dim() or v_in.dim() != q_in.dim():
        raise ValueError("attention expects q [..., Sq, D], k [..., Sk, D], v [..., Sk, D]")
    m_dim, d = q_in.shape[-2], q_in.shape[-1]
    n_dim = k_in.shape[-2]
    assert n_dim == v_in.size(-2)  # examples/attention.py:52
    assert d == k_in.size(-1) == v_in.size(-1)  # examples/attention.py:54
    if k_in.shape[:-2] != q_in.shape[:-2] or v_in.shape[:-2] != q_in.shape[:-2]:
        raise ValueError("attention: q, k and v must agree in their leading (batch) dimensions")
    out_dtype = q_in.dtype if out_dtype is None else out_dtype
    if out_dtype not in (q_in.dtype, torch.float32):
        raise TypeError(f"attention out_dtype must be {q_in.dtype} or float32, got {out_dtype}")
    dev = _require_cuda(q_in, k_in, v_in)
    bh = math.prod(q_in.shape[:-2])  # explicit: reshape(-1, ...) is ambiguous for tensors without elements
    q, k, v = (t.reshape(bh, t.shape[-2], d) for t in (q_in, k_in, v_in))
    if bh == 0 or m_dim == 0:
        return torch.empty(q_in.shape, dtype=out_dtype, device=q_in.device)
    if n_dim == 0:
        raise ValueError("attention: k and v hold no keys")
    scale_log2 = (1.0 / math.sqrt(float(d))) * 1.44269504  # qk_scale of examples/attention.py:60-61
    d_logical, d = d, _kernel_head_dim(d, "attention")
    if d != d_logical:  # zero-padded columns, the scale of the real head_dim (see fp8_attention)
        q, k, v = (_pad_last(t, d) for t in (q, k, v))
    q, k, v = (t if t.stride(2) == 1 and t.stride(1) % 8 == 0 and t.stride(0) % 8 == 0 else t.contiguous() for t in (q, k, v))
    out = torch.empty((bh, m_dim, d), dtype=out_dtype, device=q.device)
    if balanced is None:
        balanced = n_dim >= 2048
    ws = torch.empty(_lib.ATTN_WORKSPACE_BYTES, dtype=torch.uint8, device=q.device) if balanced else None
    arr = ctypes.c_int64 * 3
    code = _lib.load().hb200_attention_16bit(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), bh, m_dim, n_dim, d,
        arr(*q.stride()), arr(*k.stride()), arr(*v.stride()), arr(*out.stride()), scale_log2,
        _OUT_DT[q_in.dtype], _OUT_DT[out_dtype], ws.data_ptr() if ws is not None else None,
        ws.numel() if ws is not None else 0, dev, _stream_ptr(dev),
    )
    _lib.raise_for(code, "attention")
    if d != d_logical:
        out = out[..., :d_logical].contiguous()
    return out.view(q_in.shape)
