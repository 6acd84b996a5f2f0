"""FP8 attention behind the entry points of pytorch-labs/helion's ``examples/fp8_attention.py``.

Same module-level names and positional signatures as the reference module
(benchmarks/run.py:94-98 of the reference imports ``examples.fp8_attention`` and calls
``fp8_attention_tritonbench``).  The kernel body is the hand-written sm_100a CUDA kernel of
``helion_b200``.
"""
from __future__ import annotations

import math
from typing import Callable

import torch

from helion_b200 import _lib
from helion_b200 import ops as _ops
from helion_b200.kernel import DropInKernel


def _fp8_attention_spec(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, batch: int, heads: int
) -> torch.Tensor:
    """Per batch*head: softmax(q k^T / sqrt(D)) v with e4m3 operands, fp32 online softmax (exp2),
    P cast to e4m3 un-normalised before P@V, result / row-sum cast to e4m3 [batch, heads, seq, dim]."""
    raise NotImplementedError("specification only; the CUDA kernel implements it")


_fp8_attention_spec.__name__ = "fp8_attention_kernel"


def _launch(args, cfg_id, **kwargs):
    q, k, v, batch, heads = args
    return _ops.fp8_attention(q, k, v, batch, heads, config=cfg_id, **kwargs)


def _select(args):
    return 0


def _describe(args, cfg_id):
    return _lib.describe_config(_lib.OP_ATTENTION, 0 if cfg_id is None else cfg_id)


#: Drop-in for the reference's ``fp8_attention_kernel`` (examples/fp8_attention.py:22-106):
#: ``fp8_attention_kernel(q [BH,S,D], k [BH,S,D], v [BH,D,S], batch, heads) -> e4m3 [B,H,S,D]``.
fp8_attention_kernel = DropInKernel(_fp8_attention_spec, _launch, _select, _describe, static_shapes=True)


def preprocess_fp8_attention_inputs(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """[B,H,S,D] float tensors -> e4m3 q [BH,S,D], k [BH,S,D], v [BH,D,S] (examples/fp8_attention.py:110-133).

    As in the reference, ``v.permute(...).to(e4m3)`` keeps the strides of the permuted view, so
    the returned ``v`` is a [BH, D, S] view of memory that is physically [BH, S, D]; the CUDA
    kernel reads either layout without a copy.
    """
    if q.is_cuda and q.dtype == k.dtype == v.dtype and q.dtype in (torch.float16, torch.bfloat16, torch.float32):
        # the three casts as one CUDA kernel (hb200_fp8_attention_preprocess)
        return _ops.preprocess_fp8_attention_inputs(q, k, v)
    q_fp8 = q.to(torch.float8_e4m3fn)
    k_fp8 = k.to(torch.float8_e4m3fn)
    v_fp8 = v.permute(0, 1, 3, 2).to(torch.float8_e4m3fn)
    batch, heads, seq_len, head_dim = q.shape
    return (
        q_fp8.reshape(batch * heads, seq_len, head_dim),
        k_fp8.reshape(batch * heads, seq_len, head_dim),
        v_fp8.reshape(batch * heads, head_dim, seq_len),
    )


def fp8_attention_tritonbench(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> Callable[[], torch.Tensor]:
    """Preprocess once, return the timed closure (examples/fp8_attention.py:137-154)."""
    batch, heads, seq_len, head_dim = q.shape
    q_fp8, k_fp8, v_fp8 = preprocess_fp8_attention_inputs(q, k, v)
    return lambda: fp8_attention_kernel(q_fp8, k_fp8, v_fp8, batch, heads)


def _fp8_attention_pytorch_impl(q_fp8, k_fp8, v_fp8, batch, heads, seq_len, head_dim) -> torch.Tensor:
    """The reference's loose PyTorch baseline (examples/fp8_attention.py:158-238): per-head
    ``_scaled_mm`` with P normalised BEFORE the e4m3 cast, hence only comparable at atol 0.1-0.2."""
    sm_scale = 1.0 / math.sqrt(float(head_dim))
    one = torch.tensor(1.0, device=q_fp8.device)
    outs = []
    for i in range(batch * heads):
        kt = k_fp8[i].contiguous().t()
        qk = torch._scaled_mm(q_fp8[i], kt, one, one, use_fast_accum=False, out_dtype=torch.float32)
        qk_max = torch.amax(qk, dim=-1, keepdim=True)
        p = torch.exp2((qk * sm_scale - qk_max * sm_scale) * 1.44269504)
        p_fp8 = (p / p.sum(dim=-1, keepdim=True)).to(torch.float8_e4m3fn)
        vt = v_fp8[i].contiguous().t()
        o = torch._scaled_mm(p_fp8, vt, one, one, use_fast_accum=False, out_dtype=torch.float32)
        outs.append(o.to(torch.float8_e4m3fn))
    return torch.stack(outs, dim=0).reshape(batch, heads, seq_len, head_dim)


def fp8_attention_pytorch(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> Callable[[], torch.Tensor]:
    """Baseline closure with the reference's signature (examples/fp8_attention.py:242-256)."""
    batch, heads, seq_len, head_dim = q.shape
    q_fp8, k_fp8, v_fp8 = preprocess_fp8_attention_inputs(q, k, v)
    return lambda: _fp8_attention_pytorch_impl(q_fp8, k_fp8, v_fp8, batch, heads, seq_len, head_dim)


def check(batch: int, heads: int, seq_len: int, head_dim: int) -> None:
    """Kernel vs the loose PyTorch baseline with the reference's tolerances (atol = rtol = 0.1,
    examples/fp8_attention.py:260-284)."""
    torch.manual_seed(42)
    q = torch.randn(batch, heads, seq_len, head_dim, dtype=torch.float16, device="cuda")
    k = torch.randn(batch, heads, seq_len, head_dim, dtype=torch.float16, device="cuda")
    v = torch.randn(batch, heads, seq_len, head_dim, dtype=torch.float16, device="cuda")
    out = fp8_attention_tritonbench(q, k, v)()
    expected = fp8_attention_pytorch(q, k, v)()
    torch.testing.assert_close(out.float(), expected.float(), atol=0.1, rtol=0.1)
    print(f"fp8_attention B{batch} H{heads} S{seq_len} D{head_dim}: matches the PyTorch baseline")


def main() -> None:
    check(1, 2, 128, 64)
    check(2, 4, 256, 64)
    check(4, 8, 512, 128)


if __name__ == "__main__":
    main()
