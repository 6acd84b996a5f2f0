"""fp16 / bf16 attention behind the entry points of pytorch-labs/helion's ``examples/attention.py``.

Same module-level names and positional signatures as the reference module (``attention(q_in, k_in, v_in)``,
``attention_dynamic``, ``test``, ``main``; benchmarks/run.py:78-85 of the reference imports
``examples.attention`` and calls ``attention``).  The kernel body is the hand-written sm_100a CUDA kernel
of ``helion_b200`` (kind::f16 tensor-core instructions).  Only the 16-bit dtypes are built: the
reference's default ``dtype=torch.float32`` of ``test`` raises ``TypeError`` here instead of falling back.
"""
from __future__ import annotations

import math

import torch

from helion_b200 import ops as _ops
from helion_b200.kernel import DropInKernel


def _attention_spec(q_in: torch.Tensor, k_in: torch.Tensor, v_in: torch.Tensor) -> torch.Tensor:
    """softmax(q k^T / sqrt(head_dim)) v over the last two dimensions; leading dimensions are batch."""
    raise NotImplementedError("specification only; the CUDA kernel implements it")


_attention_spec.__name__ = "attention"


def _launch(args, cfg_id, **kwargs):
    q, k, v = args
    return _ops.attention(q, k, v, **kwargs)


def _select(args):
    return None  # one kernel per head_dim and dtype: nothing to choose


def _describe(args, cfg_id):
    return "attention16_kernel: 128 query rows x 64-key steps, two CTAs per SM, kind::f16 MMAs, fp32 online softmax"


#: Drop-in for the reference's ``attention`` kernel object (examples/attention.py:29-84).
attention = DropInKernel(_attention_spec, _launch, _select, _describe, static_shapes=True)
#: The reference's dynamic-shape variant (examples/attention.py:89-97); shapes are always runtime values here.
attention_dynamic = DropInKernel(_attention_spec, _launch, _select, _describe, static_shapes=False)


def test(z: int, h: int, n_ctx: int, head_dim: int, dtype: torch.dtype = torch.float16,
         device: torch.device | str = "cuda") -> None:
    """The reference's comparison against PyTorch attention (examples/attention.py:103-146) with the
    harness's default tolerances (helion/_testing.py:341-405: rtol 1e-2, atol 1e-1)."""
    q, k, v = [torch.randn((z, h, n_ctx, head_dim), dtype=dtype, device=device) for _ in range(3)]

    def ref_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        p = torch.matmul(q, k.transpose(2, 3)) / math.sqrt(head_dim)
        p = torch.softmax(p.float(), dim=-1).to(dtype)
        return torch.matmul(p, v)

    out = attention(q, k, v)
    torch.testing.assert_close(out, torch.nn.functional.scaled_dot_product_attention(q, k, v), rtol=1e-2, atol=1e-1)
    torch.testing.assert_close(out, ref_attention(q, k, v), rtol=1e-2, atol=1e-1)
    print(f"attention z{z} h{h} n{n_ctx} d{head_dim} {dtype}: matches torch SDPA and the manual reference")


def main() -> None:
    test(2, 32, 1024, 64, torch.float16)


if __name__ == "__main__":
    main()
