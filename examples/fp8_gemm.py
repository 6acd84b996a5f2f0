"""FP8 GEMM behind the entry points of pytorch-labs/helion's ``examples/fp8_gemm.py``.

Same module-level names and positional signatures as the reference module, so callers that do
``importlib.import_module("examples.fp8_gemm")`` (benchmarks/run.py:73-77 of the reference) or
``import_path(EXAMPLES_DIR / "fp8_gemm.py")`` (helion/_testing.py:420) can be pointed at this
file.  The kernel body is the hand-written sm_100a CUDA kernel of ``helion_b200``.
"""
from __future__ import annotations

import torch

from helion_b200 import _lib
from helion_b200 import ops as _ops
from helion_b200.kernel import DropInKernel


def _fp8_gemm_spec(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """out[m, n] = fp16( sum_k fp32(x[m, k] * y[k, n]) ) for float8_e4m3fn x [m, k], y [k, n]."""
    raise NotImplementedError("specification only; the CUDA kernel implements it")


_fp8_gemm_spec.__name__ = "fp8_gemm"


def _launch(args, cfg_id, **kwargs):
    x, y = args
    return _ops.fp8_gemm(x, y, config=cfg_id, **kwargs)


def _select(args):
    x, y = args
    return _lib.load().hb200_fp8_gemm_select_config(x.shape[0], y.shape[1], x.shape[1], int(y.stride(0) == 1), 0)


def _describe(args, cfg_id):
    if cfg_id is None:
        cfg_id = _select(args)
    return _lib.describe_config(_lib.OP_GEMM, cfg_id)


#: Drop-in for the reference's ``fp8_gemm`` kernel object (examples/fp8_gemm.py:29-57):
#: ``fp8_gemm(x, y) -> fp16 [m, n]``; keyword-only extensions ``out_dtype``, ``config``, ``out``.
fp8_gemm = DropInKernel(_fp8_gemm_spec, _launch, _select, _describe, static_shapes=True)


def reference_fp8_gemm_pytorch(x_fp8: torch.Tensor, y_fp8: torch.Tensor) -> torch.Tensor:
    """cuBLASLt baseline, same call as the reference's (examples/fp8_gemm.py:61-78)."""
    y_fp8_t = y_fp8.T.contiguous().T
    scale_a = torch.tensor(1.0, device=x_fp8.device)
    scale_b = torch.tensor(1.0, device=x_fp8.device)
    return torch._scaled_mm(x_fp8, y_fp8_t, scale_a, scale_b, use_fast_accum=False, out_dtype=torch.float16)


def fp8_gemm_tritonbench(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Wrapper with the tritonbench operator signature (examples/fp8_gemm.py:82-91)."""
    return fp8_gemm(a, b)


def check(m: int, k: int, n: int) -> None:
    """Compare the kernel with the cuBLASLt baseline on unseeded N(0,1) inputs, with the reference
    harness's default tolerances (helion/_testing.py:341-405: rtol 1e-2, atol 1e-1)."""
    x = torch.randn([m, k], device="cuda", dtype=torch.float32)
    y = torch.randn([k, n], device="cuda", dtype=torch.float32)
    x_fp8 = x.to(torch.float8_e4m3fn)
    y_fp8 = y.to(torch.float8_e4m3fn)
    out = fp8_gemm(x_fp8, y_fp8)
    expected = reference_fp8_gemm_pytorch(x_fp8, y_fp8)
    torch.testing.assert_close(out.float(), expected.float(), rtol=1e-2, atol=1e-1)
    print(f"fp8_gemm {m}x{k}x{n}: matches torch._scaled_mm")


def main() -> None:
    check(256, 256, 256)
    check(512, 512, 512)
    check(1024, 1024, 1024)


if __name__ == "__main__":
    main()
