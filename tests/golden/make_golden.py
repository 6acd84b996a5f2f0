"""Generate the golden fixtures in this directory from the UNMODIFIED reference.

Runs pytorch-labs/helion's own ``examples/fp8_gemm.py``, ``test/test_dot.py`` (fp32-output
fp8 dot kernel) and ``examples/fp8_attention.py`` in ref-eager mode (``HELION_INTERPRET=1``)
on CPU tensors and stores inputs (e4m3 bit patterns) and outputs as ``.npz`` files.

Usage (needs a checkout of the reference; the fixtures themselves are committed, so the test
suite never needs it):

    HELION_INTERPRET=1 PYTHONPATH=<path-to-helion-checkout> python tests/golden/make_golden.py
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint8).numpy().copy()


def main() -> None:
    if os.environ.get("HELION_INTERPRET") != "1":
        sys.exit("set HELION_INTERPRET=1 (ref-eager mode) before running this script")
    from helion._testing import EXAMPLES_DIR, import_path

    ref_root = Path(EXAMPLES_DIR).parent
    sys.path.insert(0, str(ref_root))
    gemm_mod = import_path(EXAMPLES_DIR / "fp8_gemm.py")
    attn_mod = import_path(EXAMPLES_DIR / "fp8_attention.py")
    import test.test_dot as test_dot  # the reference's fp32-accumulator dot kernel

    # ---- GEMM: (name, M, N, K, seed, y column-major?) -----------------------------------
    gemm_cases = [
        ("gemm_256_colmajor", 256, 256, 256, 0, True),
        ("gemm_256_rowmajor", 256, 256, 256, 10, False),
        ("gemm_ragged_colmajor", 200, 144, 96, 11, True),
        ("gemm_ragged_rowmajor", 72, 272, 160, 12, False),
        ("gemm_skinny_colmajor", 16, 512, 1024, 13, True),
    ]
    for name, m, n, k, seed, colmajor in gemm_cases:
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(m, k, generator=g).clamp_(-448, 448).to(torch.float8_e4m3fn)
        y = torch.randn(k, n, generator=g).clamp_(-448, 448).to(torch.float8_e4m3fn)
        if colmajor:
            y = y.T.contiguous().T
        out16 = gemm_mod.fp8_gemm(x, y)
        out32 = test_dot.dot_kernel_acc_arg(x, y, torch.float32)
        assert out16.dtype == torch.float16 and out32.dtype == torch.float32
        np.savez_compressed(
            HERE / f"{name}.npz",
            x=_bits(x),
            y=_bits(y),  # logical [K, N], stored row-major; layout is recreated by the tests
            y_colmajor=np.array(colmajor),
            out_fp16=out16.numpy(),
            out_fp32=out32.numpy(),
        )
        print(name, tuple(out16.shape))

    # ---- attention: (name, B, H, S, D, seed) --------------------------------------------
    attn_cases = [
        ("attn_b1h2s128d64", 1, 2, 128, 64, 42),
        ("attn_b2h4s256d64", 2, 4, 256, 64, 43),
        ("attn_b1h2s512d128", 1, 2, 512, 128, 44),
        ("attn_b1h1s80d64", 1, 1, 80, 64, 45),
    ]
    for name, b, h, s, d, seed in attn_cases:
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(b, h, s, d, generator=g)
        k = torch.randn(b, h, s, d, generator=g)
        v = torch.randn(b, h, s, d, generator=g)
        q8, k8, v8 = attn_mod.preprocess_fp8_attention_inputs(q, k, v)
        out = attn_mod.fp8_attention_kernel(q8, k8, v8, b, h)
        assert out.dtype == torch.float8_e4m3fn and tuple(out.shape) == (b, h, s, d)
        np.savez_compressed(
            HERE / f"{name}.npz",
            q=_bits(q8),
            k=_bits(k8),
            v_sd=_bits(v8.permute(0, 2, 1)),  # physical layout [BH, S, D] (stride trap of preprocess)
            v_strides=np.array(v8.stride()),
            batch=np.array(b),
            heads=np.array(h),
            out=_bits(out),
        )
        print(name, tuple(out.shape), "v strides", v8.stride())


if __name__ == "__main__":
    main()
