"""Empty operands: every operator returns what the eager PyTorch expression of its reference returns
(an empty tensor, or zeros / the bias for an empty contraction) without launching a kernel."""
from __future__ import annotations

import pytest
import torch

from helion_b200 import _lib

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def hb(built_library):
    import helion_b200

    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    _lib.reset_status(0)
    yield helion_b200
    torch.cuda.synchronize()
    _lib.check_status(0)


def _e4m3(*shape):
    return torch.zeros(*shape, device="cuda").to(torch.float8_e4m3fn)


@pytest.mark.parametrize("m,n,k", [(0, 64, 32), (64, 0, 32), (0, 0, 0), (48, 80, 0)])
def test_fp8_gemm_with_an_empty_dimension(hb, m, n, k):
    out = hb.fp8_gemm(_e4m3(m, k), _e4m3(k, n), out_dtype=torch.float32)
    assert tuple(out.shape) == (m, n) and out.dtype == torch.float32
    assert torch.equal(out, torch.zeros(m, n, device="cuda"))  # x.float() @ y.float() of the same shapes
    sa, sb = torch.ones(m, 1, device="cuda"), torch.ones(1, n, device="cuda")
    if m and n:
        assert torch.equal(hb.fp8_gemm(_e4m3(m, k), _e4m3(k, n), out_dtype=torch.float32, scale_a=sa, scale_b=sb), out)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_matmul_with_an_empty_dimension(hb, dtype):
    bias = torch.linspace(-1, 1, 24, device="cuda").to(dtype)
    x, y = torch.zeros(16, 0, device="cuda", dtype=dtype), torch.zeros(0, 24, device="cuda", dtype=dtype)
    assert torch.equal(hb.matmul(x, y), torch.zeros(16, 24, device="cuda", dtype=dtype))
    want = torch.relu(x @ y + bias)  # the reference's check expression (examples/matmul.py:110-117)
    assert torch.equal(hb.matmul(x, y, bias=bias, relu=True), want)
    assert tuple(hb.matmul(torch.zeros(0, 8, device="cuda", dtype=dtype), torch.zeros(8, 24, device="cuda", dtype=dtype)).shape) == (0, 24)
    assert tuple(hb.matmul(torch.zeros(16, 8, device="cuda", dtype=dtype), torch.zeros(8, 0, device="cuda", dtype=dtype)).shape) == (16, 0)


def test_attention_with_no_slices_or_no_queries(hb):
    out = hb.fp8_attention(_e4m3(0, 128, 64), _e4m3(0, 128, 64), _e4m3(0, 64, 128), 0, 4)
    assert tuple(out.shape) == (0, 4, 128, 64) and out.dtype == torch.float8_e4m3fn
    out = hb.fp8_attention(_e4m3(2, 0, 64), _e4m3(2, 128, 64), _e4m3(2, 64, 128), 1, 2)
    assert tuple(out.shape) == (1, 2, 0, 64)
    q = torch.zeros(2, 0, 64, device="cuda", dtype=torch.float16)
    kv = torch.zeros(2, 32, 64, device="cuda", dtype=torch.float16)
    assert tuple(hb.attention(q, kv, kv).shape) == (2, 0, 64)
    with pytest.raises(ValueError, match="no keys"):
        hb.attention(kv, q, q)
    # the e4m3 kernel has no meaningful answer without keys either (softmax over nothing): it must refuse, not hang
    with pytest.raises(ValueError):
        hb.fp8_attention(_e4m3(2, 128, 64), _e4m3(2, 0, 64), _e4m3(2, 64, 0), 1, 2)


def test_preprocess_of_empty_tensors(hb):
    q = torch.zeros(0, 4, 128, 64, device="cuda", dtype=torch.float16)
    q8, k8, v8 = hb.preprocess_fp8_attention_inputs(q, q, q)
    assert q8.dtype == torch.float8_e4m3fn and tuple(q8.shape) == (0, 128, 64) and tuple(v8.shape) == (0, 64, 128)
