"""The attention input preparation on a B200: hb200_fp8_attention_preprocess (q, k, v -> e4m3 in one
launch) against the oracle's restatement of torch's float8_e4m3fn cast and against the reference
function's own definition (examples/fp8_attention.py:110-133: three ``.to(torch.float8_e4m3fn)``
casts and stride-only reshapes).  Byte work, so the bar is bit-exactness."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helion_b200 import _lib
from oracle import fp8_oracle as o

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def hb(built_library):
    import helion_b200

    _lib.reset_status(0)
    yield helion_b200
    torch.cuda.synchronize()
    _lib.check_status(0)


def reference_definition(q, k, v):
    """The reference's function, restated with torch ops on whatever device the inputs are on."""
    batch, heads, seq, dim = q.shape
    q8, k8 = q.to(torch.float8_e4m3fn), k.to(torch.float8_e4m3fn)
    v8 = v.permute(0, 1, 3, 2).to(torch.float8_e4m3fn)
    return (q8.reshape(batch * heads, seq, dim), k8.reshape(batch * heads, seq, dim),
            v8.reshape(batch * heads, dim, seq))


def same_bytes_or_both_nan(got: torch.Tensor, want_bits: np.ndarray):
    g = got.contiguous().view(torch.uint8).cpu().numpy().reshape(-1)
    w = want_bits.reshape(-1)
    nan_g, nan_w = (g & 0x7F) == 0x7F, (w & 0x7F) == 0x7F
    assert np.array_equal(nan_g, nan_w)
    assert np.array_equal(g[~nan_g], w[~nan_w])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32], ids=["fp16", "bf16", "fp32"])
@pytest.mark.parametrize("shape", [(1, 2, 128, 64), (2, 3, 80, 128), (4, 48, 1024, 64)])
def test_matches_the_oracle_cast_and_the_reference_definition(hb, dtype, shape):
    g = torch.Generator().manual_seed(sum(shape))
    q, k, v = (torch.randn(shape, generator=g).to(dtype) for _ in range(3))
    k = k * 40.0   # into the top binades
    v = v * 1e-2   # into the subnormals
    q8, k8, v8 = hb.preprocess_fp8_attention_inputs(q.cuda(), k.cuda(), v.cuda())
    rq, rk, rv = reference_definition(q, k, v)
    for got, want, src in ((q8, rq, q), (k8, rk, k), (v8, rv, v)):
        assert got.dtype == torch.float8_e4m3fn and got.shape == want.shape and got.stride() == want.stride()
        # bit patterns: the oracle's encoder (pinned against torch's cast in tests/test_oracle.py) ...
        want_bits = o.e4m3_encode(src.float().numpy())
        if got is v8:
            want_bits = want_bits.reshape(-1, shape[2], shape[3]).transpose(0, 2, 1)
        same_bytes_or_both_nan(got, np.ascontiguousarray(want_bits))
        # ... and torch's own cast as the reference's function applies it
        same_bytes_or_both_nan(got, want.contiguous().view(torch.uint8).numpy())


def test_edge_values(hb):
    """Ties, the largest finite value, the overflow threshold, infinities, NaN, signed zeros and
    subnormals; torch's cast turns everything that rounds beyond 448 into NaN instead of clamping."""
    specials = [0.0, -0.0, 448.0, -448.0, 463.9, 464.0, 464.1, 465.0, -464.0, -480.0, 1e9, -1e9, float("inf"),
                float("-inf"), float("nan"), 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -10, 2.0 ** -11, 3.0 * 2.0 ** -10,
                0.0009765625, 17.0, 18.0, 19.0, 20.0, 22.0, 26.0, 0.40625, 0.4375, 0.46875, 1.0625, 1.1875]
    base = torch.tensor(specials, dtype=torch.float32)
    src = torch.cat([base, -base, torch.linspace(-500, 500, 4096 - 2 * len(specials))]).reshape(1, 1, 64, 64)
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        s = src.to(dtype)
        q8, k8, v8 = hb.preprocess_fp8_attention_inputs(s.cuda(), s.cuda(), s.cuda())
        want = o.e4m3_encode(s.float().numpy())
        same_bytes_or_both_nan(q8, want)
        same_bytes_or_both_nan(k8, want)
        same_bytes_or_both_nan(v8.permute(0, 2, 1), want)
        torch_bits = s.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        same_bytes_or_both_nan(q8, torch_bits)
        got = q8.view(torch.uint8).cpu().numpy().reshape(-1)
        assert (got[np.abs(s.float().numpy().reshape(-1)) > 464.0] & 0x7F == 0x7F).all()  # no clamping


def test_feeds_the_attention_kernel_like_the_torch_casts(hb):
    import examples.fp8_attention as mod

    g = torch.Generator(device="cuda").manual_seed(3)
    q, k, v = (torch.randn(2, 4, 256, 64, device="cuda", dtype=torch.float16, generator=g) for _ in range(3))
    a = mod.fp8_attention_tritonbench(q, k, v)()
    rq, rk, rv = reference_definition(q, k, v)
    b = hb.fp8_attention(rq, rk, rv, 2, 4)
    assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))


def test_argument_checks(hb, built_library):
    x = torch.zeros(1, 1, 16, 64, device="cuda", dtype=torch.float16)
    with pytest.raises(TypeError, match="share one dtype"):
        hb.preprocess_fp8_attention_inputs(x, x.float(), x)
    with pytest.raises(ValueError, match=r"\[B,H,S,D\]"):
        hb.preprocess_fp8_attention_inputs(x[0], x[0], x[0])
    out = torch.empty(1024, dtype=torch.uint8, device="cuda")
    call = built_library.hb200_fp8_attention_preprocess
    stream = torch.cuda.current_stream().cuda_stream
    p, d = x.data_ptr(), out.data_ptr()
    assert call(p, p, p, d, d, d, 1000, _lib.DT_FP16, 0, stream) == _lib.ERR_BAD_SHAPE      # not a multiple of 16
    assert call(p, p, p, d, d, d, 1024, _lib.DT_E4M3, 0, stream) == _lib.ERR_BAD_DTYPE
    assert call(p, p, p + 2, d, d, d, 1008, _lib.DT_FP16, 0, stream) == _lib.ERR_ALIGN
    assert call(p, p, None, d, d, d, 1024, _lib.DT_FP16, 0, stream) == _lib.ERR_ALIGN
