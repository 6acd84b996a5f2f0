"""The CPU oracle against the reference's own outputs (tests/golden, produced by running the
unmodified reference in ref-eager mode) and against torch's float8_e4m3fn codec."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import ATTN_GOLDEN, GEMM_GOLDEN, load_golden
from oracle import fp8_oracle as o


def test_e4m3_decode_matches_torch():
    bits = np.arange(256, dtype=np.uint8)
    want = torch.from_numpy(bits).view(torch.float8_e4m3fn).float().numpy()
    got = o.e4m3_decode(bits)
    assert np.array_equal(np.isnan(want), np.isnan(got))
    assert np.array_equal(want[~np.isnan(want)], got[~np.isnan(got)])


def test_e4m3_encode_matches_torch_cast():
    g = torch.Generator().manual_seed(7)
    x = torch.randn(1 << 18, generator=g) * torch.logspace(-4, 2.7, 1 << 18)
    edge = torch.tensor(
        [0.0, -0.0, 448.0, 463.9, 464.0, 465.0, 480.0, 1e9, -1e9, 2.0**-10, 2.0**-10 * 1.0001, 3 * 2.0**-10,
         2.0**-9, 2.0**-6, 0.0175, float("nan")]
    )
    x = torch.cat([x, edge])
    want = x.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = o.e4m3_encode(x.numpy())
    assert np.array_equal(want, got)


def test_e4m3_roundtrip_is_identity_on_finite_codes():
    bits = np.array([b for b in range(256) if (b & 0x7F) != 0x7F], dtype=np.uint8)
    assert np.array_equal(o.e4m3_encode(o.e4m3_decode(bits)), bits)


def test_bf16_rounding_matches_torch():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(1 << 16, generator=g) * 1000
    want = x.to(torch.bfloat16).float().numpy()
    assert np.array_equal(o.round_to_dtype(x.numpy(), "bf16"), want)


@pytest.mark.parametrize("name", GEMM_GOLDEN)
def test_gemm_oracle_matches_reference(name):
    z = load_golden(name)
    got16 = o.fp8_gemm(z["x"], z["y"], "fp16")
    got32 = o.fp8_gemm(z["x"], z["y"], "fp32")
    # fp32 accumulation order is the only freedom: the reference's fp16 output must be reproduced
    # exactly (up to ties, none occur) and the fp32 output to summation-order noise.
    assert (got16 == z["out_fp16"].astype(np.float32)).mean() > 0.9999
    assert o.rel_frobenius(got32, z["out_fp32"]) < 1e-6
    np.testing.assert_allclose(got32, z["out_fp32"], rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("name", ATTN_GOLDEN)
def test_attention_oracle_matches_reference(name):
    z = load_golden(name)
    v = np.transpose(z["v_sd"], (0, 2, 1))  # logical [BH, D, S] over physical [BH, S, D]
    got = o.fp8_attention(z["q"], z["k"], v, int(z["batch"]), int(z["heads"]))
    got_bits = o.e4m3_encode(got)
    # numpy's exp2/sum may differ from ATen's in the last bit, which can flip an e4m3 rounding.
    assert (got_bits == z["out"]).mean() > 0.999
    np.testing.assert_allclose(got, o.e4m3_decode(z["out"]), rtol=0.13, atol=2e-3)


@pytest.mark.parametrize("name", ["attn_b2h4s256d64", "attn_b1h2s512d128"])
def test_blocked_attention_stays_within_tolerance_of_single_tile(name):
    """Walking the keys in blocks of 128 (what a compiled kernel does) changes how P rounds to
    e4m3; the fp32 result must stay within allclose(2e-2, 2e-2) of the single-tile result."""
    z = load_golden(name)
    v = np.transpose(z["v_sd"], (0, 2, 1))
    b, h = int(z["batch"]), int(z["heads"])
    _, one = o.fp8_attention(z["q"], z["k"], v, b, h, return_parts=True)
    _, blk = o.fp8_attention(z["q"], z["k"], v, b, h, return_parts=True, block_n=128)
    np.testing.assert_allclose(blk, one, rtol=2e-2, atol=2e-2)
    assert not np.array_equal(blk, one)


def test_attention_single_block_equals_single_tile():
    z = load_golden("attn_b1h2s128d64")
    v = np.transpose(z["v_sd"], (0, 2, 1))
    a = o.fp8_attention(z["q"], z["k"], v, 1, 2)
    b = o.fp8_attention(z["q"], z["k"], v, 1, 2, block_n=128)
    assert np.array_equal(a, b)


def test_gemm_oracle_rejects_mismatched_k():
    with pytest.raises(AssertionError, match="size mismatch"):
        o.fp8_gemm(np.zeros((4, 16), np.uint8), np.zeros((32, 8), np.uint8))


def test_input_generators_are_seeded_and_in_range():
    x1, y1 = o.gemm_inputs(64, 48, 32, seed=5)
    x2, y2 = o.gemm_inputs(64, 48, 32, seed=5)
    assert torch.equal(x1.view(torch.uint8), x2.view(torch.uint8))
    assert y1.shape == (32, 48) and y1.stride() == (1, 32)  # column-major
    assert not torch.isnan(y1.float()).any()
    _, w = o.gemm_inputs(64, 48, 32, seed=5, weight_like=True)
    assert w.float().abs().max() == 448.0


def test_scaled_gemm_oracle_against_aten_and_its_own_identities():
    """The op the reference calls is ATen's _scaled_mm (examples/fp8_gemm.py:74-78, with both scales
    1.0).  Its CPU build takes per-tensor scales: the restatement must agree with it to fp32
    rounding.  Row-wise scales exist only in ATen's CUDA build, so that form is pinned by
    identities: constant vectors equal the per-tensor form bit for bit, unit scales equal the
    unscaled oracle, and powers of two commute with every rounding."""
    x, y = o.gemm_inputs(48, 80, 64, seed=21)
    xb, yb = o.torch_fp8_to_bits(x), o.torch_fp8_to_bits(y)
    sa, sb = np.float32(0.37), np.float32(2.5)
    want = torch._scaled_mm(x, y, torch.tensor(float(sa)), torch.tensor(float(sb)), out_dtype=torch.float32).numpy()
    got = o.fp8_gemm_scaled(xb, yb, sa, sb, "fp32")
    np.testing.assert_allclose(got, want, rtol=2e-6, atol=1e-5)
    rows = o.fp8_gemm_scaled(xb, yb, np.full(48, sa), np.full(80, sb), "fp32")
    assert np.array_equal(rows, got)
    assert np.array_equal(o.fp8_gemm_scaled(xb, yb, 1.0, 1.0, "bf16"), o.fp8_gemm(xb, yb, "bf16"))
    assert np.array_equal(o.fp8_gemm_scaled(xb, yb, 0.25, 8.0, "fp32"), 2.0 * o.fp8_gemm(xb, yb, "fp32"))
    ra = np.linspace(0.5, 1.5, 48, dtype=np.float32)
    rb = np.linspace(2.0, 0.25, 80, dtype=np.float32)
    full = o.fp8_gemm(xb, yb, "fp32")
    np.testing.assert_array_equal(o.fp8_gemm_scaled(xb, yb, ra, rb, "fp32"), (full * ra[:, None]) * rb[None, :])
    with pytest.raises(ValueError):
        o.fp8_gemm_scaled(xb, yb, ra, np.float32(1.0), "fp32")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
def test_matmul_16bit_oracle_against_torch(dtype):
    """The reference's matmul example cannot run in ref-eager mode on a CPU (aten::mm.dtype is
    CUDA-only), so its restatement is checked against torch's own fp32 matmul of the upcast operands
    and torch's casts: same values up to the order of the fp32 K sum."""
    g = torch.Generator().manual_seed(9)
    x = torch.randn(72, 160, generator=g).to(dtype)
    y = torch.randn(160, 136, generator=g).to(dtype)
    bias = torch.randn(136, generator=g).to(dtype)
    name = "fp16" if dtype == torch.float16 else "bf16"
    acc = x.float() @ y.float()
    for b, relu in ((None, False), (bias, False), (bias, True)):
        want = acc if b is None else acc + b.float()
        want = torch.relu(want) if relu else want
        got = o.matmul_16bit(x.float().numpy(), y.float().numpy(), None if b is None else b.float().numpy(), relu, name)
        got32 = o.matmul_16bit(x.float().numpy(), y.float().numpy(), None if b is None else b.float().numpy(), relu, "fp32")
        np.testing.assert_allclose(got32, want.numpy(), rtol=1e-5, atol=1e-4)
        # after the cast at most the last bit differs (where the fp32 values straddle a rounding boundary)
        np.testing.assert_allclose(got, want.to(dtype).float().numpy(), rtol=2 ** -7 if name == "bf16" else 2 ** -10, atol=1e-3)
    with pytest.raises(AssertionError, match="size mismatch"):
        o.matmul_16bit(np.zeros((4, 8), np.float32), np.zeros((16, 4), np.float32))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
def test_attention_16bit_oracle_against_torch(dtype):
    """examples/attention.py cannot run in ref-eager mode on a CPU either (aten::bmm.dtype is CUDA-only),
    so its restatement is checked against the same sequence of eager torch operations written with
    ``bmm(...).float()`` in place of the mixed-precision baddbmm, and against exact softmax attention."""
    import math

    g = torch.Generator().manual_seed(4)
    q, k, v = (torch.randn(2, n, 64, generator=g).to(dtype) for n in (48, 80, 80))
    name = "fp16" if dtype == torch.float16 else "bf16"
    qk_scale = (1.0 / math.sqrt(64.0)) * 1.44269504
    qk = torch.bmm(q, k.transpose(1, 2))
    m = torch.amax(qk, -1).float() * 0 + (torch.amax(qk, -1) * qk_scale).float()
    x = (qk * qk_scale).float() - m[:, :, None]
    p = torch.exp2(x)
    l = p.sum(-1)
    acc = torch.bmm(p.to(dtype).float(), v.float())
    want = (acc / l[:, :, None]).to(dtype)
    got = o.attention_16bit(q.float().numpy(), k.float().numpy(), v.float().numpy(), name)
    ulp = 2.0 ** -7 if name == "bf16" else 2.0 ** -10
    np.testing.assert_allclose(got, want.float().numpy(), rtol=2 * ulp, atol=1e-3)
    exact = torch.softmax((q.double() @ k.double().transpose(1, 2)) / 8.0, -1) @ v.double()
    np.testing.assert_allclose(got, exact.float().numpy(), rtol=2e-2, atol=2e-2)
    blocked = o.attention_16bit(q.float().numpy(), k.float().numpy(), v.float().numpy(), name, block_n=32)
    np.testing.assert_allclose(blocked, got, rtol=2e-2, atol=2e-2)
