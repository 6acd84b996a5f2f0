"""Value extremes of e4m3 operands: the largest finite magnitude (an fp16 output overflows to infinity exactly where
the rounded fp32 sum does), subnormals (products are exact in fp32), NaN operands (propagate), and attention rows
whose softmax is a one-hot or uniform distribution."""
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

    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    _lib.reset_status(0)
    yield helion_b200
    torch.cuda.synchronize()
    _lib.check_status(0)


def _from_bits(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.astype(np.uint8)).view(torch.float8_e4m3fn)


@pytest.mark.parametrize("m", [16, 160])
def test_gemm_largest_and_smallest_magnitudes(hb, m):
    rng = np.random.default_rng(m)
    n, k = 256, 512
    # bytes 0x7e / 0xfe = +-448, 0x01 / 0x81 = +-2^-9 (subnormal), 0x00 / 0x80 = +-0
    pool = np.array([0x7E, 0xFE, 0x01, 0x81, 0x00, 0x80, 0x38, 0xB8], dtype=np.uint8)
    xb = pool[rng.integers(0, len(pool), size=(m, k))]
    yb = pool[rng.integers(0, len(pool), size=(k, n))]
    xb[0, :], yb[:, 0] = 0x7E, 0x7E  # one dot product of 512 x 448^2 = 1.03e8: beyond fp16, fine in bf16 / fp32
    xd = _from_bits(xb).cuda()
    yd = _from_bits(np.ascontiguousarray(yb.T)).cuda().t()
    # Every product is exact in fp32; sums of +-448^2 terms cancel, so the error of ANY fp32 summation order is
    # bounded relative to sum |x||y|, not to the result: a few fp32 ulps of that magnitude.
    x64, y64 = o.e4m3_decode(xb).astype(np.float64), o.e4m3_decode(yb).astype(np.float64)
    exact = x64 @ y64
    bound = 4e-7 * (np.abs(x64) @ np.abs(y64)) + 1e-30
    got32 = hb.fp8_gemm(xd, yd, out_dtype=torch.float32).cpu().numpy()
    assert np.isfinite(got32).all()
    assert (np.abs(got32 - exact) <= bound).all()
    assert (np.abs(o.fp8_gemm(xb, yb, "fp32") - exact) <= bound).all()  # the oracle obeys the same bound
    assert got32[0, 0] == np.float32(512 * 448.0 * 448.0)  # no cancellation here: exact
    got16 = hb.fp8_gemm(xd, yd).float().cpu().numpy()
    overflow = np.abs(exact) - bound > 65520.0    # certainly beyond the largest fp16 value after rounding
    in_range = np.abs(exact) + bound < 65504.0
    assert overflow[0, 0] and np.isinf(got16[overflow]).all() and np.isfinite(got16[in_range]).all()
    assert (np.abs(got16 - exact)[in_range] <= (bound + np.abs(exact) * 2.0 ** -11 + 2.0 ** -24)[in_range]).all()
    gotbf = hb.fp8_gemm(xd, yd, out_dtype=torch.bfloat16).float().cpu().numpy()
    assert (np.abs(gotbf - exact) <= bound + np.abs(exact) * 2.0 ** -8).all()


def test_gemm_nan_operand_poisons_its_row_and_column_only(hb):
    x, y = o.gemm_inputs(130, 272, 256, seed=77)
    xb, yb = o.torch_fp8_to_bits(x).copy(), o.torch_fp8_to_bits(y).copy()
    xb[5, 17] = 0x7F   # NaN in row 5 of x
    yb[40, 9] = 0xFF   # NaN in column 9 of y
    got = hb.fp8_gemm(_from_bits(xb).cuda(), _from_bits(np.ascontiguousarray(yb.T)).cuda().t(), out_dtype=torch.float32).cpu().numpy()
    nan = np.isnan(got)
    want_nan = np.zeros_like(nan)
    want_nan[5, :] = True
    want_nan[:, 9] = True
    assert np.array_equal(nan, want_nan)
    xb[5, 17], yb[40, 9] = 0, 0
    clean = o.fp8_gemm(xb, yb, "fp32")
    np.testing.assert_allclose(got[~nan], clean[~want_nan], rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("d", [64, 128])
def test_attention_one_hot_and_uniform_rows(hb, d):
    bh, s = 2, 256
    g = torch.Generator().manual_seed(d)
    v = torch.randn(bh, s, d, generator=g).to(torch.float8_e4m3fn)
    # slice 0: q = k = 0 -> every score 0 -> uniform softmax -> each output row is the mean of v
    # slice 1: query i matches key i with a score far above the rest -> one-hot softmax -> output row i = v[i]
    q = torch.zeros(bh, s, d)
    k = torch.zeros(bh, s, d)
    # row i carries the 8 bits of i as +-32 in its first 8 columns: q_i . k_j = 1024 (8 - 2 hamming(i, j)),
    # largest at j = i by 2048 -- hundreds of binades after the softmax scale
    bits_of = ((torch.arange(s)[:, None] >> torch.arange(8)[None, :]) & 1).float() * 64.0 - 32.0
    q[1, :, :8], k[1, :, :8] = bits_of, bits_of
    q8, k8 = q.to(torch.float8_e4m3fn), k.to(torch.float8_e4m3fn)
    got = hb.fp8_attention(q8.cuda(), k8.cuda(), v.cuda().permute(0, 2, 1), 1, bh, out_dtype=torch.float32).cpu().numpy()[0]
    _, want = o.fp8_attention(o.torch_fp8_to_bits(q8), o.torch_fp8_to_bits(k8), o.torch_fp8_to_bits(v.permute(0, 2, 1)), 1, bh,
                              return_parts=True, block_n=128)
    assert np.isfinite(got).all()
    np.testing.assert_allclose(got, np.asarray(want)[0], rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(got[0], np.broadcast_to(v[0].float().numpy().mean(axis=0), (s, d)), rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(got[1], v[1].float().numpy(), rtol=1e-6, atol=1e-6)  # one-hot rows return v[i]
