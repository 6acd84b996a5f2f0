"""fp16 / bf16 attention on a B200: attention16_kernel, called through the C ABI (helion_b200.ops.attention
-> hb200_attention_16bit), against the CPU oracle (oracle.attention_16bit, the restatement of the
reference's examples/attention.py in ref-eager mode).

The kernel walks the keys in blocks of 64; the oracle does the same (``block_n=64``) for the tight
comparison (fp32 output within 2e-3 of it: ex2.approx, summation order and rare 16-bit rounding flips of
P) and as one tile (what ref-eager does) for the stated tolerance allclose(2e-2, 2e-2)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helion_b200 import _lib
from oracle import fp8_oracle as o

pytestmark = pytest.mark.gpu

NAME = {torch.float16: "fp16", torch.bfloat16: "bf16"}


@pytest.fixture(scope="module")
def hb(built_library):
    import helion_b200

    _lib.reset_status(0)
    yield helion_b200
    torch.cuda.synchronize()
    _lib.check_status(0)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize(
    "lead,sq,sk,dim",
    [((1, 2), 128, 128, 64), ((2, 4), 256, 256, 64), ((1, 2), 512, 512, 128), ((3,), 80, 208, 64), ((1, 1), 16, 16, 128),
     ((2, 2), 1024, 1040, 64), ((1, 3), 200, 72, 128), ((5, 7), 144, 144, 64), ((), 192, 320, 128),
     ((2, 2), 100, 77, 32), ((3,), 256, 130, 96), ((1, 2), 64, 64, 80)],  # head_dims in between: zero-padded columns
)
def test_matches_oracle(hb, lead, sq, sk, dim, dtype):
    g = torch.Generator().manual_seed(sq + sk + dim)
    q = torch.randn(*lead, sq, dim, generator=g).to(dtype)
    k = torch.randn(*lead, sk, dim, generator=g).to(dtype)
    v = torch.randn(*lead, sk, dim, generator=g).to(dtype)
    f3 = lambda t: t.float().reshape(-1, t.shape[-2], dim).numpy()  # noqa: E731
    one, one_raw = o.attention_16bit(f3(q), f3(k), f3(v), NAME[dtype], return_parts=True)
    # the kernel walks 128 keys per step at (padded) head_dim 64 and 64 at head_dim 128
    blk, blk_raw = o.attention_16bit(f3(q), f3(k), f3(v), NAME[dtype], block_n=128 if dim <= 64 else 64, return_parts=True)
    out = hb.attention(q.cuda(), k.cuda(), v.cuda())
    out32 = hb.attention(q.cuda(), k.cuda(), v.cuda(), out_dtype=torch.float32)
    assert out.dtype == dtype and out.shape == q.shape and out32.shape == q.shape
    got32 = out32.cpu().numpy().reshape(-1, sq, dim)
    got = out.float().cpu().numpy().reshape(-1, sq, dim)
    assert np.isfinite(got32).all()
    off = np.abs(got32 - blk_raw) > 2e-3 + 2e-3 * np.abs(blk_raw)
    assert off.mean() <= 2e-3, f"{off.sum()} of {off.size} elements differ from the blocked oracle by more than 2e-3"
    np.testing.assert_allclose(got32, one_raw, rtol=2e-2, atol=2e-2)
    np.testing.assert_allclose(got, one, rtol=2e-2, atol=2e-2)
    # the 16-bit output is the fp32 result rounded to nearest even
    assert (got == o.round_to_dtype(got32, NAME[dtype])).mean() >= 0.9999
    for balanced in (False, True):
        assert torch.equal(hb.attention(q.cuda(), k.cuda(), v.cuda(), balanced=balanced), out)


def test_example_module_and_argument_checks(hb):
    import examples.attention as mod

    mod.test(2, 4, 256, 64, torch.float16)
    mod.test(1, 2, 512, 128, torch.bfloat16)
    q = torch.randn(2, 3, 128, 64, device="cuda", dtype=torch.float16)
    assert torch.equal(mod.attention_dynamic(q, q, q), mod.attention(q, q, q))
    with pytest.raises(TypeError, match="float16 or three bfloat16"):
        mod.attention(q.float(), q.float(), q.float())  # the reference's fp32 default is not built
    wide = torch.zeros(2, 128, 256, device="cuda", dtype=torch.float16)
    with pytest.raises(ValueError, match=r"head_dim must be in \[1, 128\]"):
        hb.attention(wide, wide, wide)
    with pytest.raises(AssertionError):
        hb.attention(q, q[:, :, :64], q)


def test_full_size_properties(hb):
    """B4 H48 S1024 D64 in bf16: slices against the oracle, slice permutation commutes exactly."""
    g = torch.Generator(device="cuda").manual_seed(8)
    q, k, v = (torch.randn(4, 48, 1024, 64, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
    out = hb.attention(q, k, v, out_dtype=torch.float32)
    for b, h in ((0, 0), (2, 17), (3, 47)):
        f = lambda t: t[b, h].float().cpu().numpy()[None]  # noqa: E731
        _, raw = o.attention_16bit(f(q), f(k), f(v), "bf16", return_parts=True)
        np.testing.assert_allclose(out[b, h].cpu().numpy(), raw[0], rtol=2e-2, atol=2e-2)
    perm = torch.randperm(48, device="cuda", generator=torch.Generator(device="cuda").manual_seed(9))
    assert torch.equal(hb.attention(q[:, perm], k[:, perm], v[:, perm]), hb.attention(q, k, v)[:, perm])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("b,h,s,d", [(2, 4, 512, 64), (1, 8, 1024, 128), (2, 2, 200, 64)])
def test_against_atens_attention_on_the_gpu(hb, b, h, s, d, dtype):
    """What the reference's own example checks against (examples/attention.py:128-145: a matmul / softmax / matmul
    baseline and ``torch.nn.functional.scaled_dot_product_attention``, through run_example with rtol 1e-2, atol
    1e-1): both on the same GPU, held to allclose(2e-2, 2e-2) here."""
    g = torch.Generator().manual_seed(9000 + s + d)
    q, k, v = (torch.randn(b, h, s, d, generator=g).to(dtype).cuda() for _ in range(3))
    got = hb.attention(q, k, v)
    sdpa = torch.nn.functional.scaled_dot_product_attention(q, k, v)
    p = torch.softmax(torch.matmul(q.float(), k.float().transpose(2, 3)) / (d ** 0.5), dim=-1)
    plain = torch.matmul(p, v.float())
    torch.testing.assert_close(got, sdpa, rtol=1e-2, atol=1e-1)  # the reference's gate
    torch.testing.assert_close(got.float(), sdpa.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(got.float(), plain, rtol=2e-2, atol=2e-2)

