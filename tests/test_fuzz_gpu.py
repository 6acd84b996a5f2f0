"""Seeded random shapes, layouts, strides and output types through the C ABI on a B200, each compared
with the CPU oracle at the stated gates.  The fixed-shape tests pin the cases the reference's own
tests use; this file walks the supported domain more widely (ragged M / N / K, padded leading
dimensions, few-row problems that take the operand-swapped kernel, long and ragged sequences)."""
from __future__ import annotations

import random

import numpy as np
import pytest
import torch

from helion_b200 import _lib
from oracle import fp8_oracle as o

pytestmark = pytest.mark.gpu

NAME = {torch.float16: "fp16", torch.bfloat16: "bf16", torch.float32: "fp32"}


@pytest.fixture(scope="module")
def hb(built_library):
    import helion_b200

    _lib.reset_status(0)
    yield helion_b200
    torch.cuda.synchronize()
    _lib.check_status(0)


def _gemm_cases(count, seed):
    rng = random.Random(seed)
    for i in range(count):
        m = rng.choice([1, 3, 16, 17, 31, 64, 65, 127, 128, 129, 255, 300, 513, 1000])
        n = 8 * rng.randint(1, 160)
        k = 16 * rng.randint(1, 96)
        colmajor = rng.random() < 0.6 or n % 16 != 0
        pad_x = 16 * rng.randint(0, 2)
        pad_y = 16 * rng.randint(0, 2)
        dt = rng.choice([torch.float16, torch.bfloat16, torch.float32])
        scaled = rng.choice([None, None, "tensor", "rows"])
        yield pytest.param(m, n, k, colmajor, pad_x, pad_y, dt, scaled, 1000 + i, id=f"{m}x{n}x{k}-{'col' if colmajor else 'row'}-{NAME[dt]}-{scaled}")


@pytest.mark.parametrize("m,n,k,colmajor,pad_x,pad_y,dt,scaled,seed", list(_gemm_cases(40, seed=20240)))
def test_random_fp8_gemm(hb, m, n, k, colmajor, pad_x, pad_y, dt, scaled, seed):
    x, y = o.gemm_inputs(m, n, k, seed=seed)
    # operands as views of wider buffers: leading dimensions larger than the logical extents
    xbuf = torch.zeros(m, k + pad_x, dtype=torch.uint8).view(torch.float8_e4m3fn)
    xbuf[:, :k] = x
    xd = xbuf.cuda()[:, :k]
    if colmajor:
        ybuf = torch.zeros(n, k + pad_y, dtype=torch.uint8).view(torch.float8_e4m3fn)
        ybuf[:, :k] = y.t()
        yd = ybuf.cuda()[:, :k].t()
    else:
        ybuf = torch.zeros(k, n + pad_y, dtype=torch.uint8).view(torch.float8_e4m3fn)
        ybuf[:, :n] = y
        yd = ybuf.cuda()[:, :n]
    xb, yb = o.torch_fp8_to_bits(x), o.torch_fp8_to_bits(y)
    g = torch.Generator().manual_seed(seed)
    if scaled is None:
        got = hb.fp8_gemm(xd, yd, out_dtype=dt)
        want = o.fp8_gemm(xb, yb, NAME[dt])
        exact = o.fp8_gemm(xb, yb, "fp32")
    else:
        sa = torch.rand(1 if scaled == "tensor" else m, 1, generator=g) + 0.5
        sb = torch.rand(1, 1 if scaled == "tensor" else n, generator=g) + 0.5
        got = hb.fp8_gemm(xd, yd, out_dtype=dt, scale_a=sa.cuda(), scale_b=sb.cuda())
        want = o.fp8_gemm_scaled(xb, yb, sa.numpy(), sb.numpy(), NAME[dt])
        exact = o.fp8_gemm_scaled(xb, yb, sa.numpy(), sb.numpy(), "fp32")
    got = got.float().cpu().numpy()
    np.testing.assert_allclose(got, want, rtol=2e-2, atol=2e-2)
    assert o.rel_frobenius(got, exact) <= (2.5e-3 if dt == torch.bfloat16 else 1e-3)


def _row_cases(count, seed):
    rng = random.Random(seed)
    for i in range(count):
        few = rng.random() < 0.4
        row = rng.choice([18, 22, 23]) if few else rng.choice([6, 14, 21])
        m = rng.choice([1, 7, 16, 33, 64]) if few else rng.choice([130, 300, 513, 1000, 1500])
        n = 8 * rng.randint(1, 170)
        k = 16 * rng.randint(1, 64)
        pad_x = 16 * rng.randint(0, 2)
        pad_y = 16 * rng.randint(0, 2)
        dt = rng.choice([torch.float16, torch.bfloat16, torch.float32])
        scaled = rng.choice([None, None, "tensor", "rows"])
        yield pytest.param(row, m, n, k, pad_x, pad_y, dt, scaled, 3000 + i, id=f"row{row}-{m}x{n}x{k}-{NAME[dt]}-{scaled}")


@pytest.mark.parametrize("row,m,n,k,pad_x,pad_y,dt,scaled,seed", list(_row_cases(30, seed=515)))
def test_random_fp8_gemm_on_explicit_table_rows(hb, row, m, n, k, pad_x, pad_y, dt, scaled, seed):
    """The rows the automatic choice reaches only for particular shapes -- the CTA-pair tiles (6, 14, the 224-wide
    21) and the few-row kernels (18 and its chain forms 22 / 23) -- on ragged sizes, padded leading dimensions,
    every output type and both scale modes, column-major y."""
    x, y = o.gemm_inputs(m, n, k, seed=seed)
    xbuf = torch.zeros(m, k + pad_x, dtype=torch.uint8).view(torch.float8_e4m3fn)
    xbuf[:, :k] = x
    xd = xbuf.cuda()[:, :k]
    ybuf = torch.zeros(n, k + pad_y, dtype=torch.uint8).view(torch.float8_e4m3fn)
    ybuf[:, :k] = y.t()
    yd = ybuf.cuda()[:, :k].t()
    xb, yb = o.torch_fp8_to_bits(x), o.torch_fp8_to_bits(y)
    g = torch.Generator().manual_seed(seed)
    if scaled is None:
        got = hb.fp8_gemm(xd, yd, out_dtype=dt, config=row)
        want = o.fp8_gemm(xb, yb, NAME[dt])
        exact = o.fp8_gemm(xb, yb, "fp32")
    else:
        sa = torch.rand(1 if scaled == "tensor" else m, 1, generator=g) + 0.5
        sb = torch.rand(1, 1 if scaled == "tensor" else n, generator=g) + 0.5
        got = hb.fp8_gemm(xd, yd, out_dtype=dt, scale_a=sa.cuda(), scale_b=sb.cuda(), config=row)
        want = o.fp8_gemm_scaled(xb, yb, sa.numpy(), sb.numpy(), NAME[dt])
        exact = o.fp8_gemm_scaled(xb, yb, sa.numpy(), sb.numpy(), "fp32")
    got = got.float().cpu().numpy()
    np.testing.assert_allclose(got, want, rtol=2e-2, atol=2e-2)
    assert o.rel_frobenius(got, exact) <= (2.5e-3 if dt == torch.bfloat16 else 1e-3)


def _attn_cases(count, seed):
    rng = random.Random(seed)
    for i in range(count):
        b, h = rng.randint(1, 3), rng.randint(1, 5)
        s = 16 * rng.choice([1, 2, 5, 8, 9, 16, 23, 40, 64, 65, 130])
        d = rng.choice([64, 128])
        v_contig = rng.random() < 0.4
        cfg = rng.choice([None, None, 0, 4])
        yield pytest.param(b, h, s, d, v_contig, cfg, 2000 + i, id=f"B{b}H{h}S{s}D{d}-{'vDS' if v_contig else 'vSD'}-cfg{cfg}")


@pytest.mark.parametrize("b,h,s,d,v_contig,cfg,seed", list(_attn_cases(24, seed=777)))
def test_random_fp8_attention(hb, b, h, s, d, v_contig, cfg, seed):
    q, k, v = o.attention_inputs(b, h, s, d, seed)
    q8, k8, v8 = (t.to(torch.float8_e4m3fn).reshape(b * h, s, d) for t in (q, k, v))
    v_host = v8.permute(0, 2, 1).contiguous() if v_contig else v8.permute(0, 2, 1)
    v_dev = v_host.cuda() if v_contig else v8.cuda().permute(0, 2, 1)
    bits = lambda t: t.contiguous().view(torch.uint8).numpy()  # noqa: E731
    vbits = v_host.view(torch.uint8).numpy()
    _, one_raw = o.fp8_attention(bits(q8), bits(k8), vbits, b, h, return_parts=True)
    got = hb.fp8_attention(q8.cuda(), k8.cuda(), v_dev, b, h, out_dtype=torch.float32, config=cfg).cpu().numpy()
    assert np.isfinite(got).all()
    # Against the oracle that walks the keys in the kernel's own steps: all but a few elements within 1e-3 (one P
    # element on the other side of an e4m3 rounding boundary moves its whole row), every element within 2e-2.
    bn = 64 if d == 64 and cfg == 4 else 128  # the default row walks 128-key steps for every shape drawn here
    _, blk_raw = o.fp8_attention(bits(q8), bits(k8), vbits, b, h, return_parts=True, block_n=bn)
    off = np.abs(got - blk_raw) > 1e-3 + 1e-3 * np.abs(blk_raw)
    assert off.mean() <= 2e-3
    np.testing.assert_allclose(got, blk_raw, rtol=2e-2, atol=2e-2)
    # The parity contract of the attention kernel is the comparison above: the reference's own loop
    # (examples/fp8_attention.py:67-101) walked at the kernel's key-block size, every element within
    # allclose(rtol = atol = 2e-2) and all but 0.2 % within 1e-3.  The single-tile evaluation (what ref-eager
    # computes when the whole key range is one tile) is a different schedule of the same loop: the running max of
    # a blocked walk changes how the un-normalised P rounds to e4m3, which the reference's compiled kernel shares
    # with this one.  Against it a bounded excess is allowed: at most 1e-4 of a case's elements beyond 2e-2, none
    # beyond 4e-2.  (A sweep of 150 random cases with 128 to 4096 keys met no element beyond 2e-2, the largest
    # difference being 1.5e-2 at 256 keys; the allowance is headroom for rarer draws.)
    viol = np.abs(got - one_raw) > 2e-2 + 2e-2 * np.abs(one_raw)
    assert viol.mean() <= 1e-4 and np.abs(got - one_raw).max() <= 4e-2
    out8 = hb.fp8_attention(q8.cuda(), k8.cuda(), v_dev, b, h, config=cfg).view(torch.uint8).cpu().numpy()
    assert (out8 == o.e4m3_encode(got)).mean() >= 0.9999  # the e4m3 output is the fp32 result rounded once
    assert (out8 == o.e4m3_encode(blk_raw)).mean() >= 0.995  # and matches the blocked oracle's bytes


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
def test_random_16bit_matmul(hb, dtype):
    rng = random.Random(99)
    for i in range(12):
        m = rng.choice([1, 7, 64, 129, 300, 777])
        n, k = 8 * rng.randint(1, 120), 8 * rng.randint(1, 150)
        colmajor = rng.random() < 0.5
        g = torch.Generator().manual_seed(3000 + i)
        x = torch.randn(m, k, generator=g).to(dtype)
        y = torch.randn(n, k, generator=g).to(dtype).t() if colmajor else torch.randn(k, n, generator=g).to(dtype)
        bias = torch.randn(n, generator=g).to(dtype)
        relu = rng.random() < 0.5
        yd = y.t().contiguous().cuda().t() if colmajor else y.cuda()
        got = hb.matmul(x.cuda(), yd, bias=bias.cuda(), relu=relu).float().cpu().numpy()
        want = o.matmul_16bit(x.float().numpy(), y.float().numpy(), bias.float().numpy(), relu, NAME[dtype])
        np.testing.assert_allclose(got, want, rtol=2e-2, atol=2e-2, err_msg=f"{m}x{n}x{k} colmajor={colmajor}")
