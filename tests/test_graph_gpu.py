"""CUDA-graph capture of the operators: the launch path allocates nothing outside torch's (graph-aware)
caching allocator, never synchronises and passes everything by value, so a captured call replays on new
data in the same buffers -- the property the reference's launcher has through Triton's
(helion/runtime/__init__.py:55-65) and that a decode loop needs (a 20 us kernel is launch-bound)."""
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


def _capture(fn):
    """Warm up on a side stream (first-call set-up is not capturable), capture one call, return the graph."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    return graph


@pytest.mark.parametrize("m,n,k", [(16, 512, 1024), (128, 1024, 512), (512, 768, 2048)])
def test_gemm_replays_on_new_data(hb, m, n, k):
    x, y = o.gemm_inputs(m, n, k, seed=1)
    xd, yd = x.cuda(), y.t().contiguous().cuda().t()
    out = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
    graph = _capture(lambda: hb.fp8_gemm(xd, yd, out_dtype=torch.bfloat16, out=out))
    for seed in (2, 3):
        x2, y2 = o.gemm_inputs(m, n, k, seed=seed)
        xd.copy_(x2.cuda())
        yd.copy_(y2.t().contiguous().cuda().t())
        out.zero_()
        graph.replay()
        eager = hb.fp8_gemm(xd, yd, out_dtype=torch.bfloat16)
        assert torch.equal(out, eager)
        want = o.fp8_gemm(o.torch_fp8_to_bits(x2), o.torch_fp8_to_bits(y2), "bf16")
        np.testing.assert_allclose(out.float().cpu().numpy(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("balanced", [False, True])
@pytest.mark.parametrize("causal", [False, True])
def test_attention_replays_on_new_data(hb, balanced, causal):
    b, h, s, d = 1, 4, 384, 64
    q, k, v = o.attention_inputs(b, h, s, d, seed=5)
    q8, k8, v8 = (t.to(torch.float8_e4m3fn).reshape(b * h, s, d).cuda() for t in (q, k, v))
    vt = v8.permute(0, 2, 1)
    out = torch.zeros(b, h, s, d, device="cuda").to(torch.float8_e4m3fn)
    graph = _capture(lambda: hb.fp8_attention(q8, k8, vt, b, h, out=out, balanced=balanced, causal=causal))
    for seed in (6, 7):
        q2, k2, v2 = o.attention_inputs(b, h, s, d, seed=seed)
        for dst, src in ((q8, q2), (k8, k2), (v8, v2)):
            dst.copy_(src.to(torch.float8_e4m3fn).reshape(b * h, s, d).cuda())
        out.view(torch.uint8).zero_()
        graph.replay()  # the balanced order's tile counter is cleared inside the graph
        eager = hb.fp8_attention(q8, k8, vt, b, h, balanced=balanced, causal=causal)
        assert torch.equal(out.view(torch.uint8), eager.view(torch.uint8))


def test_matmul_and_16bit_attention_replay(hb):
    g = torch.Generator().manual_seed(9)
    x = torch.randn(256, 512, generator=g).bfloat16().cuda()
    y = torch.randn(512, 384, generator=g).bfloat16().cuda()
    bias = torch.randn(384, generator=g).bfloat16().cuda()
    out = torch.zeros(256, 384, dtype=torch.bfloat16, device="cuda")
    graph = _capture(lambda: hb.matmul(x, y, bias=bias, relu=True, out=out))
    x.copy_(torch.randn(256, 512, generator=g).bfloat16())
    out.zero_()
    graph.replay()
    assert torch.equal(out, hb.matmul(x, y, bias=bias, relu=True))

    q = torch.randn(2, 2, 256, 64, generator=g).half().cuda()
    res = {}

    def run():
        res["out"] = hb.attention(q, q, q)

    graph = _capture(run)
    q.copy_(torch.randn(2, 2, 256, 64, generator=g).half())
    graph.replay()
    assert torch.equal(res["out"], hb.attention(q, q, q))
