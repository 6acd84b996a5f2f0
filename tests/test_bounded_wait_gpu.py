"""Failure behaviour of device-side waits, without faulting or hanging the GPU: a wait that nothing
will ever satisfy runs into its limit, the kernel returns normally, the host reads the status word,
and the context keeps working."""
from __future__ import annotations

import ctypes
import time

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_is_reported_and_the_context_survives(built_library):
    import helion_b200 as hb
    from helion_b200 import _lib
    from oracle import fp8_oracle as o

    lib = built_library
    _lib.reset_status(0)
    stream = torch.cuda.current_stream().cuda_stream
    t0 = time.perf_counter()
    assert lib.hb200_debug_wait_selftest(0, 200, stream) == 0
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert 0.15 < elapsed < 5.0  # the wait really lasted about its limit, and ended by itself

    site = ctypes.c_uint32(0)
    assert lib.hb200_read_status(0, ctypes.byref(site)) == _lib.ERR_TIMEOUT
    assert site.value >> 16 == 40  # the self-test's wait site
    with pytest.raises(_lib.DeviceWaitTimeout, match="site 40"):
        _lib.check_status(0)
    _lib.reset_status(0)
    _lib.check_status(0)

    # the same context still computes correctly afterwards
    x, y = o.gemm_inputs(256, 256, 256, seed=0)
    out = hb.fp8_gemm(x.cuda(), y.t().contiguous().cuda().t(), out_dtype=torch.float32)
    want = o.fp8_gemm(o.torch_fp8_to_bits(x), o.torch_fp8_to_bits(y), "fp32")
    np.testing.assert_allclose(out.cpu().numpy(), want, rtol=1e-5, atol=1e-4)
    _lib.check_status(0)


def test_selftest_rejects_long_limits(built_library):
    from helion_b200 import _lib

    assert built_library.hb200_debug_wait_selftest(0, 5000, None) == _lib.ERR_BAD_CONFIG
