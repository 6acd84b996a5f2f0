"""The allocation-free split-K GEMM entry point (``hb200_fp8_gemm_splitk_static``).

Some callers of this library cannot allocate device memory around a GEMM: a serving loop that
handed out all of its device memory at start-up, an operator hook running inside another runtime
that owns the allocator, a host callback where the device-wide synchronisation an allocation may
cause would stall unrelated streams.  For them the library offers one split-K entry point whose
scratch (the fp32 partial sums) is a fixed 4 MiB array compiled into the library, so the call itself
never allocates.  This test calls it through the C ABI, twice in a row (the second call reuses the
array with the first call's contents still in it), and compares each result with the ordinary entry
point running the same split-K row of the table on a caller-provided workspace.  Both paths run the
same two kernels, so the results must be identical, not merely close.

Collected last on purpose (file name): a run that stops at the first failure has then already run
every other test.
"""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(lib, _lib, x, y, out, splits):
    m, k = x.shape
    n = y.shape[1]
    code = lib.hb200_fp8_gemm_splitk_static(
        x.data_ptr(), y.data_ptr(), out.data_ptr(), m, n, k,
        x.stride(0), x.stride(1), y.stride(0), y.stride(1), out.stride(0),
        {torch.float16: _lib.DT_FP16, torch.bfloat16: _lib.DT_BF16, torch.float32: _lib.DT_FP32}[out.dtype],
        splits, 0, torch.cuda.current_stream().cuda_stream,
    )
    return code


def test_static_scratch_split_k_matches_the_workspace_path(built_library):
    import helion_b200 as hb
    from helion_b200 import _lib
    from oracle import fp8_oracle as o

    lib = built_library
    dev = torch.device("cuda:0")
    cases = [
        # (M, N, K, splits, table row with the same split factor, y column-major?)
        (16, 14336, 4096, 4, 12, True),   # the skinny MLP shape: 4 * 16 * 14336 * 4 B = 3.5 MiB of scratch
        (100, 272, 1152, 2, 11, False),   # ragged rows, row-major y, a different part of the array in use
    ]
    for m, n, k, splits, row, colmajor in cases:
        x, y = o.gemm_inputs(m, n, k, seed=500 + m)
        xd = x.to(dev)
        yd = y.t().contiguous().to(dev).t() if colmajor else y.contiguous().to(dev)
        for out_dtype in (torch.bfloat16, torch.float32):
            # the allocation-free calls come first: in a fresh process the very first of them also
            # performs the per-device set-up (address look-up of the static array)
            results = []
            for attempt in range(2):
                got = torch.full((m, n), float("nan"), dtype=out_dtype, device=dev)
                torch.cuda.synchronize()
                free_before, held_before = torch.cuda.mem_get_info(dev)[0], torch.cuda.memory_allocated(dev)
                code = _call_static(lib, _lib, xd, yd, got, splits)
                assert code == 0, _lib.last_error()
                torch.cuda.synchronize()
                if attempt == 1:
                    # the warmed-up call takes no device memory, neither from the driver nor from torch's pool
                    assert torch.cuda.mem_get_info(dev)[0] == free_before
                    assert torch.cuda.memory_allocated(dev) == held_before
                results.append(got)
            want = hb.fp8_gemm(xd, yd, out_dtype=out_dtype, config=row)  # allocates its workspace through torch
            for attempt, got in enumerate(results):
                assert torch.equal(got, want), f"call {attempt} differs for {m}x{n}x{k} {out_dtype}"
            # and the values are right, not just equal: the stated GEMM tolerance against the oracle
            ref = o.fp8_gemm(o.torch_fp8_to_bits(x), o.torch_fp8_to_bits(y),
                             "bf16" if out_dtype == torch.bfloat16 else "fp32")
            torch.testing.assert_close(got.float().cpu(), torch.from_numpy(ref), rtol=2e-2, atol=2e-2)
    # Waits that ran out in the static calls are recorded from the moment the device context exists (the
    # hb.fp8_gemm call above creates it in a fresh process), so this covers every static call after the first pair.
    _lib.check_status(0)


def test_static_scratch_rejects_what_does_not_fit(built_library):
    from helion_b200 import _lib

    lib = built_library
    dev = torch.device("cuda:0")
    x = torch.zeros(128, 4096, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    y = torch.zeros(14336, 4096, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn).t()
    out = torch.empty(128, 14336, dtype=torch.bfloat16, device=dev)
    # 4 * 128 * 14336 * 4 B = 28 MiB: beyond the 4 MiB array
    assert _call_static(lib, _lib, x, y, out, 4) == _lib.ERR_WORKSPACE
    assert "exceeds the static scratch" in _lib.last_error()
    assert _call_static(lib, _lib, x[:16], y, out[:16], 1) == _lib.ERR_BAD_CONFIG  # not a split
    assert _call_static(lib, _lib, x[:16, :128], y[:128], out[:16], 2) == _lib.ERR_BAD_CONFIG  # K too short to split
    assert 4 * 16 * 14336 * 4 <= _lib.STATIC_SCRATCH_BYTES
