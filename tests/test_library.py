"""The C-ABI library without a GPU: it builds, loads, exports every symbol the header declares,
and validates arguments before touching a device.  The Python host layer refuses CPU tensors."""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest
import torch

from helion_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "helion_b200.h"


def declared_symbols():
    text = HEADER.read_text()
    return sorted(set(re.findall(r"HB200_API[^;(]*?\b(hb200_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for required in ("hb200_fp8_gemm", "hb200_fp8_attention", "hb200_last_error", "hb200_read_status"):
        assert required in names
    assert set(names) == set(_lib.SIGNATURES), "ctypes signatures and header must list the same symbols"


def test_library_exports_every_declared_symbol(built_library):
    for name in declared_symbols():
        assert hasattr(built_library, name), f"{name} is declared in the header but not exported"
    assert built_library.hb200_version() == 1


def test_config_table_is_described(built_library):
    n = _lib.num_configs(_lib.OP_GEMM)
    assert n >= 3
    for i in range(n):
        assert f"gemm cfg {i}" in _lib.describe_config(_lib.OP_GEMM, i)
    assert _lib.num_configs(_lib.OP_ATTENTION) >= 1
    # split-K rows say how much scratch they need; the others need none
    lib = built_library
    assert lib.hb200_fp8_gemm_workspace_bytes(16, 14336, 4096, _lib.DT_BF16, 12) == 4 * 16 * 14336 * 4
    assert lib.hb200_fp8_gemm_workspace_bytes(8192, 8192, 8192, _lib.DT_BF16, -1) == 0
    assert lib.hb200_fp8_gemm_workspace_bytes(16, 14336, 4096, _lib.DT_BF16, -1) == 0  # automatic choice: no scratch
    assert lib.hb200_fp8_gemm_workspace_bytes(16, 14336, 4096, _lib.DT_BF16, 0) == 0
    with pytest.raises(ValueError):
        _lib.describe_config(_lib.OP_GEMM, 10_000)


def _gemm(lib, M, N, K, x_rs, x_cs, y_rs, y_cs, out_rs, dt=_lib.DT_FP16, x=256, y=512, out=1024):
    return lib.hb200_fp8_gemm(x, y, out, M, N, K, x_rs, x_cs, y_rs, y_cs, out_rs, dt, -1, None, 0, 0, None)


def test_gemm_argument_validation_needs_no_gpu(built_library):
    lib = built_library
    assert _gemm(lib, 128, 128, 100, 112, 1, 1, 112, 128) == _lib.ERR_BAD_SHAPE  # K % 16
    assert "multiple of 16" in _lib.last_error()
    assert _gemm(lib, 128, 100, 128, 128, 1, 1, 128, 104) == _lib.ERR_BAD_SHAPE  # N % 8
    assert _gemm(lib, 0, 128, 128, 128, 1, 1, 128, 128) == _lib.ERR_BAD_SHAPE
    assert _gemm(lib, 128, 128, 128, 1, 128, 1, 128, 128) == _lib.ERR_BAD_STRIDE  # x column-major
    assert _gemm(lib, 128, 128, 128, 128, 1, 2, 256, 128) == _lib.ERR_BAD_STRIDE  # y neither layout
    assert _gemm(lib, 128, 128, 128, 128, 1, 1, 128, 128, dt=_lib.DT_E4M3) == _lib.ERR_BAD_DTYPE
    assert _gemm(lib, 128, 128, 128, 128, 1, 1, 128, 128, x=260) == _lib.ERR_ALIGN
    assert _gemm(lib, 128, 128, 128, 128, 1, 1, 128, 128, x=None) == _lib.ERR_ALIGN
    assert _gemm(lib, 128, 128, 128, 128, 1, 1, 128, 64) == _lib.ERR_BAD_STRIDE  # out rows overlap


def test_attention_argument_validation_needs_no_gpu(built_library):
    lib = built_library
    arr = ctypes.c_int64 * 3

    def call(BH=2, S=128, D=64, q=(8192, 64, 1), k=(8192, 64, 1), v=(8192, 1, 64), o=(8192, 64, 1), dt=_lib.DT_E4M3):
        return lib.hb200_fp8_attention(256, 512, 1024, 2048, BH, S, D, arr(*q), arr(*k), arr(*v), arr(*o),
                                       0.18, dt, -1, 0, None)

    assert call(D=96) == _lib.ERR_BAD_SHAPE
    assert "head_dim" in _lib.last_error()
    assert call(S=0) == _lib.ERR_BAD_SHAPE
    assert call(S=100, v=(6400, 100, 1)) == _lib.ERR_BAD_STRIDE  # key-contiguous v with unaligned rows
    assert call(dt=_lib.DT_FP16) == _lib.ERR_BAD_DTYPE
    assert call(q=(8192, 1, 128)) == _lib.ERR_BAD_STRIDE
    assert call(v=(8192, 2, 128)) == _lib.ERR_BAD_STRIDE


def test_error_codes_map_to_python_exceptions(built_library):
    _gemm(built_library, 128, 128, 100, 112, 1, 1, 112, 128)
    with pytest.raises(ValueError, match="multiple of 16"):
        _lib.raise_for(_lib.ERR_BAD_SHAPE, "fp8_gemm")
    with pytest.raises(TypeError):
        _lib.raise_for(_lib.ERR_BAD_DTYPE, "x")
    with pytest.raises(_lib.DeviceWaitTimeout):
        _lib.raise_for(_lib.ERR_TIMEOUT, "x")
    with pytest.raises(RuntimeError):
        _lib.raise_for(_lib.ERR_CUDA, "x")
    _lib.raise_for(0, "x")


def test_select_config_prefers_wide_tiles_for_big_problems(built_library):
    lib = built_library
    big = lib.hb200_fp8_gemm_select_config(8192, 8192, 8192, 1, _lib.DT_BF16)
    assert "256x256" in _lib.describe_config(_lib.OP_GEMM, big) or "128x256" in _lib.describe_config(_lib.OP_GEMM, big)
    small = lib.hb200_fp8_gemm_select_config(256, 256, 256, 1, _lib.DT_FP16)
    assert 0 <= small < _lib.num_configs(_lib.OP_GEMM)
    # 128x64 tiles are only built for column-major y
    assert lib.hb200_fp8_gemm_select_config(128, 2048, 256, 0, _lib.DT_FP16) in (0, 1)
    # row shards of the 8192^3 problem: 37 column blocks of 224 give every CTA pair a tile where 32 blocks of
    # 256 leave pairs idle; the whole problem keeps the wider tile (7 rounds against 8); row-major y has no 224 row
    for rows in (1024, 2048, 4096):
        assert "512x224" in _lib.describe_config(_lib.OP_GEMM, lib.hb200_fp8_gemm_select_config(rows, 8192, 8192, 1, _lib.DT_BF16))
        assert "512x224" not in _lib.describe_config(_lib.OP_GEMM, lib.hb200_fp8_gemm_select_config(rows, 8192, 8192, 0, _lib.DT_BF16))
    assert "512x256" in _lib.describe_config(_lib.OP_GEMM, big)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setenv("HB200_LIB", str(tmp_path / "nope.so"))
    monkeypatch.setattr(_lib, "_lib", None)
    with pytest.raises(_lib.LibraryNotBuiltError, match="no CPU or Triton fallback"):
        _lib.load()


def test_ops_refuse_cpu_tensors():
    import helion_b200 as hb

    x = torch.zeros(16, 16).to(torch.float8_e4m3fn)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        hb.fp8_gemm(x, x)
    q = torch.zeros(2, 16, 64).to(torch.float8_e4m3fn)
    v = torch.zeros(2, 64, 16).to(torch.float8_e4m3fn)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        hb.fp8_attention(q, q, v, 1, 2)


def test_ops_check_dtypes_and_shapes_like_the_reference():
    import helion_b200 as hb

    x = torch.zeros(16, 16).to(torch.float8_e4m3fn)
    with pytest.raises(TypeError):
        hb.fp8_gemm(torch.zeros(16, 16), x)
    with pytest.raises(AssertionError, match="size mismatch 16 != 32"):
        hb.fp8_gemm(x, torch.zeros(32, 16).to(torch.float8_e4m3fn))
    with pytest.raises(TypeError):
        hb.fp8_gemm(x, x, out_dtype=torch.int8)
    q = torch.zeros(2, 16, 64).to(torch.float8_e4m3fn)
    with pytest.raises(ValueError, match="shape mismatch"):
        hb.fp8_attention(q, q, q, 1, 2)
    v = torch.zeros(2, 64, 16).to(torch.float8_e4m3fn)
    with pytest.raises(ValueError, match="batch\\*heads"):
        hb.fp8_attention(q, q, v, 3, 2)


def test_sweep_tool_needs_a_gpu_and_knows_the_benchmark_shapes():
    """The table sweep is a GPU tool: without a device it says so and exits 2 (no CPU path)."""
    import torch

    from helion_b200 import sweep

    assert (8192, 8192, 8192) in sweep.GEMM_SHAPES and (16, 14336, 4096) in sweep.GEMM_SHAPES
    assert (4, 48, 1024, 64) in sweep.ATTN_SHAPES and (8, 32, 4096, 128) in sweep.ATTN_SHAPES
    if not torch.cuda.is_available():
        assert sweep.main(["--op", "gemm"]) == 2
