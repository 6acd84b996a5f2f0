"""ctypes binding of the C-ABI library declared in ``include/helion_b200.h``.

There is no fallback: if the shared library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

LIB_NAME = "libhelion_b200.so"
_LIB_PATH = Path(__file__).resolve().parent / "_C" / LIB_NAME

# error codes (include/helion_b200.h)
OK = 0
ERR_BAD_DTYPE = -1
ERR_BAD_SHAPE = -2
ERR_BAD_STRIDE = -3
ERR_ALIGN = -4
ERR_UNSUPPORTED_ARCH = -5
ERR_CUDA = -6
ERR_TIMEOUT = -7
ERR_BAD_CONFIG = -8
ERR_WORKSPACE = -9

DT_FP16, DT_BF16, DT_FP32, DT_E4M3 = 0, 1, 2, 3
OP_GEMM, OP_ATTENTION = 0, 1
STATIC_SCRATCH_BYTES = 4 << 20
ATTN_WORKSPACE_BYTES = 16
SCALE_NONE, SCALE_TENSOR, SCALE_ROWWISE = 0, 1, 2

# Every symbol the header declares, with (restype, argtypes).
_i64 = ctypes.c_int64
_vp = ctypes.c_void_p
_i64x3 = ctypes.POINTER(ctypes.c_int64)
SIGNATURES = {
    "hb200_fp8_gemm": (
        ctypes.c_int,
        [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, ctypes.c_int, ctypes.c_int, _vp,
         ctypes.c_size_t, ctypes.c_int, _vp],
    ),
    "hb200_fp8_gemm_scaled": (
        ctypes.c_int,
        [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, ctypes.c_int, _vp, _vp, ctypes.c_int,
         ctypes.c_int, _vp, ctypes.c_size_t, ctypes.c_int, _vp],
    ),
    "hb200_gemm_16bit": (
        ctypes.c_int,
        [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, ctypes.c_int, ctypes.c_int, _vp, ctypes.c_int,
         ctypes.c_int, ctypes.c_int, _vp],
    ),
    "hb200_fp8_gemm_splitk_static": (
        ctypes.c_int,
        [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, ctypes.c_int, ctypes.c_int, ctypes.c_int, _vp],
    ),
    "hb200_fp8_gemm_workspace_bytes": (ctypes.c_size_t, [_i64, _i64, _i64, ctypes.c_int, ctypes.c_int]),
    "hb200_fp8_gemm_select_config": (ctypes.c_int, [_i64, _i64, _i64, ctypes.c_int, ctypes.c_int]),
    "hb200_fp8_attention": (
        ctypes.c_int,
        [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64x3, _i64x3, _i64x3, _i64x3, ctypes.c_float, ctypes.c_int,
         ctypes.c_int, ctypes.c_int, _vp],
    ),
    "hb200_fp8_attention_ex": (
        ctypes.c_int,
        [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64x3, _i64x3, _i64x3, _i64x3, ctypes.c_float, ctypes.c_int,
         ctypes.c_int, ctypes.c_int, _vp, ctypes.c_size_t, ctypes.c_int, _vp],
    ),
    "hb200_attention_16bit": (
        ctypes.c_int,
        [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64x3, _i64x3, _i64x3, _i64x3, ctypes.c_float, ctypes.c_int,
         ctypes.c_int, _vp, ctypes.c_size_t, ctypes.c_int, _vp],
    ),
    "hb200_fp8_attention_preprocess": (
        ctypes.c_int,
        [_vp, _vp, _vp, _vp, _vp, _vp, _i64, ctypes.c_int, ctypes.c_int, _vp],
    ),
    "hb200_fp8_attention_ws": (
        ctypes.c_int,
        [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64x3, _i64x3, _i64x3, _i64x3, ctypes.c_float, ctypes.c_int,
         ctypes.c_int, _vp, ctypes.c_size_t, ctypes.c_int, _vp],
    ),
    "hb200_debug_softmax_ceiling": (
        ctypes.c_int,
        [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, _vp, ctypes.c_int, _vp],
    ),
    "hb200_debug_wait_selftest": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, _vp]),
    "hb200_num_configs": (ctypes.c_int, [ctypes.c_int]),
    "hb200_describe_config": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_char_p, ctypes.c_int]),
    "hb200_read_status": (ctypes.c_int, [ctypes.c_int, ctypes.POINTER(ctypes.c_uint32)]),
    "hb200_reset_status": (ctypes.c_int, [ctypes.c_int]),
    "hb200_num_sms": (ctypes.c_int, [ctypes.c_int]),
    "hb200_last_error": (ctypes.c_char_p, []),
    "hb200_version": (ctypes.c_int, []),
}


class LibraryNotBuiltError(RuntimeError):
    pass


class DeviceWaitTimeout(RuntimeError):
    """A bounded device-side wait ran out; the kernel returned early and its output is invalid."""


_lock = threading.Lock()
_lib = None


def lib_path() -> Path:
    return Path(os.environ.get("HB200_LIB", str(_LIB_PATH)))


def load() -> ctypes.CDLL:
    """Load the shared library (once) and declare every entry point's signature."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = lib_path()
        if not path.exists():
            raise LibraryNotBuiltError(
                f"{path} not found: build the CUDA library first (python -m helion_b200.build); "
                "there is no CPU or Triton fallback"
            )
        lib = ctypes.CDLL(str(path))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def last_error() -> str:
    msg = load().hb200_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def raise_for(code: int, what: str) -> None:
    """Map a negative return code to the exception type the reference would raise."""
    if code >= 0:
        return
    text = f"{what}: {last_error()} (code {code})"
    if code == ERR_BAD_DTYPE:
        raise TypeError(text)
    if code in (ERR_BAD_SHAPE, ERR_BAD_STRIDE, ERR_ALIGN, ERR_BAD_CONFIG, ERR_WORKSPACE):
        raise ValueError(text)
    if code == ERR_TIMEOUT:
        raise DeviceWaitTimeout(text)
    raise RuntimeError(text)


def check_status(device: int) -> None:
    """Raise DeviceWaitTimeout if a kernel on ``device`` recorded a wait that ran out."""
    site = ctypes.c_uint32(0)
    code = load().hb200_read_status(device, ctypes.byref(site))
    raise_for(code, "device status")


def reset_status(device: int) -> None:
    raise_for(load().hb200_reset_status(device), "reset status")


def describe_config(op: int, cfg_id: int) -> str:
    buf = ctypes.create_string_buffer(256)
    n = load().hb200_describe_config(op, cfg_id, buf, 256)
    raise_for(n, "describe_config")
    return buf.value.decode()


def num_configs(op: int) -> int:
    return load().hb200_num_configs(op)
