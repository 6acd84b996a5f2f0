"""helion_b200: B200-native (sm_100a) FP8 GEMM and FP8 attention behind Helion's example signatures.

Public surface:
    fp8_gemm, fp8_attention         -- operators on torch CUDA tensors (helion_b200.ops)
    preprocess_fp8_attention_inputs -- q, k, v -> e4m3 in one kernel, with the reference's views
    HostGemm                        -- fp8_gemm on pinned host buffers with overlapped PCIe copies
    matmul                          -- fp16 / bf16 sibling of fp8_gemm with the bias / ReLU epilogues
    attention                       -- fp16 / bf16 sibling of fp8_attention (examples/attention.py)
    DropInKernel                    -- object with the protocol of helion.runtime.kernel.Kernel
                                       that the reference's test and benchmark harness touch
There is no CPU, Triton or PyTorch fallback: calls fail loudly when the CUDA library is missing.
"""
from __future__ import annotations

from ._lib import DeviceWaitTimeout, LibraryNotBuiltError
from .host_io import HostGemm
from .ops import attention, attention_into, fp8_attention, fp8_gemm, matmul, preprocess_fp8_attention_inputs

__all__ = [
    "fp8_gemm",
    "fp8_attention",
    "attention_into",
    "preprocess_fp8_attention_inputs",
    "HostGemm",
    "matmul",
    "attention",
    "DeviceWaitTimeout",
    "LibraryNotBuiltError",
]
