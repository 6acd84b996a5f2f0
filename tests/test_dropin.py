"""The drop-in boundary: the example modules keep the reference's names and positional
signatures, and the kernel objects answer the protocol the reference's harness uses."""
from __future__ import annotations

import inspect

import pytest
import torch

import examples.fp8_attention as attn_mod
import examples.fp8_gemm as gemm_mod
from helion_b200.kernel import BoundDropInKernel, DropInKernel


def params(fn):
    return list(inspect.signature(fn).parameters)


def test_module_level_names_of_the_reference_exist():
    for name in ("fp8_gemm", "reference_fp8_gemm_pytorch", "fp8_gemm_tritonbench", "check", "main"):
        assert hasattr(gemm_mod, name)
    for name in ("fp8_attention_kernel", "preprocess_fp8_attention_inputs", "fp8_attention_tritonbench",
                 "fp8_attention_pytorch", "check", "main"):
        assert hasattr(attn_mod, name)


def test_positional_signatures_match_the_reference():
    assert params(gemm_mod.fp8_gemm.fn) == ["x", "y"]
    assert params(gemm_mod.fp8_gemm_tritonbench) == ["a", "b"]
    assert params(gemm_mod.reference_fp8_gemm_pytorch) == ["x_fp8", "y_fp8"]
    assert params(gemm_mod.check) == ["m", "k", "n"]
    assert params(attn_mod.fp8_attention_kernel.fn) == ["q", "k", "v", "batch", "heads"]
    assert params(attn_mod.preprocess_fp8_attention_inputs) == ["q", "k", "v"]
    assert params(attn_mod.fp8_attention_tritonbench) == ["q", "k", "v"]
    assert params(attn_mod.check) == ["batch", "heads", "seq_len", "head_dim"]


def test_kernel_objects_answer_the_harness_protocol(built_library):
    k = gemm_mod.fp8_gemm
    assert isinstance(k, DropInKernel) and callable(k)
    k.settings.static_shapes = False  # helion/_testing.py:421-423 writes this
    k.settings.force_autotune = True  # benchmarks/run.py:405
    k.settings.static_shape = True
    args = (torch.zeros(256, 128).to(torch.float8_e4m3fn), torch.zeros(128, 512).to(torch.float8_e4m3fn))
    bound = k.bind(args)
    assert isinstance(bound, BoundDropInKernel)
    assert bound.kernel.settings is k.settings
    assert k.bind(args) is bound  # cached on (dtype, device, sizes, strides)
    assert k.bind((args[0], args[1].t().contiguous().t())) is not bound  # strides are part of the key
    cfg = bound.config_spec.default_config()
    text = bound.to_triton_code(cfg)
    assert "sm_100a" in text and "gemm cfg" in text
    assert callable(bound.compile_config(cfg))
    assert "cfg_id" in k.autotune(args)
    k.reset()
    assert k.bind(args) is not bound
    assert k.configs == []


def test_preprocess_keeps_the_reference_stride_trap():
    q = torch.randn(2, 3, 32, 64)
    q8, k8, v8 = attn_mod.preprocess_fp8_attention_inputs(q, q, q)
    assert q8.shape == (6, 32, 64) and v8.shape == (6, 64, 32)
    assert v8.stride() == (32 * 64, 1, 64)  # logical [BH, D, S] over physical [BH, S, D]
    assert q8.dtype == v8.dtype == torch.float8_e4m3fn


def test_ref_eager_flag_is_refused(monkeypatch):
    monkeypatch.setenv("HELION_INTERPRET", "1")
    x = torch.zeros(16, 16).to(torch.float8_e4m3fn)
    with pytest.raises(RuntimeError, match="no CPU path"):
        gemm_mod.fp8_gemm(x, x)


def test_calls_without_a_gpu_fail_loudly():
    x = torch.zeros(16, 16).to(torch.float8_e4m3fn)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        gemm_mod.fp8_gemm_tritonbench(x, x)


def test_matmul_epilogue_recognition_needs_no_gpu():
    """examples/matmul.py recognises the reference's three epilogues (examples/matmul.py:92-117) by
    running the closure on a recording stand-in; everything else must raise instead of falling back."""
    import torch

    import examples.matmul as mod

    bias = torch.arange(8, dtype=torch.float16)
    assert mod._recognise(None, 8) == (None, False)
    assert mod._recognise(lambda acc, tile: acc, 8) == (None, False)
    b, relu = mod._recognise(lambda acc, tile: acc + bias[tile[1]], 8)
    assert torch.equal(b, bias) and relu is False
    b, relu = mod._recognise(lambda acc, tile: torch.relu(bias[tile[1]] + acc), 8)
    assert torch.equal(b, bias) and relu is True
    b, relu = mod._recognise(lambda acc, tile: torch.nn.functional.relu(acc), 8)
    assert b is None and relu is True
    for bad in (lambda acc, tile: acc * 2, lambda acc, tile: torch.tanh(acc), lambda acc, tile: torch.relu(acc) + bias,
                lambda acc, tile: acc + bias.reshape(1, 8), lambda acc, tile: bias):
        with pytest.raises(NotImplementedError):
            mod._recognise(bad, 8)
    with pytest.raises(ValueError, match="bias has"):
        mod._recognise(lambda acc, tile: acc + bias[:4], 8)


def test_sibling_example_modules_expose_the_reference_names():
    """examples/matmul.py and examples/attention.py of the reference: the names benchmarks/run.py and the
    examples' own main() use must exist here with a Kernel-like object behind them."""
    import examples.attention as attn
    import examples.matmul as mm
    from helion_b200.kernel import DropInKernel

    for mod, names in ((mm, ("matmul", "matmul_tritonbench", "check", "main")),
                       (attn, ("attention", "attention_dynamic", "test", "main"))):
        for name in names:
            assert hasattr(mod, name), f"{mod.__name__}.{name}"
    for k in (mm.matmul, attn.attention, attn.attention_dynamic):
        assert isinstance(k, DropInKernel) and callable(k) and hasattr(k, "bind") and hasattr(k, "settings")
    assert attn.attention_dynamic.settings.static_shapes is False and attn.attention.settings.static_shapes is True
