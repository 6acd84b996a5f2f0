"""fp16 / bf16 matmul with an epilogue behind the entry points of pytorch-labs/helion's ``examples/matmul.py``.

Same module-level names and positional signatures as the reference module (``matmul(x, y, epilogue)``,
``check``, ``matmul_tritonbench``, ``main``).  The kernel body is the hand-written sm_100a CUDA GEMM
of ``helion_b200`` (kind::f16 tensor-core instructions, fp32 accumulation).

The reference's ``epilogue`` is an arbitrary Python closure over the fp32 accumulator tile that its
compiler traces into the kernel (examples/matmul.py:32-55).  There is no compiler here; the closure
is *recognised* instead: it is called once on a recording stand-in for the accumulator, and must
turn out to be one of the epilogues the reference's own checks and benchmark wrapper use
(examples/matmul.py:92-117, 124-138): the identity, ``acc + bias[tile[1]]`` and
``relu(acc + bias[tile[1]])``.  Anything else raises ``NotImplementedError`` -- never a silent
fallback to PyTorch.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
from torch import Tensor

from helion_b200 import _lib
from helion_b200 import ops as _ops
from helion_b200.kernel import DropInKernel


class _Acc:
    """Stand-in for the fp32 accumulator tile: records ``+ vector`` and ``relu`` applied to it."""

    def __init__(self, bias: Optional[Tensor] = None, relu: bool = False) -> None:
        self.bias = bias
        self.relu = relu

    def _add(self, other):
        if self.relu or self.bias is not None or not isinstance(other, Tensor) or other.dim() != 1:
            raise NotImplementedError(
                "matmul epilogue: only `acc`, `acc + bias[tile[1]]` and `relu(acc + bias[tile[1]])` "
                "(bias a vector with one element per output column) are built into the CUDA kernel"
            )
        return _Acc(other, False)

    __add__ = _add
    __radd__ = _add

    def _unsupported(self, *_args):
        raise NotImplementedError(
            "matmul epilogue: only `acc`, `acc + bias[tile[1]]` and `relu(acc + bias[tile[1]])` are built into the CUDA kernel"
        )

    __mul__ = __rmul__ = __sub__ = __rsub__ = __truediv__ = __rtruediv__ = __neg__ = __pow__ = __matmul__ = _unsupported
    __getitem__ = _unsupported

    def __getattr__(self, name):  # tensor methods such as .relu(), .to(), .clamp() are not recorded
        raise NotImplementedError(f"matmul epilogue: `acc.{name}` is not built into the CUDA kernel")

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if func in (torch.relu, torch.nn.functional.relu, Tensor.relu) and len(args) == 1 and isinstance(args[0], _Acc):
            if args[0].relu:
                raise NotImplementedError("matmul epilogue: relu applied twice")
            return _Acc(args[0].bias, True)
        if func in (torch.add, Tensor.add, Tensor.__add__, Tensor.__radd__) and len(args) == 2 and not kwargs:
            acc, other = (args[0], args[1]) if isinstance(args[0], _Acc) else (args[1], args[0])
            return acc._add(other)
        raise NotImplementedError(f"matmul epilogue: {getattr(func, '__name__', func)} is not built into the CUDA kernel")


def _recognise(epilogue: Optional[Callable], n: int):
    """Returns (bias or None, relu) for a supported epilogue closure."""
    if epilogue is None:
        return None, False
    # tile[1] is the slice of output columns; the whole row of columns stands for every tile
    result = epilogue(_Acc(), (slice(None), slice(None)))
    if not isinstance(result, _Acc):
        raise NotImplementedError("matmul epilogue must return the (transformed) accumulator")
    if result.bias is not None and result.bias.shape[0] != n:
        raise ValueError(f"matmul epilogue: bias has {result.bias.shape[0]} elements, out has {n} columns")
    return result.bias, result.relu


def _matmul_spec(x: Tensor, y: Tensor, epilogue: Callable = lambda acc, tile: acc) -> Tensor:
    """out[m, n] = cast(epilogue(sum_k fp32(x[m, k] * y[k, n]))) for fp16 or bf16 x [m, k], y [k, n]."""
    raise NotImplementedError("specification only; the CUDA kernel implements it")


_matmul_spec.__name__ = "matmul"


def _split(args):
    x, y = args[0], args[1]
    epilogue = args[2] if len(args) > 2 else None
    return x, y, epilogue


def _launch(args, cfg_id, **kwargs):
    x, y, epilogue = _split(args)
    if "epilogue" in kwargs:
        epilogue = kwargs.pop("epilogue")
    bias, relu = _recognise(epilogue, y.shape[1])
    return _ops.matmul(x, y, bias=bias, relu=relu, config=cfg_id, **kwargs)


def _select(args):
    x, y, _ = _split(args)
    # the table row is chosen over the byte length of K, as for e4m3 operands
    return _lib.load().hb200_fp8_gemm_select_config(x.shape[0], y.shape[1], 2 * x.shape[1], int(y.stride(0) == 1), 0)


def _describe(args, cfg_id):
    if cfg_id is None:
        return "gemm table row chosen by the library for 16-bit operands (hb200_gemm_16bit, cfg_id = -1)"
    return _lib.describe_config(_lib.OP_GEMM, cfg_id)


#: Drop-in for the reference's ``matmul`` kernel object (examples/matmul.py:26-56).
matmul = DropInKernel(_matmul_spec, _launch, _select, _describe, static_shapes=True)


def check(m: int, k: int, n: int) -> None:
    """The three comparisons of the reference's check (examples/matmul.py:80-117) against PyTorch,
    with the reference harness's default tolerances (helion/_testing.py:341-405: rtol 1e-2, atol 1e-1)."""
    x = torch.randn([m, k], device="cuda", dtype=torch.float16)
    y = torch.randn([k, n], device="cuda", dtype=torch.float16)
    bias = torch.randn([n], device="cuda", dtype=torch.float16)
    torch.testing.assert_close(matmul(x, y), torch.matmul(x, y), rtol=1e-2, atol=1e-1)
    torch.testing.assert_close(
        matmul(x, y, lambda acc, tile: acc + bias[tile[1]]), torch.nn.functional.linear(x, y.T, bias), rtol=1e-2, atol=1e-1
    )

    def epilogue(acc: Tensor, tile) -> Tensor:
        return torch.relu(acc + bias[tile[1]])

    torch.testing.assert_close(matmul(x, y, epilogue), torch.relu(x @ y + bias), rtol=1e-2, atol=1e-1)
    print(f"matmul {m}x{k}x{n}: matches torch (plain, + bias, relu(+ bias))")


def matmul_tritonbench(a: Tensor, b: Tensor, bias: Optional[Tensor]) -> Callable[[], Tensor]:
    """Wrapper with the tritonbench operator signature (examples/matmul.py:124-138): the closure that
    is timed; ``bias`` may be None."""
    if bias is not None:
        return lambda: matmul(a, b, lambda acc, tile: acc + bias[tile[1]])
    return lambda: matmul(a, b)


def main() -> None:
    check(1024, 1024, 1024)


if __name__ == "__main__":
    main()
