"""``DropInKernel``: the slice of ``helion.runtime.kernel.Kernel`` that callers of the two FP8
examples touch, backed by the hand-written CUDA kernels instead of Helion's compiler.

What the reference's harness does with a kernel object (pytorch-labs/helion):
  * calls it                                               (helion/runtime/kernel.py:259-272)
  * pokes ``.settings.static_shapes / force_autotune / static_shape`` (helion/_testing.py:421-423,
    benchmarks/run.py:405-406)
  * ``.bind(args)`` -> bound object with ``.kernel.settings``, ``._config``,
    ``.config_spec.default_config()``, ``.to_triton_code(cfg)``, ``.compile_config(cfg)``
    (helion/_testing.py:313-332)
  * ``.reset()``, ``.configs``, ``.fn``, ``.autotune(args)``  (benchmarks/run.py:401; kernel.py:190-279)

There is no Triton here, so ``to_triton_code`` returns a description of the CUDA kernel and the
chosen tile configuration; the autotuner is replaced by the tile-config tables inside the library
(``hb200_describe_config`` prints them), so ``autotune`` just reports the table's choice.  Ref-eager mode (``HELION_INTERPRET=1``) is the reference's CPU interpreter; this
library has no CPU path and refuses to run in that mode rather than silently launching CUDA.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Optional, Sequence

import torch

from . import _lib


class ShimRefMode(str):
    """Value of ``settings.ref_mode``.  The reference's harness tests it with
    ``settings.ref_mode != RefMode.OFF`` (helion/runtime/ref_mode.py:41-43), where ``RefMode`` is an enum with
    the values "off" and "eager"; this string compares equal to the enum member of the same value (and to the
    member's name in either case), so that check works on these settings without importing helion."""

    def _same(self, other: Any) -> bool:
        value = getattr(other, "value", other)
        return isinstance(value, str) and value.lower() == self.lower()

    def __eq__(self, other: Any) -> bool:  # type: ignore[override]
        return self._same(other)

    def __ne__(self, other: Any) -> bool:  # type: ignore[override]
        return not self._same(other)

    def __hash__(self) -> int:
        return hash(self.lower())


@dataclass
class ShimSettings:
    """Mutable attribute bag with the names of ``helion.runtime.settings.Settings`` that the
    harness sets (helion/runtime/settings.py:71-98).  Only ``static_shapes`` has an effect here:
    the CUDA kernels always specialise on sizes and strides at launch, so both values behave the
    same."""

    static_shapes: bool = True
    static_shape: bool = True  # the attribute name benchmarks/run.py:406 writes
    force_autotune: bool = False
    use_default_config: bool = False
    print_output_code: bool = False
    ref_mode: Any = ShimRefMode("off")
    autotune_compile_timeout: int = 60
    extra: Dict[str, Any] = field(default_factory=dict)


class ShimConfig(dict):
    """Stands in for ``helion.Config``: a mapping of tuning knobs.  ``cfg_id`` selects a row of the
    library's tile-config table; Helion-style keys (``block_sizes``, ``num_warps``, ``num_stages``,
    ...) are accepted and kept for display, but do not steer the hand-written kernels."""

    @property
    def config(self) -> dict:
        return dict(self)


class _ConfigSpec:
    def __init__(self, kernel: "DropInKernel") -> None:
        self._kernel = kernel

    def default_config(self) -> ShimConfig:
        return ShimConfig(cfg_id=None)


def _ref_eager_requested() -> bool:
    return os.environ.get("HELION_INTERPRET", "0") == "1"


class BoundDropInKernel:
    """Counterpart of ``helion.runtime.kernel.BoundKernel`` (kernel.py:282-583)."""

    def __init__(self, kernel: "DropInKernel", args: Sequence[Any]) -> None:
        self.kernel = kernel
        self._args = tuple(args)
        self._config: Optional[ShimConfig] = kernel._fixed_config
        self.config_spec = _ConfigSpec(kernel)

    @property
    def settings(self) -> ShimSettings:
        return self.kernel.settings

    def _cfg_id(self, config: Optional[dict]) -> Optional[int]:
        if config is None:
            return None
        cfg_id = config.get("cfg_id") if isinstance(config, dict) else None
        return None if cfg_id is None else int(cfg_id)

    def to_triton_code(self, config: Optional[dict] = None) -> str:
        """There is no Triton source; return what runs instead."""
        cfg_id = self._cfg_id(config if config is not None else self._config)
        chosen = self.kernel._describe(self._args, cfg_id)
        return f"# {self.kernel.name}: hand-written sm_100a CUDA kernel ({_lib.LIB_NAME})\n# {chosen}\n"

    def compile_config(self, config: Optional[dict] = None, *, allow_print: bool = True) -> Callable[..., Any]:
        cfg_id = self._cfg_id(config)

        def run(*args: Any) -> Any:
            return self.kernel._launch(args, cfg_id)

        return run

    def set_config(self, config: Optional[dict]) -> None:
        self._config = ShimConfig(config) if config is not None else None

    def autotune(self, args: Sequence[Any], *, force: bool = False, **_: Any) -> ShimConfig:
        cfg = ShimConfig(cfg_id=self.kernel._select(args))
        self._config = cfg
        return cfg

    def __call__(self, *args: Any) -> Any:
        return self.kernel._launch(args, self._cfg_id(self._config))


class DropInKernel:
    """Callable with the surface of ``helion.runtime.kernel.Kernel`` (kernel.py:59-279)."""

    def __init__(
        self,
        fn: Callable[..., Any],
        launch: Callable[[Sequence[Any], Optional[int]], Any],
        select: Callable[[Sequence[Any]], Optional[int]],
        describe: Callable[[Sequence[Any], Optional[int]], str],
        *,
        config: Optional[dict] = None,
        static_shapes: bool = True,
    ) -> None:
        self.fn = fn  # the Python function whose semantics the CUDA kernel implements
        self.name = fn.__name__
        self.__name__ = fn.__name__
        self.__doc__ = fn.__doc__
        self.settings = ShimSettings(static_shapes=static_shapes, static_shape=static_shapes)
        self._fixed_config = ShimConfig(config) if config is not None else None
        self.configs = [self._fixed_config] if self._fixed_config is not None else []
        self._launch_fn = launch
        self._select = select
        self._describe = describe
        self._bound: Dict[Any, BoundDropInKernel] = {}

    # -- helion.Kernel protocol -----------------------------------------------------------------
    def bind(self, args: Sequence[Any]) -> BoundDropInKernel:
        key = tuple(
            (a.dtype, a.device.type, tuple(a.shape), tuple(a.stride())) if isinstance(a, torch.Tensor)
            else getattr(a, "__code__", a)  # a closure argument (an epilogue) is keyed by its code, not its identity
            for a in args
        )  # the reference's static-shape specialisation key, helion/runtime/kernel.py:656-665
        bound = self._bound.get(key)
        if bound is None:
            bound = BoundDropInKernel(self, args)
            self._bound[key] = bound
        return bound

    def autotune(self, args: Sequence[Any], *, force: bool = False, **kwargs: Any) -> ShimConfig:
        return self.bind(args).autotune(args, force=force, **kwargs)

    def reset(self) -> None:
        self._bound.clear()

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        if kwargs:  # keyword-only extensions (out_dtype, out, config, ...): same guard, no bind cache
            return self._launch(args, None, **kwargs)
        return self.bind(args)(*args)

    # -- internals ------------------------------------------------------------------------------
    def _launch(self, args: Sequence[Any], cfg_id: Optional[int], **kwargs: Any) -> Any:
        mode = getattr(self.settings.ref_mode, "value", self.settings.ref_mode)
        if _ref_eager_requested() or str(mode).upper().endswith("EAGER"):
            raise RuntimeError(
                f"{self.name}: ref-eager mode (HELION_INTERPRET=1) is the reference's CPU interpreter; "
                "helion_b200 has no CPU path and will not silently run CUDA under that flag"
            )
        return self._launch_fn(args, cfg_id, **kwargs)
