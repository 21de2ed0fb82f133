"""Module registry and `quantize_model()`.

`QuantizedModule.register(nn.Linear)` maps a high-precision module class to its
quantized replacement; `quantize_model` walks a model and swaps every registered
module in place (reference: src/fouroversix/model/quantize.py:13-127).
"""

from __future__ import annotations

from collections.abc import Callable
from typing import Any, ClassVar

import torch.nn as nn

from .config import ModelQuantizationConfig


class QuantizedModule:
    """Registry of quantized replacements, keyed by the class they replace."""

    _registry: ClassVar[dict[type[nn.Module], type[nn.Module]]] = {}
    _should_replace_existing_modules_in_model: ClassVar[dict[type[nn.Module], bool]] = {}

    @classmethod
    def is_quantized_module_type(cls, module_type: type[nn.Module]) -> bool:
        return module_type in cls._registry.values()

    @classmethod
    def get_cls(cls, high_precision_cls: type[nn.Module]) -> type[nn.Module] | None:
        return cls._registry.get(high_precision_cls)

    @classmethod
    def should_replace_existing_modules_in_model(cls, module_type: type[nn.Module]) -> bool:
        return cls._should_replace_existing_modules_in_model.get(module_type, False)

    @classmethod
    def register(
        cls,
        high_precision_cls: type[nn.Module],
        *,
        replace_existing_modules_in_registry: bool = False,
        replace_existing_modules_in_model: bool = True,
    ) -> Callable[[type[nn.Module]], type[nn.Module]]:
        """Class decorator: the decorated class replaces `high_precision_cls`.

        Registering a class twice, or a subclass of a registered class, is an error
        unless `replace_existing_modules_in_registry` is set, in which case the older
        entries are dropped.
        """
        if high_precision_cls in cls._registry and not replace_existing_modules_in_registry:
            raise ValueError(f"High-precision module {high_precision_cls} is already registered.")
        shadowed = [known for known in cls._registry
                    if high_precision_cls is not None and issubclass(high_precision_cls, known)]
        if shadowed and not replace_existing_modules_in_registry:
            raise TypeError(f"High-precision module {high_precision_cls} is a subclass of "
                            f"{shadowed[0]}, which is already registered.")
        for known in shadowed:
            del cls._registry[known]

        def decorate(wrapped: type[nn.Module]) -> type[nn.Module]:
            cls._registry[high_precision_cls] = wrapped
            cls._should_replace_existing_modules_in_model[high_precision_cls] = replace_existing_modules_in_model
            return wrapped

        return decorate


def quantize_model(model: nn.Module, config: ModelQuantizationConfig | None = None, **kwargs: Any) -> None:
    """Replace, in place, every registered module of `model` that is not excluded by
    `config.modules_to_not_convert` (default: `lm_head`).  `config` defaults to
    `ModelQuantizationConfig()`: NVFP4 weights and activations with 4/6 MSE selection."""
    config = config or ModelQuantizationConfig()
    targets = []
    for name, module in model.named_modules():
        if not name or name in config.modules_to_not_convert:
            continue
        replacement = QuantizedModule.get_cls(type(module))
        if replacement is None or not QuantizedModule.should_replace_existing_modules_in_model(type(module)):
            continue
        targets.append((name, module, replacement))
    for name, module, replacement in targets:
        model.set_submodule(name, replacement(module, config.get_module_config(name), **kwargs))
