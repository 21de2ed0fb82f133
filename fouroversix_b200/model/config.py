"""Per-module and per-model quantization settings.

Field names and defaults follow the reference (src/fouroversix/model/config.py:16-272)
so existing configuration dictionaries load unchanged. Unset per-tensor fields inherit
`dtype` / `scale_rule`.
"""

from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass, field, fields
from typing import Any

from fouroversix_b200.quantize import QuantizationConfig
from fouroversix_b200.utils import DataType, MatmulBackend, QuantizeBackend, RoundStyle, ScaleRule

_COERCE = {
    "activation_dtype": DataType, "activation_round_style": RoundStyle, "activation_scale_rule": ScaleRule,
    "dtype": DataType, "gradient_dtype": DataType, "gradient_round_style": RoundStyle,
    "gradient_scale_rule": ScaleRule, "matmul_backend": MatmulBackend, "output_dtype": DataType,
    "quantize_backend": QuantizeBackend, "quartet_ii_dtype": DataType, "scale_rule": ScaleRule,
    "weight_dtype": DataType, "weight_round_style": RoundStyle, "weight_scale_rule": ScaleRule,
}


@dataclass
class ModuleQuantizationConfig:
    """How one module quantizes its activations, weights and gradients.

    `*_dtype` / `*_scale_rule` default to `dtype` / `scale_rule`.  `keep_master_weights`
    keeps the high-precision weight and re-quantizes it every step (training);
    otherwise the module stores packed buffers only.  `weight_scale_2d` uses 16x16
    weight blocks so W and W^T agree.  `disable_*_quantization` run that matmul in high
    precision.  `pseudo_quantize` replaces FP4 matmuls by fake-quantized high-precision
    ones.  The Quartet-II fields are accepted for compatibility and not acted on.
    """

    activation_dtype: DataType | None = None
    activation_round_style: RoundStyle = RoundStyle.nearest
    activation_scale_rule: ScaleRule | None = None
    disable_dgrad_quantization: bool = False
    disable_fprop_quantization: bool = False
    disable_wgrad_quantization: bool = False
    dtype: DataType = DataType.nvfp4
    gradient_dtype: DataType | None = None
    gradient_round_style: RoundStyle = RoundStyle.stochastic
    gradient_scale_rule: ScaleRule | None = None
    keep_master_weights: bool = False
    matmul_backend: MatmulBackend | None = None
    output_dtype: DataType = DataType.bfloat16
    pseudo_quantize: bool = False
    quantize_backend: QuantizeBackend | None = None
    quartet_ii_dtype: DataType | None = None
    quartet_ii_rerotate_had: bool = False
    scale_rule: ScaleRule = ScaleRule.mse
    weight_dtype: DataType | None = None
    weight_round_style: RoundStyle = RoundStyle.nearest
    weight_scale_2d: bool = False
    weight_scale_rule: ScaleRule | None = None
    wgrad_nvint4: bool = False

    def __post_init__(self) -> None:
        for name, enum_cls in _COERCE.items():
            value = getattr(self, name)
            if isinstance(value, str) and not isinstance(value, enum_cls):
                setattr(self, name, enum_cls(value))
        for role in ("activation", "gradient", "weight"):
            if getattr(self, f"{role}_dtype") is None:
                setattr(self, f"{role}_dtype", self.dtype)
            if getattr(self, f"{role}_scale_rule") is None:
                setattr(self, f"{role}_scale_rule", self.scale_rule)

    def _tensor_config(self, role: str, extra: dict[str, Any]) -> QuantizationConfig:
        base = {
            "backend": self.quantize_backend,
            "dtype": getattr(self, f"{role}_dtype"),
            "pseudo_quantize": self.pseudo_quantize,
            "round_style": getattr(self, f"{role}_round_style"),
            "scale_rule": getattr(self, f"{role}_scale_rule"),
        }
        if role == "weight":
            base["block_scale_2d"] = self.weight_scale_2d
        base.update(extra)
        return QuantizationConfig(**base)

    def get_activation_config(self, **kwargs: Any) -> QuantizationConfig:
        return self._tensor_config("activation", kwargs)

    def get_gradient_config(self, **kwargs: Any) -> QuantizationConfig:
        return self._tensor_config("gradient", kwargs)

    def get_weight_config(self, **kwargs: Any) -> QuantizationConfig:
        return self._tensor_config("weight", kwargs)


@dataclass
class ModelQuantizationConfig(ModuleQuantizationConfig):
    """Model-wide settings plus per-module overrides and an exclusion list."""

    module_config_overrides: dict[str, ModuleQuantizationConfig] = field(default_factory=dict)
    modules_to_not_convert: list[str] = field(default_factory=lambda: ["lm_head"])

    def __post_init__(self) -> None:
        super().__post_init__()
        if self.module_config_overrides:
            self.module_config_overrides = {
                name: ModuleQuantizationConfig(**cfg) if isinstance(cfg, dict) else cfg
                for name, cfg in self.module_config_overrides.items()
            }

    def get_module_config(self, module_name: str) -> ModuleQuantizationConfig:
        if not self.module_config_overrides:
            return self
        return self.module_config_overrides.get(module_name, self)

    def __hash__(self) -> str:  # the reference returns the hex digest, kept for parity
        def plain(v):
            if isinstance(v, dict):
                return {k: plain(x) for k, x in v.items()}
            if isinstance(v, ModuleQuantizationConfig):
                return {f.name: plain(getattr(v, f.name)) for f in fields(v)}
            return getattr(v, "value", v)

        payload = {f.name: plain(getattr(self, f.name)) for f in fields(self)}
        return hashlib.sha256(json.dumps(payload, sort_keys=True).encode()).hexdigest()
