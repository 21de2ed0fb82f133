"""`QuantizationConfig`, the per-call options of `quantize()`.

Field names, defaults and string coercion follow the reference's dataclass
(src/fouroversix/quantize/config.py:7-58) so that existing call sites keep working.
"""

from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any

from fouroversix_b200.utils import DataType, QuantizeBackend, RoundStyle, ScaleRule

_ENUM_FIELDS = {"backend": QuantizeBackend, "dtype": DataType, "round_style": RoundStyle, "scale_rule": ScaleRule}


@dataclass
class QuantizationConfig:
    """Options for quantizing one tensor.

    backend: which implementation to use; `None` or `cuda` select this package's kernels.
    block_scale_2d: one scale per 16x16 block instead of 1x16, so that a weight and its
        transpose quantize to the same values (training).
    dtype: target format (`nvfp4` or `if4` here).
    kwargs: free-form extras (unused by the kernels, kept for interface parity).
    pseudo_quantize: return the dequantized high-precision tensor instead.
    rht: apply the 16-point randomised Hadamard transform to every block of 16 first.
    round_style: `nearest` (implemented) or stochastic variants (not implemented here).
    scale_rule: 4-versus-6 selection rule; default `mse`.
    transpose: quantize the transposed input (output is K-major for the other operand).
    """

    backend: QuantizeBackend | None = None
    block_scale_2d: bool = False
    dtype: DataType = DataType.nvfp4
    kwargs: dict[str, Any] = field(default_factory=dict)
    pseudo_quantize: bool = False
    rht: bool = False
    round_style: RoundStyle = RoundStyle.nearest
    scale_rule: ScaleRule = ScaleRule.mse
    transpose: bool = False

    def __post_init__(self) -> None:
        for f in fields(self):
            enum_cls = _ENUM_FIELDS.get(f.name)
            value = getattr(self, f.name)
            if enum_cls is not None and isinstance(value, str) and not isinstance(value, enum_cls):
                setattr(self, f.name, enum_cls(value))
