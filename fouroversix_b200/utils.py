"""Enumerations of the public API: data types, scale rules, rounding styles, back ends.

Names and string values are those of the reference's `fouroversix/utils.py` so that
configurations written for it keep working (DataType `:13-189`, RoundStyle `:223-247`,
ScaleRule `:250-285`, ScaleType `:288-323`, QuantizedValueType `:326-383`). The
properties are driven by one table per enum instead of per-property dictionaries.
"""

from __future__ import annotations

from enum import Enum

import torch

SM_80, SM_100, SM_110, SM_120 = 8, 10, 11, 12
BLACKWELL_SM_IDS = {SM_100, SM_110, SM_120}


class ScaleRule(str, Enum):
    """How a block picks between mapping its maximum to 6 or to 4.

    `static_6` is ordinary NVFP4; `static_4` always uses 4; `mse`, `mae` and `abs_max`
    quantize the block both ways and keep the candidate with the smaller mean-squared,
    mean-absolute or maximum-absolute reconstruction error.
    """

    abs_max = "abs_max"
    mae = "mae"
    mse = "mse"
    static_4 = "static_4"
    static_6 = "static_6"

    @property
    def cuda_id(self) -> int:
        """Number of the rule in the native interface (FOS_RULE_* in the C header)."""
        return _RULE_IDS[self.value]

    @property
    def is_static(self) -> bool:
        return self.value.startswith("static")


_RULE_IDS = {"static_6": 0, "static_4": 1, "mae": 2, "mse": 3, "abs_max": 4}


class RoundStyle(str, Enum):
    """Rounding onto the 4-bit grid: nearest (even), or two stochastic variants."""

    nearest = "nearest"
    stochastic = "stochastic"
    stochastic_unbiased = "stochastic_unbiased"

    @property
    def adjustment_factor(self) -> float:
        return 16 / 17 if self is RoundStyle.stochastic_unbiased else 1

    @property
    def is_stochastic(self) -> bool:
        return self is not RoundStyle.nearest


class ScaleType(str, Enum):
    """Block-scale encodings: E8M0 (`mx`), E4M3 (`nv`), E4M3 whose sign bit flags an
    integer block (`nv_if`)."""

    mx = "mx"
    nv = "nv"
    nv_if = "nv_if"

    def get_maximum_value(self, scale_rule: ScaleRule) -> int | None:
        if self is ScaleType.mx:
            return None
        if self is ScaleType.nv and not scale_rule.is_static:
            return 256  # leaves head-room for the 1.5x "4" candidate
        return 448

    @property
    def torch_dtype(self) -> torch.dtype:
        return torch.float8_e8m0fnu if self is ScaleType.mx else torch.float8_e4m3fn


class QuantizedValueType(str, Enum):
    """Element encodings of the block-scaled formats."""

    fp3 = "fp3"
    fp4 = "fp4"
    fp6_e2m3 = "fp6_e2m3"
    fp6_e3m2 = "fp6_e3m2"
    if3 = "if3"
    if4 = "if4"
    if6_e2m3 = "if6_e2m3"
    if6_e3m2 = "if6_e3m2"
    int3 = "int3"
    int4 = "int4"
    int6 = "int6"

    def get_maximum_value(self, scale_rule: ScaleRule) -> float:
        if scale_rule is ScaleRule.static_4:
            return 4
        return _VALUE_TYPES[self.value][0]

    @property
    def packing_factor(self) -> int:
        return _VALUE_TYPES[self.value][1]


# value type -> (largest magnitude, elements per byte)
_VALUE_TYPES = {
    "fp3": (4, 1), "fp4": (6, 2), "fp6_e2m3": (7.5, 1), "fp6_e3m2": (28, 1),
    "if3": (4, 1), "if4": (6, 2), "if6_e2m3": (7.5, 1), "if6_e3m2": (28, 1),
    "int3": (3, 1), "int4": (7, 2), "int6": (31, 1),
}


class DataType(str, Enum):
    """High-precision types and block-scaled formats. The kernels in this package
    implement `nvfp4` and `if4`; the other members exist so that configurations that
    name them can be parsed and rejected with a clear message."""

    bfloat16 = "bfloat16"
    float16 = "float16"
    float32 = "float32"
    mxfp3 = "mxfp3"
    mxfp3_bs8 = "mxfp3_bs8"
    mxfp4 = "mxfp4"
    mxfp4_bs8 = "mxfp4_bs8"
    mxfp6_e2m3 = "mxfp6_e2m3"
    mxfp6_e3m2 = "mxfp6_e3m2"
    nvfp3 = "nvfp3"
    nvfp3_bs8 = "nvfp3_bs8"
    nvfp4 = "nvfp4"
    nvfp4_bs8 = "nvfp4_bs8"
    nvfp6_e2m3 = "nvfp6_e2m3"
    nvfp6_e3m2 = "nvfp6_e3m2"
    nvint3 = "nvint3"
    nvint3_bs8 = "nvint3_bs8"
    nvint4 = "nvint4"
    nvint4_bs8 = "nvint4_bs8"
    nvint6 = "nvint6"
    if3 = "if3"
    if3_bs8 = "if3_bs8"
    if4 = "if4"
    if4_bs8 = "if4_bs8"
    if6_e2m3 = "if6_e2m3"
    if6_e3m2 = "if6_e3m2"

    def _parts(self) -> tuple[str, str, int] | None:
        """(family, value type, block size) of a block-scaled format, else None."""
        name = self.value
        family = next((f for f in ("mx", "nv", "if") if name.startswith(f)), None)
        if family is None:
            return None
        body = name[2:]
        small = body.endswith("_bs8")
        body = body.removesuffix("_bs8")
        if family == "if":
            value = "if" + body
        elif body.startswith("int"):
            value = body
        else:
            value = body  # fp3, fp4, fp6_e2m3 ...
        block = 8 if small else (32 if family == "mx" else 16)
        return family, value, block

    @property
    def block_size(self) -> int | None:
        parts = self._parts()
        return parts[2] if parts else None

    @property
    def quantized_value_type(self) -> QuantizedValueType | None:
        parts = self._parts()
        return QuantizedValueType(parts[1]) if parts else None

    @property
    def scale_type(self) -> ScaleType | None:
        parts = self._parts()
        if parts is None:
            return None
        return {"mx": ScaleType.mx, "nv": ScaleType.nv, "if": ScaleType.nv_if}[parts[0]]

    @property
    def supported_scale_rules(self) -> set[ScaleRule]:
        parts = self._parts()
        if parts is None:
            return set()
        family, value, _ = parts
        if family == "if":
            return {r for r in ScaleRule if not r.is_static}
        if family == "mx":
            return {r for r in ScaleRule if r.is_static}
        if value == "fp4":
            return set(ScaleRule)
        return {ScaleRule.static_6}

    @property
    def torch_dtype(self) -> torch.dtype | None:
        return {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}.get(self.value)


class QuantizeBackend(str, Enum):
    """Quantization back ends by the reference's names. This package has exactly one
    implementation, the sm_100a kernels, registered as `cuda`; the other names are
    accepted in configurations and refused when used."""

    cuda = "cuda"
    pytorch = "pytorch"
    transformer_engine = "transformer_engine"
    triton = "triton"


class MatmulBackend(str, Enum):
    """Matmul back ends by the reference's names; `cutlass` names this package's
    hand-written tcgen05 kernels, the only implementation present."""

    cutlass = "cutlass"
    triton = "triton"
    pytorch = "pytorch"
