"""`QuantizedTensor`: packed 4-bit values, block scales and the per-tensor amax.

Same fields, constructor signature and padding rules as the reference container
(src/fouroversix/quantize/quantized_tensor.py:10-144): rows are padded to a multiple of
128 and columns to a multiple of four blocks, the shape the 128x4 scale tiles need.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from fouroversix_b200.utils import DataType, RoundStyle, ScaleRule

from .layout import to_blocked


def padded_shape_for(shape: tuple[int, int], dtype: DataType) -> tuple[int, int]:
    """Smallest (rows, cols) >= shape with rows % 128 == 0 and cols % (4 * block) == 0."""
    col_unit = 4 * dtype.block_size
    return (-(-shape[0] // 128) * 128, -(-shape[1] // col_unit) * col_unit)


class QuantizedTensor:
    """A 2-D tensor stored as `values` (uint8, two codes per byte, low nibble first),
    `scale_factors` (one E4M3 byte per block) and `amax` (fp32 [1])."""

    def __init__(
        self,
        values: torch.Tensor,
        scale_factors: torch.Tensor,
        amax: torch.Tensor,
        dtype: DataType,
        original_shape: tuple[int, int],
        scale_rule: ScaleRule,
        round_style: RoundStyle,
        padded_shape: tuple[int, int] | None = None,
        *,
        scale_factors_are_in_blackwell_layout: bool = True,
    ) -> None:
        self.dtype = DataType(dtype)
        self.original_shape = tuple(original_shape)
        self.scale_rule = ScaleRule(scale_rule)
        self.round_style = RoundStyle(round_style)
        self.scale_factors_are_in_blackwell_layout = bool(scale_factors_are_in_blackwell_layout)

        if padded_shape is not None:
            self.padded_shape = tuple(padded_shape)
        else:
            self.padded_shape = padded_shape_for(self.original_shape, self.dtype)
            values, scale_factors = self._pad_to(values, scale_factors)

        self.values = values
        self.scale_factors = scale_factors
        self.amax = amax

    def _pad_to(self, values: torch.Tensor, scale_factors: torch.Tensor):
        rows, cols = self.padded_shape
        per_byte = self.dtype.quantized_value_type.packing_factor
        block = self.dtype.block_size
        want_values, want_scales = rows * cols // per_byte, rows * cols // block

        if values.numel() != want_values:
            values = F.pad(values, (0, cols // per_byte - values.shape[1], 0, rows - values.shape[0]))
        # a 1-D scale tensor is taken to be in tile order already; a 2-D one is row-major
        if scale_factors.ndim > 1 and scale_factors.numel() != want_scales:
            fill = 0 if self.dtype == DataType.nvfp4 else 1
            scale_factors = F.pad(
                scale_factors,
                (0, cols // block - scale_factors.shape[1], 0, rows - scale_factors.shape[0]),
                value=fill,
            )
            if self.scale_factors_are_in_blackwell_layout:
                scale_factors = to_blocked(scale_factors)

        if values.numel() != want_values:
            raise ValueError(f"Expected {want_values} e2m1 values, got {values.numel()}")
        if scale_factors.numel() != want_scales:
            raise ValueError(f"Expected {want_scales} scale factors, got {scale_factors.numel()}")
        return values, scale_factors

    @property
    def device(self) -> torch.device:
        return self.values.device

    def __repr__(self) -> str:
        return (f"QuantizedTensor(dtype={self.dtype.value}, original_shape={self.original_shape}, "
                f"padded_shape={self.padded_shape}, scale_rule={self.scale_rule.value}, device={self.device})")
