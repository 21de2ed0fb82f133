"""Grouped FP4 GEMMs: many `quantized_matmul`s that share n, k and the output type in one launch.

The reference runs a mixture-of-experts layer as a host loop over the experts that were hit
(src/fouroversix/model/modules/gpt_oss.py:297-335): per expert it reads the routed token indices back from
the device, quantizes those tokens as a tensor of their own and calls `quantized_matmul` against that
expert's weight. Here the rows of all experts lie in one padded buffer, the row ranges stay on the device,
and one quantize launch and one GEMM launch cover every expert: no read-back, no per-expert launches.
The bits are those of the loop: every group is quantized with its own amax and multiplied with its own
weight and its own alpha.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from fouroversix_b200 import _native
from fouroversix_b200.quantize import QuantizationConfig, QuantizedTensor
from fouroversix_b200.utils import DataType, RoundStyle, ScaleRule

_OUT = {DataType.bfloat16: torch.bfloat16, DataType.float16: torch.float16, DataType.float32: torch.float32}
MAX_GROUPS = 256


@dataclass
class GroupLayout:
    """Where each group's rows lie in the padded buffer. `group_start` (num_groups + 1 values) and
    `group_rows` are int32 CUDA tensors; `capacity` is the host-side size of the buffer (the worst case for the
    given total number of rows), so nothing here waits for the device."""

    group_start: torch.Tensor
    group_rows: torch.Tensor
    capacity: int
    num_groups: int

    @classmethod
    def from_counts(cls, counts: torch.Tensor, total_rows: int) -> "GroupLayout":
        """`counts[g]` rows for group g (an integer CUDA tensor that sums to `total_rows`). Every group starts
        on a multiple of 128 rows, the height of a scale-factor tile and of a GEMM tile."""
        g = counts.numel()
        if not 0 < g <= MAX_GROUPS:
            raise ValueError(f"between 1 and {MAX_GROUPS} groups")
        padded = (counts.to(torch.int64) + 127) // 128 * 128
        start = torch.zeros(g + 1, dtype=torch.int64, device=counts.device)
        torch.cumsum(padded, 0, out=start[1:])
        capacity = (total_rows + 127 * g + 127) // 128 * 128
        return cls(start.to(torch.int32), counts.to(torch.int32).contiguous(), capacity, g)


@dataclass
class GroupedQuantizedTensor:
    """The quantized rows of every group: codes [capacity, k / 2], scale factors in 128 x 4 tiles (a group
    starts on a tile boundary), one amax per group."""

    values: torch.Tensor
    scale_factors: torch.Tensor
    amax: torch.Tensor
    layout: GroupLayout
    dtype: DataType
    scale_rule: ScaleRule
    cols: int


@dataclass
class StackedQuantizedTensor:
    """num_groups quantized matrices of one shape, stacked the way the reference stores expert weights
    (src/fouroversix/model/modules/gpt_oss.py:239-249): values [g, n_p, k_p / 2], scale factors [g, ...], amax [g]."""

    values: torch.Tensor
    scale_factors: torch.Tensor
    amax: torch.Tensor
    dtype: DataType
    scale_rule: ScaleRule
    original_shape: tuple[int, int]
    padded_shape: tuple[int, int]

    @classmethod
    def stack(cls, tensors: list[QuantizedTensor]) -> "StackedQuantizedTensor":
        first = tensors[0]
        for t in tensors:
            if (t.original_shape, t.padded_shape, t.dtype, t.scale_rule) != (
                    first.original_shape, first.padded_shape, first.dtype, first.scale_rule):
                raise ValueError("stacked tensors must share shape, format and scale rule")
            if not t.scale_factors_are_in_blackwell_layout or t.round_style == RoundStyle.stochastic_unbiased:
                raise ValueError("stacked tensors need tiled scale factors and plain rounding")
        return cls(torch.stack([t.values for t in tensors]).contiguous(),
                   torch.stack([t.scale_factors.reshape(-1) for t in tensors]).contiguous(),
                   torch.cat([t.amax.reshape(1) for t in tensors]).contiguous(),
                   first.dtype, first.scale_rule, tuple(first.original_shape), tuple(first.padded_shape))

    def __getitem__(self, g: int) -> QuantizedTensor:
        return QuantizedTensor(self.values[g], self.scale_factors[g], self.amax[g:g + 1], self.dtype,
                               self.original_shape, self.scale_rule, "nearest", self.padded_shape)


def grouped_quantize(x: torch.Tensor, layout: GroupLayout, config: QuantizationConfig | None = None,
                     amax: torch.Tensor | None = None) -> GroupedQuantizedTensor:
    """Quantizes the padded buffer x [capacity, k] (bf16 / fp16; rows outside the groups' real rows must be
    zero) group by group in one launch (fos_quantize_grouped): group g gets the bytes `quantize` gives for
    its rows alone. 1-D blocks, round to nearest, NVFP4 or IF4."""
    config = config or QuantizationConfig()
    dtype, rule = DataType(config.dtype), ScaleRule(config.scale_rule)
    if dtype not in (DataType.nvfp4, DataType.if4):
        raise ValueError("grouped quantization: nvfp4 or if4")
    if config.block_scale_2d or config.transpose or config.rht or RoundStyle(config.round_style) != RoundStyle.nearest:
        raise ValueError("grouped quantization: 1-D blocks, no transpose, no rotation, round to nearest")
    if x.dim() != 2 or x.shape[0] != layout.capacity or x.dtype not in (torch.bfloat16, torch.float16) or not x.is_cuda:
        raise ValueError("grouped quantization: x must be a [capacity, k] bf16 / fp16 CUDA tensor")
    if x.stride(1) != 1:
        x = x.contiguous()
    k = x.shape[1]
    dev = x.device
    values = torch.empty(layout.capacity, k // 2, dtype=torch.uint8, device=dev)
    scales = torch.empty(layout.capacity * k // 16, dtype=torch.uint8, device=dev)
    amax_out = torch.empty(layout.num_groups, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _native.check(_native.lib().fos_quantize_grouped(
            x.data_ptr(), _native.elem_code(x.dtype), layout.capacity, k, x.stride(0),
            _native.FOS_IF4 if dtype == DataType.if4 else _native.FOS_NVFP4, rule.cuda_id,
            layout.group_start.data_ptr(), layout.group_rows.data_ptr(), layout.num_groups,
            0 if amax is None else amax.data_ptr(), values.data_ptr(), scales.data_ptr(), amax_out.data_ptr(), 0,
            _native.stream_ptr(dev)), "fos_quantize_grouped")
    return GroupedQuantizedTensor(values, scales.view(torch.float8_e4m3fn), amax_out, layout, dtype, rule, k)


def grouped_quantized_matmul(a: GroupedQuantizedTensor, b: StackedQuantizedTensor, *,
                             out_dtype: DataType = DataType.bfloat16, out: torch.Tensor | None = None,
                             variant: int = 0, max_ctas: int = 0) -> torch.Tensor:
    """out[rows of group g] = a[rows of group g] @ b[g].T for every group, one launch
    (fos_gemm_nvfp4_grouped). Returns the padded [capacity, n] buffer; only the groups' real rows are written
    when `out` is given, and a fresh buffer is zero elsewhere."""
    if a.dtype != DataType.nvfp4 or b.dtype != DataType.nvfp4:
        raise ValueError("grouped matmul: nvfp4 operands")
    n, k = b.original_shape
    n_p, k_p = b.padded_shape
    if a.cols != k_p or b.values.shape[0] != a.layout.num_groups:
        raise ValueError("grouped matmul: operands disagree on k or on the number of groups")
    torch_out = _OUT[DataType(out_dtype)]
    dev = a.values.device
    cap = a.layout.capacity
    if out is None:
        out = torch.zeros(cap, n, dtype=torch_out, device=dev)
    elif out.shape != (cap, n) or out.dtype != torch_out or out.stride(1) != 1:
        raise ValueError("grouped matmul: `out` has the wrong shape, dtype or layout")
    alpha = torch.empty(a.layout.num_groups, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        lib, stream = _native.lib(), _native.stream_ptr(dev)
        _native.check(lib.fos_gemm_alpha_grouped(
            a.amax.data_ptr(), _native.FOS_NVFP4, a.scale_rule.cuda_id, 0,
            b.amax.data_ptr(), _native.FOS_NVFP4, b.scale_rule.cuda_id, 0,
            alpha.data_ptr(), a.layout.num_groups, stream), "fos_gemm_alpha_grouped")
        _native.check(lib.fos_gemm_nvfp4_grouped(
            a.values.data_ptr(), a.scale_factors.data_ptr(), b.values.data_ptr(), b.scale_factors.data_ptr(),
            alpha.data_ptr(), out.data_ptr(), _native.elem_code(torch_out),
            a.layout.group_start.data_ptr(), a.layout.group_rows.data_ptr(), a.layout.num_groups,
            cap, n_p, k_p, n, out.stride(0), _native.gemm_opts(variant, max_ctas), 0, stream), "fos_gemm_nvfp4_grouped")
    return out
