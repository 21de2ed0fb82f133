"""The one quantization back end of this package: hand-written sm_100a kernels behind
the C ABI in include/fouroversix_b200.h.

It fills the role of the reference's back-end plug-ins (class-method interface of
src/fouroversix/quantize/backend.py:16-234) for CUDA tensors on a B200 and takes over
what the reference splits between its CUDA back end (src/fouroversix/quantize/cuda/
backend.py:13-93: untransposed 1-D NVFP4 only) and its Triton back end
(src/fouroversix/quantize/triton.py: 2-D blocks, transposed input, IF4).
"""

from __future__ import annotations

import functools

import torch

from fouroversix_b200 import _native
from fouroversix_b200.utils import DataType, ScaleRule, RoundStyle, ScaleType

from .config import QuantizationConfig
from .quantized_tensor import QuantizedTensor, padded_shape_for

_FORMATS = {DataType.nvfp4: _native.FOS_NVFP4, DataType.if4: _native.FOS_IF4, DataType.mxfp4: _native.FOS_MXFP4}


def _is_tiled(dtype: DataType) -> bool:
    # like the reference's PyTorch back end, IF4 keeps its scales row-major
    # (src/fouroversix/quantize/pytorch/backend.py:107-120)
    return dtype in (DataType.nvfp4, DataType.mxfp4)


def _scale_view(scales: torch.Tensor, dtype: DataType) -> torch.Tensor:
    """The scale bytes typed as the reference types them: E4M3, or E8M0 for the MX formats."""
    return scales.view(torch.float8_e8m0fnu if dtype.scale_type == ScaleType.mx else torch.float8_e4m3fn)


class B200QuantizeBackend:
    """Quantize / dequantize on a B200 through libfouroversix_b200.so."""

    @classmethod
    @functools.lru_cache
    def is_available(cls) -> bool:
        if not torch.cuda.is_available() or torch.cuda.get_device_capability()[0] != 10:
            return False
        _native.lib()  # a missing extension on a GPU machine is an error, not "unavailable"
        return True

    @classmethod
    def unsupported_reason(cls, x: torch.Tensor, config: QuantizationConfig) -> str | None:
        """Why this back end cannot run the request, or None when it can."""
        if x.ndim != 2:
            return "input must be 2-D"
        if config.dtype not in _FORMATS:
            return f"dtype {config.dtype.value} is not implemented (nvfp4, if4 and mxfp4 are)"
        if config.scale_rule not in config.dtype.supported_scale_rules:
            return f"scale rule {config.scale_rule.value} is not defined for {config.dtype.value}"
        if config.round_style.is_stochastic:
            if config.block_scale_2d or config.dtype not in (DataType.nvfp4, DataType.if4):
                return "stochastic rounding is implemented for NVFP4 and IF4 with 1-D blocks"
            if config.dtype == DataType.if4 and config.scale_rule != ScaleRule.mse:
                return "stochastic rounding of IF4 compares its two grids by squared error (scale rule mse)"
        if config.rht and config.dtype == DataType.mxfp4:
            return "the random Hadamard transform is not implemented for mxfp4"
        if config.rht and x.ndim == 2 and x.shape[0 if config.transpose else 1] % 16 != 0:
            return "the random Hadamard transform needs a multiple of 16 values along the quantized axis"
        if x.device.type != "cuda":
            return "input must be a CUDA tensor (there is no CPU path)"
        if x.dtype not in (torch.bfloat16, torch.float16):
            return "input must be bfloat16 or float16"
        return None

    @classmethod
    def can_quantize(cls, x: torch.Tensor, config: QuantizationConfig) -> bool:
        return cls.unsupported_reason(x, config) is None and cls.is_available()

    @classmethod
    def quantize(cls, x: torch.Tensor, config: QuantizationConfig, *, amax: torch.Tensor | None = None,
                 exact_only: bool = False, seed: int | None = None, kernel: str = "auto") -> QuantizedTensor:
        """Quantize `x` (or its transpose). `amax`, when given, is a CUDA fp32 tensor that
        already holds max|x| and saves the extra pass that computes it. With stochastic rounding,
        `seed` selects the noise (default: drawn from torch's CPU generator, so torch.manual_seed
        makes a run repeatable). `kernel` is a testing aid (every kernel writes the same bytes):
        "no_tma" = never a kernel fed by the TMA unit, "general" = the general TMA-fed kernel also
        where a specialised one exists."""
        reason = cls.unsupported_reason(x, config)
        if reason is not None:
            raise ValueError(f"B200 quantize: {reason}")
        if x.stride(1) != 1:
            x = x.contiguous()
        rows, cols = x.shape
        out_shape = (cols, rows) if config.transpose else (rows, cols)
        rows_p, cols_p = padded_shape_for(out_shape, config.dtype)
        dev = x.device
        values = torch.empty(rows_p, cols_p // 2, dtype=torch.uint8, device=dev)
        scales = torch.empty(rows_p * cols_p // config.dtype.block_size, dtype=torch.uint8, device=dev)
        amax_out = torch.empty(1, dtype=torch.float32, device=dev)
        if amax is not None:
            amax = amax.detach().reshape(1).to(device=dev, dtype=torch.float32)
        tiled = _is_tiled(config.dtype)
        args = (x.data_ptr(), _native.elem_code(x.dtype), rows, cols, x.stride(0),
                _FORMATS[config.dtype], config.scale_rule.cuda_id, int(config.block_scale_2d),
                int(config.transpose), _native.FOS_SF_TILED if tiled else _native.FOS_SF_ROWMAJOR,
                0 if amax is None else amax.data_ptr(), values.data_ptr(), scales.data_ptr(),
                amax_out.data_ptr(),
                (_native.FOS_QUANTIZE_EXACT_ONLY if exact_only else 0) | (_native.FOS_QUANTIZE_RHT if config.rht else 0)
                | {"auto": 0, "no_tma": _native.FOS_QUANTIZE_NO_TMA, "general": _native.FOS_QUANTIZE_GENERAL_KERNEL}[kernel]
                | (_native.FOS_QUANTIZE_UNBIASED if config.round_style == RoundStyle.stochastic_unbiased else 0))
        with torch.cuda.device(dev):
            if config.round_style.is_stochastic:
                if seed is None:
                    seed = int(torch.randint(0, 2 ** 62, (1,)).item())
                status = _native.lib().fos_quantize_stochastic(*args, seed, _native.stream_ptr(dev))
                if status == -2:
                    raise ValueError("B200 quantize: stochastic rounding needs a 16-byte aligned input (base and row stride)")
            else:
                status = _native.lib().fos_quantize(*args, _native.stream_ptr(dev))
        _native.check(status, "fos_quantize")
        return QuantizedTensor(
            values, _scale_view(scales, config.dtype), amax_out, config.dtype, out_shape,
            config.scale_rule, config.round_style, (rows_p, cols_p),
            scale_factors_are_in_blackwell_layout=tiled)

    @classmethod
    def amax(cls, x: torch.Tensor) -> torch.Tensor:
        """max |x| of a 2-D bf16 / fp16 CUDA tensor as a 1-element fp32 tensor (fos_amax): the first pass of
        `quantize` on its own, for callers that quantize one tensor in pieces with a common amax."""
        if x.ndim != 2 or x.device.type != "cuda" or x.dtype not in (torch.bfloat16, torch.float16):
            raise ValueError("B200 amax: input must be a 2-D bfloat16 / float16 CUDA tensor")
        if x.stride(1) != 1:
            x = x.contiguous()
        out = torch.empty(1, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            _native.check(_native.lib().fos_amax(x.data_ptr(), _native.elem_code(x.dtype), x.shape[0], x.shape[1],
                                                 x.stride(0), out.data_ptr(), _native.stream_ptr(x.device)), "fos_amax")
        return out

    @classmethod
    def can_dequantize(cls, tensor: QuantizedTensor) -> bool:
        return tensor.dtype in _FORMATS and tensor.device.type == "cuda" and cls.is_available()

    @classmethod
    def dequantize(cls, tensor: QuantizedTensor, dtype: torch.dtype = torch.bfloat16, *,
                   intermediate_dtype: torch.dtype = torch.float16) -> torch.Tensor:
        """High-precision copy of `tensor`, cropped to its original shape. The kernel
        implements the reference's default fp16 intermediate."""
        if tensor.dtype not in _FORMATS:
            raise ValueError(f"B200 dequantize: dtype {tensor.dtype.value} is not implemented")
        if tensor.device.type != "cuda":
            raise ValueError("B200 dequantize: tensor must live on a CUDA device (there is no CPU path)")
        if intermediate_dtype not in (torch.float16, torch.float32):
            raise ValueError("B200 dequantize: the intermediate type must be float16 or float32")
        if tensor.dtype.scale_type in (ScaleType.nv, ScaleType.nv_if) and tensor.amax is None:
            raise ValueError("B200 dequantize: amax is required")
        rows, cols = tensor.original_shape
        rows_p, cols_p = tensor.padded_shape
        dev = tensor.device
        out = torch.empty(rows, cols, dtype=dtype, device=dev)
        values = tensor.values.contiguous()
        scales = tensor.scale_factors.contiguous()
        amax = None if tensor.amax is None else tensor.amax.to(device=dev, dtype=torch.float32)
        with torch.cuda.device(dev):
            status = _native.lib().fos_dequantize_ex(
                values.data_ptr(), scales.data_ptr(), 0 if amax is None else amax.data_ptr(), _FORMATS[tensor.dtype],
                tensor.scale_rule.cuda_id,
                _native.FOS_SF_TILED if tensor.scale_factors_are_in_blackwell_layout else _native.FOS_SF_ROWMAJOR,
                rows_p, cols_p, rows, cols, out.data_ptr(), _native.elem_code(dtype), out.stride(0),
                _native.elem_code(intermediate_dtype),
                _native.FOS_DEQUANT_UNBIASED if tensor.round_style == RoundStyle.stochastic_unbiased else 0,
                _native.stream_ptr(dev))
        _native.check(status, "fos_dequantize")
        return out

    @classmethod
    def dequantize_values(cls, tensor: QuantizedTensor, *, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """The raw values of a quantized tensor in `dtype`, padded shape, no scales applied (the reference's
        QuantizeBackendBase.dequantize_values, src/fouroversix/quantize/backend.py:164-189): E2M1 codes as numbers,
        IF4 integer blocks as integer * 6/7."""
        if tensor.dtype not in _FORMATS:
            raise ValueError(f"B200 dequantize: dtype {tensor.dtype.value} is not implemented")
        if tensor.device.type != "cuda":
            raise ValueError("B200 dequantize: tensor must live on a CUDA device (there is no CPU path)")
        rows_p, cols_p = tensor.padded_shape
        dev = tensor.device
        out = torch.empty(rows_p, cols_p, dtype=dtype, device=dev)
        with torch.cuda.device(dev):
            status = _native.lib().fos_dequantize_ex(
                tensor.values.contiguous().data_ptr(), tensor.scale_factors.contiguous().data_ptr(), 0,
                _FORMATS[tensor.dtype], tensor.scale_rule.cuda_id,
                _native.FOS_SF_TILED if tensor.scale_factors_are_in_blackwell_layout else _native.FOS_SF_ROWMAJOR,
                rows_p, cols_p, rows_p, cols_p, out.data_ptr(), _native.elem_code(dtype), out.stride(0),
                _native.FOS_FP16, _native.FOS_DEQUANT_VALUES_ONLY, _native.stream_ptr(dev))
        _native.check(status, "fos_dequantize_ex")
        return out

    @classmethod
    def pseudo_quantize(cls, x: torch.Tensor, config: QuantizationConfig) -> torch.Tensor:
        """Quantize then dequantize back to x's dtype: one fused kernel for 1-D blocks of an
        untransposed, 16-byte-aligned input (fos_pseudo_quantize), otherwise the quantize and the
        dequantize kernel one after the other. Same bits either way."""
        reason = cls.unsupported_reason(x, config)
        if reason is not None:
            raise ValueError(f"B200 quantize: {reason}")
        if not config.block_scale_2d and not config.transpose and not config.rht and config.dtype != DataType.mxfp4:
            if x.stride(1) != 1:
                x = x.contiguous()
            rows, cols = x.shape
            out = torch.empty(rows, cols, dtype=x.dtype, device=x.device)
            amax_out = torch.empty(1, dtype=torch.float32, device=x.device)
            with torch.cuda.device(x.device):
                status = _native.lib().fos_pseudo_quantize(
                    x.data_ptr(), _native.elem_code(x.dtype), rows, cols, x.stride(0), _FORMATS[config.dtype],
                    config.scale_rule.cuda_id, 0, out.data_ptr(), out.stride(0), amax_out.data_ptr(), 0,
                    _native.stream_ptr(x.device))
            if status == 0:
                return out
            if status != -2:   # anything but "this input needs the two-kernel path"
                _native.check(status, "fos_pseudo_quantize")
        return cls.dequantize(cls.quantize(x, config), dtype=x.dtype)
