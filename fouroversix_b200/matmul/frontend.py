"""`quantized_matmul()`: same signature as the reference front end
(src/fouroversix/matmul/frontend.py:18-132); plain tensors are quantized first."""

from __future__ import annotations

from typing import Any

import torch

from fouroversix_b200.quantize import QuantizationConfig, QuantizedTensor, quantize
from fouroversix_b200.utils import DataType, MatmulBackend

from .backend import B200MatmulBackend

AVAILABLE_BACKENDS = {
    MatmulBackend.cutlass: B200MatmulBackend,
    MatmulBackend.triton: None,
    MatmulBackend.pytorch: None,
}


def quantized_matmul(
    input: torch.Tensor | QuantizedTensor,
    other: torch.Tensor | QuantizedTensor,
    *,
    backend: MatmulBackend | None = None,
    input_config: QuantizationConfig | None = None,
    other_config: QuantizationConfig | None = None,
    out_dtype: DataType = DataType.bfloat16,
    fuse_input_quantization: bool = False,
    **kwargs: Any,
) -> torch.Tensor:
    """`input @ other.T` in FP4.  Either operand may be a high-precision CUDA tensor, in
    which case it is quantized with the matching config (default: NVFP4, 4/6 MSE).
    `fuse_input_quantization=True` (not in the reference) quantizes a high-precision `input`
    inside the GEMM when its config allows (NVFP4, static_6 / static_4, 1-D blocks): same bits,
    no packed activation in memory; other configs take the usual two steps."""
    if isinstance(other, torch.Tensor):
        other = quantize(other, other_config or QuantizationConfig())
    if fuse_input_quantization and isinstance(input, torch.Tensor) and backend in (None, MatmulBackend.cutlass):
        try:
            return B200MatmulBackend.fused_quantize_matmul(input, other, input_config or QuantizationConfig(),
                                                           out_dtype=DataType(out_dtype), **kwargs)
        except ValueError:
            pass                                   # not a case of the fused kernel: quantize first
    if isinstance(input, torch.Tensor):
        input = quantize(input, input_config or QuantizationConfig())

    impl = B200MatmulBackend if backend is None else AVAILABLE_BACKENDS.get(MatmulBackend(backend))
    if impl is None:
        raise ValueError(f"Backend {backend} does not support the given parameters "
                         "(this build contains only the B200 kernels, registered as 'cutlass')")
    reason = impl.unsupported_reason(input, other, out_dtype=out_dtype)
    if reason is not None:
        if backend is None:
            raise ValueError(f"No backend found that supports the given parameters ({reason})")
        raise ValueError(f"Backend {backend} does not support the given parameters ({reason})")
    return impl.quantized_matmul(input, other, out_dtype=DataType(out_dtype), **kwargs)
