"""`quantize()` and `dequantize()`: same call signatures as the reference front end
(src/fouroversix/quantize/frontend.py:19-157), one implementation behind them."""

from __future__ import annotations

import torch

from fouroversix_b200.utils import QuantizeBackend

from .backend import B200QuantizeBackend
from .config import QuantizationConfig
from .quantized_tensor import QuantizedTensor

# The reference probes cuda -> triton -> pytorch. Here only `cuda` maps to code.
AVAILABLE_BACKENDS = {
    QuantizeBackend.cuda: B200QuantizeBackend,
    QuantizeBackend.transformer_engine: None,
    QuantizeBackend.triton: None,
    QuantizeBackend.pytorch: None,
}


def _select(backend: QuantizeBackend | None) -> type[B200QuantizeBackend]:
    if backend is None:
        return B200QuantizeBackend
    impl = AVAILABLE_BACKENDS.get(QuantizeBackend(backend))
    if impl is None:
        raise ValueError(f"Backend {backend} does not support the given parameters "
                         "(this build contains only the B200 kernels, registered as 'cuda')")
    return impl


def quantize(x: torch.Tensor, config: QuantizationConfig | None = None) -> QuantizedTensor | torch.Tensor:
    """Quantize a 2-D bf16/fp16 CUDA tensor to NVFP4 or IF4.

    With no config: NVFP4, 1x16 blocks, round-to-nearest, Four-Over-Six with the
    mean-squared-error rule.  Returns a `QuantizedTensor`, or with
    `config.pseudo_quantize` the dequantized tensor in x's dtype.
    """
    config = config or QuantizationConfig()
    impl = _select(config.backend)
    reason = impl.unsupported_reason(x, config)
    if reason is not None:
        if config.backend is None:
            raise ValueError(f"No backend found that supports the given parameters ({reason})")
        raise ValueError(f"Backend {config.backend} does not support the given parameters ({reason})")
    if config.pseudo_quantize:
        return impl.pseudo_quantize(x, config)
    return impl.quantize(x, config)


def dequantize(tensor: QuantizedTensor, dtype: torch.dtype = torch.bfloat16, *,
               backend: QuantizeBackend | None = None,
               intermediate_dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """Return the high-precision tensor a `QuantizedTensor` stands for."""
    return _select(backend).dequantize(tensor, dtype, intermediate_dtype=intermediate_dtype)
