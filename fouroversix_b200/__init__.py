"""fouroversix_b200: NVFP4 / IF4 quantization with Four-Over-Six adaptive block scaling
and the FP4 GEMM that consumes it, as hand-written sm_100a kernels behind the public
API of mit-han-lab/fouroversix (`quantize`, `dequantize`, `quantized_matmul`,
`QuantizedTensor`, `QuantizationConfig`, `FourOverSixLinear`, `quantize_model`)."""

from .matmul import quantized_matmul
from .model import (
    FourOverSixLinear,
    ModelQuantizationConfig,
    ModuleQuantizationConfig,
    QuantizedModule,
    quantize_model,
)
from .quantize import QuantizationConfig, QuantizedTensor, dequantize, quantize
from .utils import DataType, MatmulBackend, QuantizeBackend, RoundStyle, ScaleRule

__version__ = "0.1.0"

__all__ = [
    "DataType",
    "FourOverSixLinear",
    "MatmulBackend",
    "ModelQuantizationConfig",
    "ModuleQuantizationConfig",
    "QuantizationConfig",
    "QuantizeBackend",
    "QuantizedModule",
    "QuantizedTensor",
    "RoundStyle",
    "ScaleRule",
    "dequantize",
    "quantize",
    "quantize_model",
    "quantized_matmul",
]
