from .backend import B200QuantizeBackend
from .config import QuantizationConfig
from .frontend import dequantize, quantize
from .layout import from_blocked, to_blocked
from .quantized_tensor import QuantizedTensor

__all__ = [
    "B200QuantizeBackend",
    "QuantizationConfig",
    "QuantizedTensor",
    "dequantize",
    "from_blocked",
    "quantize",
    "to_blocked",
]
