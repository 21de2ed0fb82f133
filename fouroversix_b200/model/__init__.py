from .config import ModelQuantizationConfig, ModuleQuantizationConfig
from .linear import FourOverSixLinear, FourOverSixLinearFunction
from .quantize import QuantizedModule, quantize_model

__all__ = [
    "FourOverSixLinear",
    "FourOverSixLinearFunction",
    "ModelQuantizationConfig",
    "ModuleQuantizationConfig",
    "QuantizedModule",
    "quantize_model",
]
