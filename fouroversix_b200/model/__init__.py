from .config import ModelQuantizationConfig, ModuleQuantizationConfig
from .experts import FourOverSixExperts
from .linear import FourOverSixLinear, FourOverSixLinearFunction
from .quantize import QuantizedModule, quantize_model

__all__ = [
    "FourOverSixExperts",
    "FourOverSixLinear",
    "FourOverSixLinearFunction",
    "ModelQuantizationConfig",
    "ModuleQuantizationConfig",
    "QuantizedModule",
    "quantize_model",
]
