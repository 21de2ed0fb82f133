from .backend import B200MatmulBackend
from .frontend import quantized_matmul

__all__ = ["B200MatmulBackend", "quantized_matmul"]
