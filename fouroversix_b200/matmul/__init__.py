from .backend import B200MatmulBackend
from .frontend import quantized_matmul
from .grouped import (GroupedQuantizedTensor, GroupLayout, StackedQuantizedTensor, grouped_quantize,
                      grouped_quantized_matmul)

__all__ = ["B200MatmulBackend", "GroupLayout", "GroupedQuantizedTensor", "StackedQuantizedTensor",
           "grouped_quantize", "grouped_quantized_matmul", "quantized_matmul"]
