"""B200-native kernels for the ``quantized_ops`` hot path of voyager-compiler.

Importing the package loads the CUDA shared library (there is no CPU implementation) and attaches
its kernels to ``torch.ops.quantized_ops`` -- to the upstream library definition when
``voyager_compiler`` was imported first, to its own verbatim schema definitions otherwise.
"""
from . import _lib  # noqa: F401  (fails loudly when the shared library is missing)
from . import ops, qtables, tables
from .ops import (calculate_mx_qparam, conv2d_mx, dequantize, linear_mx, matmul_mx, quantize, quantize_mx, register,
                  vmap)
from .qtables import set_table_policy, table_handle

REGISTERED_AS = register()

__all__ = ["ops", "qtables", "tables", "vmap", "quantize", "dequantize", "calculate_mx_qparam", "quantize_mx",
           "linear_mx", "matmul_mx", "conv2d_mx", "register", "set_table_policy", "table_handle", "REGISTERED_AS"]
