"""cublade_b200: the ``cublade.quantization`` hot path rebuilt for B200 (sm_100a).

FP8-E4M3 / INT8 quantize + dequantize and the W8A16 linear layer, as hand-written CUDA
behind a C ABI (``libcublade_b200.so``, declared in ``include/cublade_b200.h``) with the
reference's Python API on top (``cublade_b200.quantization``).  There is no CPU or PyTorch
fallback: using an op without the built library raises ``RuntimeError``.
"""
from . import quantization  # noqa: F401
from .quantization import (  # noqa: F401
    QuantizedTensor,
    cuBladeW8A16LinearLayer,
    cubladeW8A16LinearLayer,
    dequantize_tensor,
    quantize_model,
    quantize_tensor,
)

__version__ = "0.1.0"
