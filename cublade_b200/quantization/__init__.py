"""Drop-in for ``cublade.quantization`` (same public names as cublade/quantization/__init__.py:8-17)."""
from .utils import *  # noqa: F401,F403
from .tensor import QuantizedTensor
from .dequantizers import dequantize_tensor
from .linear import cuBladeW8A16LinearLayer, cubladeW8A16LinearLayer
from .quantizers import quantize_tensor, quantize_model
from .outlier_utils import detect_outlier_columns, separate_outliers, split_weights_by_outliers
from .fused import rmsnorm_quantize_tensor
from .linear_w4a16 import cuBladeW4A16LinearLayer
from .linear_w8a8 import cuBladeW8A8LinearLayer
from .checkpoint import load_quantized_model, load_quantized_state_dict, save_quantized_model

__all__ = [
    "quantize_model",
    "quantize_tensor",
    "dequantize_tensor",
    "QuantizedTensor",
    "cuBladeW8A16LinearLayer",
    "cubladeW8A16LinearLayer",
    "detect_outlier_columns",
    "separate_outliers",
    "split_weights_by_outliers",
    "rmsnorm_quantize_tensor",
    "cuBladeW4A16LinearLayer",
    "cuBladeW8A8LinearLayer",
    "save_quantized_model",
    "load_quantized_model",
    "load_quantized_state_dict",
]
