"""Thin per-op wrappers over the C ABI; one function per native entry point,
named like the reference's ``cublade.bindings.cuda`` functions."""
from .quantize_fp8 import quantize_per_tensor_fp8
from .dequantize_fp8 import dequantize_per_tensor_fp8
from .quantize_int8 import (quantize_per_tensor_int8, quantize_per_channel_int8, quantize_per_group_int8,
                            quantize_per_axis_int8)
from .dequantize_int8 import (dequantize_per_tensor_int8, dequantize_per_channel_int8, dequantize_per_group_int8,
                              dequantize_per_axis_int8)
from .rmsnorm_quant import rmsnorm_quantize
from .wmma import wmma_gemm

__all__ = [
    "quantize_per_tensor_fp8", "dequantize_per_tensor_fp8",
    "quantize_per_tensor_int8", "quantize_per_channel_int8", "quantize_per_group_int8",
    "dequantize_per_tensor_int8", "dequantize_per_channel_int8", "dequantize_per_group_int8",
    "quantize_per_axis_int8", "dequantize_per_axis_int8", "rmsnorm_quantize", "wmma_gemm",
]
