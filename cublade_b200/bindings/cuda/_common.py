"""Argument checks shared by the binding wrappers.

They reproduce the reference's native-side ``TORCH_CHECK``s, which surface in
Python as ``RuntimeError`` (cublade/kernels/cuda/quantization/quantize_int8.cu:453-460,
dequantize_int8.cu:193-202, dequantize_per_tensor_fp8.cu:88-97).
"""
from __future__ import annotations

import torch


def require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def check_quant_input(x: torch.Tensor, allowed, allowed_text: str) -> None:
    require(isinstance(x, torch.Tensor) and x.is_cuda, "x must be on CUDA")
    require(x.is_contiguous(), "x must be contiguous")
    require(x.dtype in allowed, f"x must be {allowed_text}")


def check_dequant_input(q: torch.Tensor, scale: torch.Tensor, out_dtype: torch.dtype, q_dtype: torch.dtype,
                        q_text: str) -> None:
    require(isinstance(q, torch.Tensor) and q.is_cuda, "q must be on CUDA")
    require(q.is_contiguous(), "q must be contiguous")
    require(q.dtype == q_dtype, f"q must be {q_text}")
    require(isinstance(scale, torch.Tensor) and scale.is_cuda, "scale must be on CUDA")
    require(scale.dtype == torch.float32, "scale must be torch.float32")
    require(out_dtype in (torch.float16, torch.bfloat16), "out_dtype must be torch.float16 or torch.bfloat16")
    require(scale.device == q.device, "scale and q must be on the same device")
