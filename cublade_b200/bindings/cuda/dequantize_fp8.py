"""Binding for per-tensor FP8 E4M3 dequantization
(same name and contract as cublade/bindings/cuda/dequantize_fp8.py:15-35)."""
from __future__ import annotations

import torch

from ... import _native as N
from ._common import check_dequant_input, require


def dequantize_per_tensor_fp8(q: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``y = (float(q) * scale).to(dtype)`` with ``dtype`` float16 or bfloat16.

    Args:
        q: contiguous CUDA float8_e4m3fn tensor.
        scale: float32 CUDA tensor with one element.
        dtype: output dtype.
    """
    check_dequant_input(q, scale, dtype, torch.float8_e4m3fn, "torch.float8_e4m3fn")
    require(scale.numel() == 1, "scale must be a 0-d or 1-element tensor")
    with N.device_guard(q):
        y = torch.empty(q.shape, dtype=dtype, device=q.device)
        N.check(N.lib().cb_dequantize_per_tensor_fp8(q.data_ptr(), scale.data_ptr(), q.numel(), N.dtype_code(dtype),
                                                     y.data_ptr(), N.stream_ptr(q)))
    return y
