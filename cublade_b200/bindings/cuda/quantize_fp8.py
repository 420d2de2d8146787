"""Binding for per-tensor FP8 E4M3 quantization
(same name and contract as cublade/bindings/cuda/quantize_fp8.py:15-34)."""
from __future__ import annotations

import torch

from ... import _native as N
from ._common import check_quant_input


def quantize_per_tensor_fp8(x: torch.Tensor, eps: float = 1e-12) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-tensor symmetric FP8 (E4M3) quantization on the GPU.

    ``inv = 448 / max(amax, eps)``; ``q = e4m3(float(x) * inv)`` (round to nearest
    even, saturating); ``scale = 1 / inv``.  Note the emitted scale is the
    reciprocal of ``inv`` (what the reference kernel writes,
    quantize_per_tensor_fp8.cu:99-102), which can sit 1 ULP from ``amax / 448``.

    Args:
        x: contiguous CUDA tensor, float16 or bfloat16.
        eps: floor on amax.
    Returns:
        ``(q, scale)``: ``q`` float8_e4m3fn with x's shape, ``scale`` 0-d float32.
    """
    check_quant_input(x, (torch.float16, torch.bfloat16), "torch.float16 or torch.bfloat16")
    with N.device_guard(x):
        q = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
        scale = torch.empty((), dtype=torch.float32, device=x.device)
        amax = torch.empty(N.per_tensor_scratch_floats(), dtype=torch.float32, device=x.device)
        N.check(N.lib().cb_quantize_per_tensor_fp8(x.data_ptr(), N.dtype_code(x.dtype), x.numel(), float(eps),
                                                   q.data_ptr(), scale.data_ptr(), amax.data_ptr(), N.stream_ptr(x)))
    return q, scale
