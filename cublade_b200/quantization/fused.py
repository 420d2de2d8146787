"""Fused producers of ``QuantizedTensor``: ops that quantize what they compute instead of writing it
to memory first.  Beyond the reference's API (it names RMSNorm-fused quantization as upcoming work,
README.md:20); the results plug into ``dequantize_tensor`` like any per-channel tensor."""
from __future__ import annotations

from typing import Optional

import torch

from .tensor import QuantizedTensor
from .quantizers import _zero_scalar


def rmsnorm_quantize_tensor(x: torch.Tensor, weight: Optional[torch.Tensor] = None, rms_eps: float = 1e-6,
                            eps: float = 1e-12) -> QuantizedTensor:
    """RMSNorm over the last axis of ``x [..., hidden]`` and per-token symmetric INT8 quantization, one pass.

    Returns a per-channel ``QuantizedTensor`` over the 2-D view ``[rows, hidden]`` (axis 0 = token), so
    ``dequantize_tensor`` gives back the normalised activations; feed ``.data`` / ``.scale`` to an
    int8 GEMM otherwise.  (E4M3 codes per token are available from the binding,
    ``cublade_b200.bindings.cuda.rmsnorm_quantize(..., dtype=torch.float8_e4m3fn)``; the container API, like the
    reference's, knows FP8 only per tensor.)"""
    from ..bindings.cuda.rmsnorm_quant import rmsnorm_quantize

    if not (isinstance(x, torch.Tensor) and x.is_cuda):
        raise ValueError(f"rmsnorm_quantize_tensor: x must be a CUDA tensor, got device={getattr(x, 'device', None)}")
    hidden = x.shape[-1]
    x2d = x.contiguous().view(-1, hidden)
    q, scale = rmsnorm_quantize(x2d, weight, rms_eps=rms_eps, dtype=torch.int8, eps=eps)
    return QuantizedTensor(data=q, scale=scale, zero_point=_zero_scalar(x.device), mode="channel", axis=0,
                           group_size=None, dtype=torch.int8, original_dtype=x.dtype)
