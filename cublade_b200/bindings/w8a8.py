"""Binding for the W8A8 linear (int8 activations x int8 weights on the integer tensor cores).

The reference reserves the layer type (cublade/quantization/quantizers.py:169-171) but has no kernel or
binding for it; the wrapper follows ``bindings/w8a16.py``.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native as N


def w8a8_linear(xq: torch.Tensor, x_scales: torch.Tensor, int8_weights: torch.Tensor, w_scales: torch.Tensor,
                bias: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y[m, n] = out_dtype((float(xq[m] . wq[n]) * x_scales[m]) * w_scales[n] + bias[n])``.

    Args:
        xq: ``[M, K]`` contiguous int8 CUDA tensor (quantized activations, one scale per row).
        x_scales: ``[M]`` float32.
        int8_weights: ``[N, K]`` contiguous int8.  w_scales: ``[N]`` (fp16 / bf16 / fp32).  bias: ``[N]`` or None.
        out_dtype: ``torch.bfloat16`` or ``torch.float16``.
    Raises:
        ValueError for CPU tensors or inconsistent shapes, NotImplementedError for other dtypes.
    """
    if not (isinstance(xq, torch.Tensor) and xq.is_cuda):
        raise ValueError(f"w8a8_linear: activations must be on CUDA, got device={getattr(xq, 'device', None)}")
    if xq.dtype != torch.int8 or int8_weights.dtype != torch.int8:
        raise NotImplementedError("w8a8_linear: activations and weights must be int8")
    if out_dtype not in (torch.float16, torch.bfloat16):
        raise NotImplementedError(f"w8a8_linear: out_dtype must be float16 or bfloat16, got {out_dtype}")
    if xq.dim() != 2 or not xq.is_contiguous() or int8_weights.dim() != 2 or not int8_weights.is_contiguous():
        raise ValueError("w8a8_linear: xq and int8_weights must be contiguous 2-D tensors")
    M, K = xq.shape
    Nout = int8_weights.shape[0]
    if int8_weights.shape[1] != K:
        raise ValueError(f"w8a8_linear: xq has {K} columns but int8_weights has {int8_weights.shape[1]}")
    if K == 0:
        raise ValueError("w8a8_linear: K must be positive")
    if x_scales.dtype != torch.float32 or x_scales.numel() != M or not x_scales.is_contiguous():
        raise ValueError("w8a8_linear: x_scales must be contiguous float32 with one entry per row of xq")
    if w_scales.numel() != Nout or not w_scales.is_contiguous():
        raise ValueError("w8a8_linear: w_scales must be contiguous with one entry per output feature")
    if bias is not None and (bias.numel() != Nout or not bias.is_contiguous()):
        raise ValueError("w8a8_linear: bias must be contiguous with one entry per output feature")
    dev = xq.device
    for name, t in (("x_scales", x_scales), ("int8_weights", int8_weights), ("w_scales", w_scales), ("bias", bias)):
        if t is not None and t.device != dev:
            raise ValueError(f"w8a8_linear: {name} is on {t.device}, activations on {dev}")
    with N.device_guard(xq):
        y = out if out is not None else torch.empty((M, Nout), dtype=out_dtype, device=dev)
        N.check(N.lib().cb_w8a8_linear(
            xq.data_ptr(), x_scales.data_ptr(), M, K, int8_weights.data_ptr(), Nout,
            w_scales.data_ptr(), N.dtype_code(w_scales.dtype),
            N.ptr(bias), N.dtype_code(bias.dtype) if bias is not None else 0,
            y.data_ptr(), y.stride(0), N.dtype_code(out_dtype), N.stream_ptr(xq)))
    return y
