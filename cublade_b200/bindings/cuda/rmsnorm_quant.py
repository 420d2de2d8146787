"""Binding for the fused RMSNorm -> per-row quantize kernel.

The reference announces this op as upcoming work (README.md:20) without shipping it, so there is
no reference binding to mirror; the wrapper follows the conventions of the quantize bindings next
to it (contiguous CUDA input, RuntimeError on contract violations, outputs allocated here).
"""
from __future__ import annotations

from typing import Optional

import torch

from ... import _native as N
from ._common import check_quant_input, require

_CODE_KIND = {torch.int8: 0, torch.float8_e4m3fn: 1}


def rmsnorm_quantize(x: torch.Tensor, weight: Optional[torch.Tensor] = None, rms_eps: float = 1e-6,
                     dtype: torch.dtype = torch.int8, eps: float = 1e-12, return_normed: bool = False,
                     return_rstd: bool = False):
    """RMSNorm over the last axis followed by symmetric per-row quantization, in one pass over ``x``.

    ``r = 1 / sqrt(mean(x^2, -1) + rms_eps)``; ``n = x.dtype(x * r)``; ``y = x.dtype(n * weight)``;
    ``inv = qmax / max(max|y|, eps)`` per row; ``q = code(float(y) * inv)``; ``scale = 1 / inv``.

    Args:
        x: contiguous CUDA tensor ``[..., hidden]``, float16 or bfloat16.
        weight: ``[hidden]`` in ``x.dtype`` (the RMSNorm gain) or None.
        dtype: ``torch.int8`` (codes in [-127, 127]) or ``torch.float8_e4m3fn``.
        return_normed / return_rstd: also return ``y`` (like ``x``) / ``r`` (float32, one per row).
    Returns:
        ``(q like x in dtype, scale float32 [rows])`` followed by the optional extras, rows = x.numel() / hidden.
    """
    check_quant_input(x, (torch.float16, torch.bfloat16), "torch.float16 or torch.bfloat16")
    require(x.dim() >= 1, "x must have at least 1 dim")
    require(dtype in _CODE_KIND, "dtype must be torch.int8 or torch.float8_e4m3fn")
    hidden = x.shape[-1]
    rows = x.numel() // hidden if hidden > 0 else 0
    if weight is not None:
        require(weight.is_cuda and weight.device == x.device, "weight must be on x's device")
        require(weight.dtype == x.dtype, "weight must have x's dtype")
        require(weight.is_contiguous() and weight.numel() == hidden, "weight must be contiguous with one entry per feature")
    with N.device_guard(x):
        q = torch.empty(x.shape, dtype=dtype, device=x.device)
        scale = torch.empty((rows,), dtype=torch.float32, device=x.device)
        y = torch.empty_like(x) if return_normed else None
        rstd = torch.empty((rows,), dtype=torch.float32, device=x.device) if return_rstd else None
        N.check(N.lib().cb_rmsnorm_quantize(x.data_ptr(), N.dtype_code(x.dtype), rows, hidden, N.ptr(weight),
                                            float(rms_eps), float(eps), _CODE_KIND[dtype], q.data_ptr(), scale.data_ptr(),
                                            N.ptr(y), N.ptr(rstd), N.stream_ptr(x)))
    out = (q, scale)
    if return_normed:
        out += (y,)
    if return_rstd:
        out += (rstd,)
    return out
