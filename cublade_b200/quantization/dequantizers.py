"""``dequantize_tensor``: inverse of ``quantize_tensor`` driven by the ``QuantizedTensor`` metadata
(dispatch and errors follow cublade/quantization/dequantizers.py:18-75)."""
from __future__ import annotations

import torch

from ..bindings.cuda.dequantize_fp8 import dequantize_per_tensor_fp8 as _fp8_tensor
from ..bindings.cuda.dequantize_int8 import (
    dequantize_per_axis_int8 as _int8_axis,
    dequantize_per_channel_int8 as _int8_channel,
    dequantize_per_group_axis_int8 as _int8_group_axis,
    dequantize_per_group_int8 as _int8_group,
    dequantize_per_tensor_int8 as _int8_tensor,
)
from .tensor import QuantizedTensor

_CODE_DTYPES = (torch.int8, torch.float8_e4m3fn)


def _require_cuda_dequant_input(q: torch.Tensor, out_dtype: torch.dtype, *, what: str) -> None:
    if not q.is_cuda:
        raise ValueError(f"{what}: tensor must be on CUDA, got device={q.device}")
    if not q.is_contiguous():
        raise ValueError(f"{what}: tensor must be contiguous")
    if q.dtype not in _CODE_DTYPES:
        raise ValueError(f"{what}: q.dtype must be torch.int8 or torch.float8_e4m3fn, got {q.dtype}")
    if out_dtype not in (torch.float16, torch.bfloat16):
        raise ValueError(f"{what}: out_dtype must be float16 or bfloat16, got {out_dtype}")


def dequantize_tensor(qt: QuantizedTensor) -> torch.Tensor:
    """Return ``float(code) * scale`` in ``qt.original_dtype`` (float16 or bfloat16 only, so a
    tensor quantized from float32 cannot come back through this call: ``ValueError``)."""
    _require_cuda_dequant_input(qt.data, qt.original_dtype, what="dequantize_tensor")

    if qt.dtype == torch.float8_e4m3fn:
        if qt.mode != "tensor":
            raise NotImplementedError("FP8 dequant only supports mode='tensor'")
        return _fp8_tensor(qt.data, qt.scale, qt.original_dtype)

    if qt.dtype == torch.int8:
        if qt.mode == "tensor":
            return _int8_tensor(qt.data, qt.scale, qt.original_dtype)
        if qt.mode == "channel":
            if qt.axis != 0:
                # beyond the reference (NotImplementedError at dequantizers.py:51-53): any axis, in place
                return _int8_axis(qt.data, qt.scale, qt.axis, qt.original_dtype)
            return _int8_channel(qt.data, qt.scale, qt.original_dtype)
        if qt.mode == "group":
            if qt.group_size is None:
                raise ValueError("INT8 group dequant needs qt.group_size")
            data = qt.data
            axis, length = qt.axis % data.dim(), data.shape[qt.axis]
            if length % qt.group_size != 0:
                raise ValueError(f"group_size {qt.group_size} must evenly divide axis length {length}")
            if axis == data.dim() - 1:
                return _int8_group(data.view(-1, qt.group_size), qt.scale, qt.group_size,
                                   qt.original_dtype).view(data.shape)
            # a non-last axis, dequantized where the codes lie (the reference moves the axis last with a copy and
            # back with another, dequantizers.py:58-72)
            return _int8_group_axis(data, qt.scale, axis, qt.group_size, qt.original_dtype)
        raise ValueError(f"Unsupported INT8 mode '{qt.mode}'")

    raise ValueError(f"No dequant kernel registered for dtype={qt.dtype}")
