"""``quantize_tensor`` and ``quantize_model``: the public quantization entry points.

Signatures, dispatch rules and exception types follow cublade/quantization/quantizers.py:22-224;
the kernels behind them are this package's sm_100a kernels, reached through the C ABI.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn

from ..bindings.cuda.quantize_fp8 import quantize_per_tensor_fp8 as _fp8_tensor
from ..bindings.cuda.quantize_int8 import (
    quantize_per_axis_int8 as _int8_axis,
    quantize_per_channel_int8 as _int8_channel,
    quantize_per_group_axis_int8 as _int8_group_axis,
    quantize_per_group_int8 as _int8_group,
    quantize_per_tensor_int8 as _int8_tensor,
)
from .tensor import QuantizedTensor
from .utils import replace_linear_layers

# (mode, storage dtype) -> binding
_CUDA_QUANT_KERNELS = {
    ("tensor", torch.float8_e4m3fn): _fp8_tensor,
    ("tensor", torch.int8): _int8_tensor,
    ("channel", torch.int8): _int8_channel,
    ("group", torch.int8): _int8_group,
}

_HALF_TYPES = {torch.float16, torch.bfloat16}
_ALLOWED_INPUT_DTYPES = {
    ("tensor", torch.float8_e4m3fn): _HALF_TYPES,
    ("tensor", torch.int8): _HALF_TYPES | {torch.float32},
    ("channel", torch.int8): _HALF_TYPES | {torch.float32},
    ("group", torch.int8): _HALF_TYPES | {torch.float32},
}


def _require_cuda_input(x: torch.Tensor, key, *, what: str) -> None:
    if not x.is_cuda:
        raise ValueError(f"{what}: tensor must be on CUDA, got device={x.device}")
    if not x.is_contiguous():
        raise ValueError(f"{what}: tensor must be contiguous")
    allowed = _ALLOWED_INPUT_DTYPES[key]
    if x.dtype not in allowed:
        raise ValueError(
            f"{what}: tensor dtype must be one of {sorted(str(d) for d in allowed)}, got {x.dtype}"
        )


_ZERO_POINTS = {}


def _zero_scalar(device: torch.device) -> torch.Tensor:
    """0-d float32 zero on ``device``.  One tensor per device is created once and shared by every
    ``QuantizedTensor`` (read-only by convention), so a quantize call launches no fill kernel."""
    z = _ZERO_POINTS.get(device)
    if z is None:
        z = _ZERO_POINTS[device] = torch.zeros((), dtype=torch.float32, device=device)
    return z


def quantize_tensor(
    x: torch.Tensor,
    scheme: str = "symmetric",
    dtype: torch.dtype = torch.int8,
    mode: str = "tensor",
    group_size: int = 32,
    ch_axis: int = 0,
    eps: float = 1e-12,
) -> QuantizedTensor:
    """Quantize a contiguous CUDA tensor.

    * ``scheme``: only ``"symmetric"`` (else ``NotImplementedError``).
    * ``dtype``: ``torch.int8`` (input fp16/bf16/fp32) or ``torch.float8_e4m3fn`` (input fp16/bf16, ``mode="tensor"`` only).
    * ``mode``: ``"tensor"`` one scale; ``"channel"`` one scale per index of ``ch_axis`` (the reference serves
      axis 0 only and raises ``NotImplementedError`` otherwise; here any axis is quantized in place, with the
      result of moving the axis to the front, quantizing and moving it back); ``"group"`` one scale per ``group_size`` consecutive elements
      along ``ch_axis`` (``group_size`` must divide it, else ``ValueError``).  Group scales come back flat,
      ``(num_groups,)``, in the order of the layout with ``ch_axis`` moved last, as in the reference -- which
      gets there through two transposing copies; here a non-last axis is quantized where it lies.
    * an unregistered ``(mode, dtype)`` pair, a CPU / non-contiguous tensor or a wrong input dtype raise ``ValueError``.

    Returns a ``QuantizedTensor`` whose ``zero_point`` is a 0-d float32 zero.
    """
    if scheme != "symmetric":
        raise NotImplementedError(f"quantize_tensor: only scheme='symmetric' is supported, got '{scheme}'")

    key = (mode, dtype)
    kernel = _CUDA_QUANT_KERNELS.get(key)
    if kernel is None:
        raise ValueError(f"No quant kernel registered for mode='{mode}', dtype={dtype}")
    _require_cuda_input(x, key, what="quantize_tensor")

    if mode == "tensor":
        q, scale = kernel(x, eps)
    elif mode == "channel":
        if ch_axis == 0:
            q, scale = kernel(x, eps)
        else:
            # beyond the reference, which stops here with NotImplementedError (quantizers.py:117-120):
            # any axis, quantized where it lies
            if not -x.dim() <= ch_axis < x.dim():
                raise ValueError(f"quantize_tensor: ch_axis {ch_axis} out of range for a {x.dim()}-d tensor")
            q, scale = _int8_axis(x, ch_axis, eps)
    elif mode == "group":
        if not -x.dim() <= ch_axis < x.dim():
            raise IndexError(f"Dimension out of range (expected to be in range of [{-x.dim()}, {x.dim() - 1}], "
                             f"but got {ch_axis})")
        axis, length = ch_axis % x.dim(), x.shape[ch_axis]
        if length % group_size != 0:
            raise ValueError(f"group_size {group_size} must evenly divide axis length {length}")
        if axis == x.dim() - 1:  # groups are contiguous runs already
            q_rows, scale = kernel(x.view(-1, group_size), group_size, eps)
            q = q_rows.view(x.shape)
        else:
            # the reference copies the axis last, quantizes rows and copies the codes back (quantizers.py:122-132);
            # same codes and scales, same scale order, computed where the data lies
            q, scale = _int8_group_axis(x, axis, group_size, eps)
    else:  # unreachable: the registry lookup above already rejected unknown modes
        raise ValueError(f"Unsupported mode '{mode}'; expected tensor / channel / group")

    return QuantizedTensor(q, scale, _zero_scalar(x.device), mode, ch_axis, group_size, dtype, x.dtype)


QUANT_LAYER_REGISTRY = {}


def _init_registry():
    if not QUANT_LAYER_REGISTRY:
        from .linear import cuBladeW8A16LinearLayer
        from .linear_w4a16 import cuBladeW4A16LinearLayer
        from .linear_w8a8 import cuBladeW8A8LinearLayer

        QUANT_LAYER_REGISTRY["w4a16"] = cuBladeW4A16LinearLayer  # reserved, not implemented, in the reference
        QUANT_LAYER_REGISTRY["w8a16"] = cuBladeW8A16LinearLayer
        QUANT_LAYER_REGISTRY["w8a8"] = cuBladeW8A8LinearLayer  # reserved, not implemented, in the reference


def quantize_model(
    model: nn.Module,
    quant_type: str = "w8a16",
    target_modules: Optional[List[str]] = None,
    exclude_modules: Optional[List[str]] = None,
    inplace: bool = True,
    **quant_kwargs,
):
    """Replace the model's ``nn.Linear`` layers by quantized layers.

    ``quant_type`` must be a registered scheme (``"w8a16"``; anything else raises ``ValueError``
    listing what is available).  ``target_modules`` / ``exclude_modules`` select layers by
    substring of their dotted path.  ``inplace=False`` works on a deep copy.  Extra keyword
    arguments (``handle_outliers``, ``outlier_threshold`` ...) go to the layer constructor.
    """
    _init_registry()
    if quant_type not in QUANT_LAYER_REGISTRY:
        available = ", ".join(QUANT_LAYER_REGISTRY.keys())
        raise ValueError(f"Unknown quant_type '{quant_type}'. Available: {available}")
    if not inplace:
        from copy import deepcopy

        model = deepcopy(model)
    replace_linear_layers(
        model,
        target_class=QUANT_LAYER_REGISTRY[quant_type],
        target_modules=target_modules,
        exclude_modules=exclude_modules,
        quant_kwargs=quant_kwargs,
    )
    return model
