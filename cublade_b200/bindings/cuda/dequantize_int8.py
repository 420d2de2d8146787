"""Bindings for symmetric INT8 dequantization ``y = (float(q) * scale_D).to(dtype)``
(same names and contracts as cublade/bindings/cuda/dequantize_int8.py:18-79).
``dtype=torch.float16`` is the reference's "legacy" FP16 output path."""
from __future__ import annotations

import torch

from ... import _native as N
from ._common import check_dequant_input, require


def dequantize_per_tensor_int8(q: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    check_dequant_input(q, scale, dtype, torch.int8, "torch.int8")
    require(scale.numel() == 1, "scale must be a scalar for per-tensor mode")
    with N.device_guard(q):
        y = torch.empty(q.shape, dtype=dtype, device=q.device)
        N.check(N.lib().cb_dequantize_per_tensor_int8(q.data_ptr(), scale.data_ptr(), q.numel(), N.dtype_code(dtype),
                                                      y.data_ptr(), N.stream_ptr(q)))
    return y


def dequantize_per_channel_int8(q: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``q`` is viewed as ``[C, F]`` with ``scale[C]``; ``F`` must be a multiple of 8."""
    check_dequant_input(q, scale, dtype, torch.int8, "torch.int8")
    require(q.dim() >= 1, "q must have at least 1 dim")
    C = q.size(0)
    F = q.numel() // C if C > 0 else 0
    require(scale.numel() == C, "scale must have C elements (size(0) of q)")
    with N.device_guard(q):
        y = torch.empty(q.shape, dtype=dtype, device=q.device)
        N.check(N.lib().cb_dequantize_per_channel_int8(q.data_ptr(), scale.data_ptr(), C, F, N.dtype_code(dtype),
                                                       y.data_ptr(), N.stream_ptr(q)))
    return y


def dequantize_per_group_int8(q_grouped: torch.Tensor, scale: torch.Tensor, group_size: int,
                              dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    check_dequant_input(q_grouped, scale, dtype, torch.int8, "torch.int8")
    require(q_grouped.dim() == 2, "q_grouped must be 2D (num_groups, group_size)")
    require(q_grouped.size(1) == group_size, "q_grouped.size(1) must equal group_size")
    require(0 < group_size <= 4096, "group_size must be in (0, 4096]")
    G = q_grouped.size(0)
    require(scale.numel() == G, "scale must have num_groups elements")
    with N.device_guard(q_grouped):
        y = torch.empty(q_grouped.shape, dtype=dtype, device=q_grouped.device)
        N.check(N.lib().cb_dequantize_per_group_int8(q_grouped.data_ptr(), scale.data_ptr(), G, int(group_size),
                                                     N.dtype_code(dtype), y.data_ptr(), N.stream_ptr(q_grouped)))
    return y


def dequantize_per_axis_int8(q: torch.Tensor, scale: torch.Tensor, axis: int,
                             dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``y = dtype(float(q) * scale[index along axis])`` for any ``axis`` of a contiguous code tensor, in place
    (the inverse of ``quantize_per_axis_int8``; the reference's dequantizer serves axis 0 only,
    cublade/quantization/dequantizers.py:51-53)."""
    check_dequant_input(q, scale, dtype, torch.int8, "torch.int8")
    require(q.dim() >= 1, "q must have at least 1 dim")
    require(-q.dim() <= axis < q.dim(), f"axis {axis} out of range for a {q.dim()}-d tensor")
    axis %= q.dim()
    C = q.size(axis)
    require(scale.numel() == C and scale.is_contiguous(), "scale must be contiguous with one entry per index of axis")
    outer = 1
    for d in q.shape[:axis]:
        outer *= d
    inner = 1
    for d in q.shape[axis + 1:]:
        inner *= d
    with N.device_guard(q):
        y = torch.empty(q.shape, dtype=dtype, device=q.device)
        N.check(N.lib().cb_dequantize_per_axis_int8(q.data_ptr(), scale.data_ptr(), outer, C, inner, N.dtype_code(dtype),
                                                    y.data_ptr(), N.stream_ptr(q)))
    return y


def dequantize_per_group_axis_int8(q: torch.Tensor, scale: torch.Tensor, axis: int, group_size: int,
                                   dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Inverse of ``quantize_per_group_axis_int8``: ``y = dtype(float(q) * scale[group])`` with the groups along
    ``axis`` and the scales flat in the reference's moved-axis order (cublade/quantization/dequantizers.py:58-72),
    computed where the codes lie."""
    check_dequant_input(q, scale, dtype, torch.int8, "torch.int8")
    require(q.dim() >= 1, "q must have at least 1 dim")
    require(-q.dim() <= axis < q.dim(), f"axis {axis} out of range for a {q.dim()}-d tensor")
    axis %= q.dim()
    outer = 1
    for d in q.shape[:axis]:
        outer *= d
    inner = 1
    for d in q.shape[axis + 1:]:
        inner *= d
    C = q.size(axis)
    require(scale.is_contiguous() and scale.numel() * int(group_size) == q.numel(),
            "scale must be contiguous with one entry per group")
    with N.device_guard(q):
        y = torch.empty(q.shape, dtype=dtype, device=q.device)
        N.check(N.lib().cb_dequantize_per_group_axis_int8(q.data_ptr(), scale.data_ptr(), outer, C, inner,
                                                          int(group_size), N.dtype_code(dtype), y.data_ptr(),
                                                          N.stream_ptr(q)))
    return y
