"""Bindings for symmetric INT8 quantization: per tensor, per channel (axis 0), per group
(same names and contracts as cublade/bindings/cuda/quantize_int8.py:18-87).

Arithmetic for every reduction domain D (tensor / row / group):
``inv = fp32(127 / max(amax_D, eps))``, ``q = clamp(round_half_even(float(x) * inv), -127, 127)``,
``scale_D = fp32(1 / inv)`` (quantize_int8.cu:120-126).
"""
from __future__ import annotations

import torch

from ... import _native as N
from ._common import check_quant_input, require

_ALLOWED = (torch.float16, torch.bfloat16, torch.float32)
_TEXT = "torch.float16, torch.bfloat16, or torch.float32"


def quantize_per_tensor_int8(x: torch.Tensor, eps: float = 1e-12) -> tuple[torch.Tensor, torch.Tensor]:
    """One scale for the whole tensor. Returns ``(q int8 like x, scale 0-d float32)``."""
    check_quant_input(x, _ALLOWED, _TEXT)
    with N.device_guard(x):
        q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
        scale = torch.empty((), dtype=torch.float32, device=x.device)
        amax = torch.empty(N.per_tensor_scratch_floats(), dtype=torch.float32, device=x.device)
        N.check(N.lib().cb_quantize_per_tensor_int8(x.data_ptr(), N.dtype_code(x.dtype), x.numel(), float(eps),
                                                    q.data_ptr(), scale.data_ptr(), amax.data_ptr(), N.stream_ptr(x)))
    return q, scale


def quantize_per_channel_int8(x: torch.Tensor, eps: float = 1e-12) -> tuple[torch.Tensor, torch.Tensor]:
    """One scale per index of axis 0. ``x`` is viewed as ``[C, F]``; ``F * element_size`` must be
    a multiple of 16 (RuntimeError otherwise, as in the reference). Returns ``(q, scale[C])``."""
    check_quant_input(x, _ALLOWED, _TEXT)
    require(x.dim() >= 1, "x must have at least 1 dim for per-channel quant")
    C = x.size(0)
    F = x.numel() // C if C > 0 else 0
    with N.device_guard(x):
        q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
        scale = torch.empty((C,), dtype=torch.float32, device=x.device)
        N.check(N.lib().cb_quantize_per_channel_int8(x.data_ptr(), N.dtype_code(x.dtype), C, F, float(eps),
                                                     q.data_ptr(), scale.data_ptr(), N.stream_ptr(x)))
    return q, scale


def quantize_per_group_int8(x_grouped: torch.Tensor, group_size: int, eps: float = 1e-12) -> tuple[torch.Tensor, torch.Tensor]:
    """One scale per row of the contiguous ``[num_groups, group_size]`` input.
    ``group_size`` must equal ``x_grouped.size(1)`` and lie in (0, 4096]."""
    check_quant_input(x_grouped, _ALLOWED, _TEXT)
    require(x_grouped.dim() == 2, "x_grouped must be 2D (num_groups, group_size)")
    require(x_grouped.size(1) == group_size, "x_grouped.size(1) must equal group_size")
    require(0 < group_size <= 4096, "group_size must be in (0, 4096]")
    G = x_grouped.size(0)
    with N.device_guard(x_grouped):
        q = torch.empty(x_grouped.shape, dtype=torch.int8, device=x_grouped.device)
        scale = torch.empty((G,), dtype=torch.float32, device=x_grouped.device)
        N.check(N.lib().cb_quantize_per_group_int8(x_grouped.data_ptr(), N.dtype_code(x_grouped.dtype), G,
                                                   int(group_size), float(eps), q.data_ptr(), scale.data_ptr(),
                                                   N.stream_ptr(x_grouped)))
    return q, scale


def quantize_per_axis_int8(x: torch.Tensor, axis: int, eps: float = 1e-12) -> tuple[torch.Tensor, torch.Tensor]:
    """One scale per index of ``axis`` (any axis) of a contiguous tensor, quantized in place without
    moving the axis.  Beyond the reference, whose per-channel kernel serves axis 0 only
    (cublade/quantization/quantizers.py:117-120); the result equals
    ``quantize_per_channel_int8(x.movedim(axis, 0).contiguous())`` moved back, bit for bit.
    Returns ``(q int8 like x, scale float32 [x.shape[axis]])``."""
    check_quant_input(x, _ALLOWED, _TEXT)
    require(x.dim() >= 1, "x must have at least 1 dim for per-channel quant")
    require(-x.dim() <= axis < x.dim(), f"axis {axis} out of range for a {x.dim()}-d tensor")
    axis %= x.dim()
    C = x.size(axis)
    outer = 1
    for d in x.shape[:axis]:
        outer *= d
    inner = 1
    for d in x.shape[axis + 1:]:
        inner *= d
    with N.device_guard(x):
        q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
        scale = torch.empty((C,), dtype=torch.float32, device=x.device)
        scratch = torch.empty((max(C, 1),), dtype=torch.float32, device=x.device)
        N.check(N.lib().cb_quantize_per_axis_int8(x.data_ptr(), N.dtype_code(x.dtype), outer, C, inner, float(eps),
                                                  q.data_ptr(), scale.data_ptr(), scratch.data_ptr(), N.stream_ptr(x)))
    return q, scale


def _outer_c_inner(shape, axis):
    outer = 1
    for d in shape[:axis]:
        outer *= d
    inner = 1
    for d in shape[axis + 1:]:
        inner *= d
    return outer, shape[axis], inner


def quantize_per_group_axis_int8(x: torch.Tensor, axis: int, group_size: int,
                                 eps: float = 1e-12) -> tuple[torch.Tensor, torch.Tensor]:
    """Groups of ``group_size`` consecutive indices along ``axis`` (any axis) of a contiguous tensor,
    quantized where they lie.  Equals the reference's route for ``mode="group"`` with a non-last
    ``ch_axis`` (cublade/quantization/quantizers.py:122-132: move the axis last with a copy, quantize
    rows of ``group_size``, move the codes back with a second copy) bit for bit, scales in the same flat
    order, without either copy.  Returns ``(q int8 like x, scale float32 [x.numel() // group_size])``."""
    check_quant_input(x, _ALLOWED, _TEXT)
    require(x.dim() >= 1, "x must have at least 1 dim for per-group quant")
    require(-x.dim() <= axis < x.dim(), f"axis {axis} out of range for a {x.dim()}-d tensor")
    axis %= x.dim()
    outer, C, inner = _outer_c_inner(tuple(x.shape), axis)
    with N.device_guard(x):
        q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
        scale = torch.empty((x.numel() // max(int(group_size), 1),), dtype=torch.float32, device=x.device)
        N.check(N.lib().cb_quantize_per_group_axis_int8(x.data_ptr(), N.dtype_code(x.dtype), outer, C, inner,
                                                        int(group_size), float(eps), q.data_ptr(), scale.data_ptr(),
                                                        N.stream_ptr(x)))
    return q, scale
