"""Bindings for the W4A16 path: 4-bit weight quantizer, unpacker and linear.

The reference reserves the layer type (cublade/quantization/quantizers.py:169-171) but has no kernel, binding
or storage format for it; the wrappers follow ``bindings/w8a16.py``.  Packed layout: row ``n`` is ``K / 2``
bytes, 32-bit word ``i`` of a row holds the codes ``k = 8i .. 8i + 7`` as two's-complement nibbles, byte ``j``
= ``code[8i + j] | code[8i + 4 + j] << 4``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _native as N


def _check_cuda(name: str, t: torch.Tensor) -> None:
    if not (isinstance(t, torch.Tensor) and t.is_cuda):
        raise ValueError(f"{name}: tensor must be on CUDA, got device={getattr(t, 'device', None)} (this build has no CPU path)")


def w4_quantize_rows(weight: torch.Tensor, eps: float = 1e-12) -> Tuple[torch.Tensor, torch.Tensor]:
    """``weight [N, K]`` (fp16 / bf16 / fp32, K % 8 == 0) -> ``(packed uint8 [N, K // 2], scale float32 [N])``.

    Symmetric per row with qmax = 7: ``a = max(amax, eps); inv = float(7 / double(a)); scale = float(1 / double(inv));
    code = clamp(rint(w * inv), -7, 7)`` (the reference's INT8 arithmetic, quantize_int8.cu:245-296, at 4 bits).
    """
    _check_cuda("w4_quantize_rows", weight)
    if weight.dim() != 2 or not weight.is_contiguous():
        raise ValueError("w4_quantize_rows: weight must be a contiguous 2-D tensor")
    if weight.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise NotImplementedError(f"w4_quantize_rows: unsupported dtype {weight.dtype}")
    n, k = weight.shape
    if k % 8 != 0:
        raise ValueError(f"w4_quantize_rows: in_features must be a multiple of 8, got {k}")
    with N.device_guard(weight):
        packed = torch.empty((n, k // 2), dtype=torch.uint8, device=weight.device)
        scale = torch.empty((n,), dtype=torch.float32, device=weight.device)
        N.check(N.lib().cb_w4_quantize_rows(weight.data_ptr(), N.dtype_code(weight.dtype), n, k, float(eps),
                                            packed.data_ptr(), scale.data_ptr(), N.stream_ptr(weight)))
    return packed, scale


def w4_unpack(packed: torch.Tensor) -> torch.Tensor:
    """``packed uint8 [N, K // 2]`` -> int8 codes ``[N, K]``."""
    _check_cuda("w4_unpack", packed)
    if packed.dim() != 2 or not packed.is_contiguous() or packed.dtype != torch.uint8:
        raise ValueError("w4_unpack: packed must be a contiguous 2-D uint8 tensor")
    n, half = packed.shape
    if half % 4 != 0:
        raise ValueError("w4_unpack: rows must hold a multiple of 8 codes")
    with N.device_guard(packed):
        out = torch.empty((n, 2 * half), dtype=torch.int8, device=packed.device)
        N.check(N.lib().cb_w4_unpack(packed.data_ptr(), n, 2 * half, out.data_ptr(), N.stream_ptr(packed)))
    return out


def w4a16_linear(x: torch.Tensor, int4_weights: torch.Tensor, scales: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y[m, n] = T((sum_k x[m, k] * code[n, k]) * scales[n] + bias[n])`` with fp32 accumulation.

    Args:
        x: ``[M, K]`` fp16 / bf16 CUDA tensor, unit stride along K.
        int4_weights: ``[N, K // 2]`` contiguous uint8 (packed layout above).  scales: ``[N]``.  bias: ``[N]`` or None.
    Raises:
        ValueError for CPU tensors or inconsistent shapes, NotImplementedError for other dtypes.
    """
    _check_cuda("w4a16_linear", x)
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise NotImplementedError(f"w4a16_linear: activations must be float16 or bfloat16, got {x.dtype}")
    if x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("w4a16_linear: x must be 2-D with unit stride along its last axis")
    if int4_weights.dim() != 2 or not int4_weights.is_contiguous() or int4_weights.dtype != torch.uint8:
        raise ValueError("w4a16_linear: int4_weights must be a contiguous 2-D uint8 tensor")
    M, K = x.shape
    Nout = int4_weights.shape[0]
    if int4_weights.shape[1] * 2 != K:
        raise ValueError(f"w4a16_linear: x has {K} columns but int4_weights holds {int4_weights.shape[1] * 2} codes per row")
    if K == 0 or K % 8 != 0:
        raise ValueError(f"w4a16_linear: in_features must be a positive multiple of 8, got {K}")
    if scales.numel() != Nout or not scales.is_contiguous():
        raise ValueError("w4a16_linear: scales must be contiguous with one entry per output feature")
    if bias is not None and (bias.numel() != Nout or not bias.is_contiguous()):
        raise ValueError("w4a16_linear: bias must be contiguous with one entry per output feature")
    dev = x.device
    for name, t in (("int4_weights", int4_weights), ("scales", scales), ("bias", bias)):
        if t is not None and t.device != dev:
            raise ValueError(f"w4a16_linear: {name} is on {t.device}, activations on {dev}")
    with N.device_guard(x):
        y = out if out is not None else torch.empty((M, Nout), dtype=x.dtype, device=dev)
        ws_bytes = int(N.lib().cb_w4a16_workspace_bytes(M, Nout, K)) if (M > 16 or K % 128 or Nout % 16 or
                                                                          (x.stride(0) * 2) % 16 or x.data_ptr() % 16 or
                                                                          int4_weights.data_ptr() % 16) else 0
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev) if ws_bytes else None
        N.check(N.lib().cb_w4a16_linear(
            x.data_ptr(), N.dtype_code(x.dtype), M, K, x.stride(0), int4_weights.data_ptr(), Nout,
            scales.data_ptr(), N.dtype_code(scales.dtype), N.ptr(bias), N.dtype_code(bias.dtype) if bias is not None else 0,
            y.data_ptr(), y.stride(0), N.ptr(ws), ws_bytes, N.stream_ptr(x)))
    return y
