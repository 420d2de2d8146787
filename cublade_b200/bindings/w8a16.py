"""Binding for the fused W8A16 linear kernel (``cb_w8a16_linear``).

Stands in for the chain the reference runs per forward call -- int8 -> 16-bit cast of the whole
weight, transpose copy, Triton GEMM, scale multiply, bias add (cublade/quantization/linear.py:123-135,
cublade/bindings/triton/matmul.py:17-132) -- with one kernel that reads the int8 weights once.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native as N

PATH_AUTO, PATH_STREAM, PATH_TENSOR_CORE, PATH_TENSOR_CORE_SINGLE = 0, 1, 2, 3


def _check_2d(t: torch.Tensor, name: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with unit inner stride")


def gather_columns(src: torch.Tensor, cols: torch.Tensor, ld_dst: Optional[int] = None,
                   pad_to: Optional[int] = None) -> torch.Tensor:
    """``src[:, cols]`` for a 2-D CUDA tensor of a 2- or 4-byte dtype; the result's row stride is
    ``ld_dst`` elements (default: the column count rounded up to a multiple of 8).  With ``pad_to``
    the result has ``pad_to`` columns, the ones behind ``len(cols)`` zero."""
    _check_2d(src, "src")
    if not src.is_cuda or not cols.is_cuda or cols.dtype != torch.int64:
        raise ValueError("gather_columns: src and cols (int64) must be CUDA tensors")
    M, n = src.shape[0], cols.numel()
    width = n if pad_to is None else int(pad_to)
    if width < n:
        raise ValueError("gather_columns: pad_to is smaller than the number of columns")
    ld = ld_dst if ld_dst is not None else (width + 7) // 8 * 8
    with N.device_guard(src):
        buf = torch.empty((M, max(ld, 1)), dtype=src.dtype, device=src.device)
        N.check(N.lib().cb_gather_columns_padded(src.data_ptr(), M, src.stride(0), cols.data_ptr(), n, width,
                                                 buf.data_ptr(), buf.stride(0), src.element_size(), N.stream_ptr(src)))
    return buf[:, :width]


def w8a16_linear(
    x2d: torch.Tensor,
    int8_weights: torch.Tensor,
    scales: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    x_outlier: Optional[torch.Tensor] = None,
    w_outlier: Optional[torch.Tensor] = None,
    path: int = PATH_AUTO,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """``y = (x2d @ int8_weights.T) * scales [+ x_outlier @ w_outlier.T] [+ bias]`` with fp32
    accumulation, rounded to ``x2d.dtype`` after the GEMM, after the scales, after the outlier product and after the
    bias -- the places where the reference's chain of kernels rounds (cublade/quantization/linear.py:97-135).

    Args:
        x2d: ``[M, K]`` float16 / bfloat16 CUDA tensor (rows may be strided).
        int8_weights: ``[N, K]`` contiguous int8.
        scales: ``[N]`` float16 / bfloat16 / float32.
        bias: optional ``[N]``.
        x_outlier, w_outlier: optional ``[M, KO]`` / ``[N, KO]`` in ``x2d.dtype`` (LLM.int8 side product).
        path: 0 automatic, 1 weight-streaming kernel, 2 tcgen05 CTA-pair kernel, 3 tcgen05 single-CTA kernel.
    """
    if not x2d.is_cuda:
        raise ValueError(f"w8a16_linear: activations must be on CUDA, got device={x2d.device}")
    if x2d.dtype not in (torch.float16, torch.bfloat16):
        raise NotImplementedError(f"w8a16_linear: activations must be float16 or bfloat16, got {x2d.dtype}")
    _check_2d(x2d, "x2d")
    if int8_weights.dtype != torch.int8 or int8_weights.dim() != 2 or not int8_weights.is_contiguous():
        raise ValueError("w8a16_linear: int8_weights must be a contiguous 2-D int8 tensor")
    M, K = x2d.shape
    Nout = int8_weights.shape[0]
    if int8_weights.shape[1] != K:
        raise ValueError(f"w8a16_linear: x2d has {K} columns but int8_weights has {int8_weights.shape[1]}")
    if scales.numel() != Nout or not scales.is_contiguous():
        raise ValueError("w8a16_linear: scales must be contiguous with one entry per output feature")
    if bias is not None and (bias.numel() != Nout or not bias.is_contiguous()):
        raise ValueError("w8a16_linear: bias must be contiguous with one entry per output feature")
    dev = x2d.device
    for name, t in (("int8_weights", int8_weights), ("scales", scales), ("bias", bias), ("x_outlier", x_outlier),
                    ("w_outlier", w_outlier)):
        if t is not None and t.device != dev:
            raise ValueError(f"w8a16_linear: {name} is on {t.device}, activations on {dev}")
    KO = 0
    if x_outlier is not None or w_outlier is not None:
        if x_outlier is None or w_outlier is None:
            raise ValueError("w8a16_linear: x_outlier and w_outlier come together")
        _check_2d(x_outlier, "x_outlier")
        KO = x_outlier.shape[1]
        if (x_outlier.shape[0] != M or w_outlier.shape != (Nout, KO) or not w_outlier.is_contiguous()
                or x_outlier.dtype != x2d.dtype or w_outlier.dtype != x2d.dtype):
            raise ValueError("w8a16_linear: outlier operands must be [M, KO] / contiguous [N, KO] in the activation dtype")
    L = N.lib()
    with N.device_guard(x2d):
        y = out if out is not None else torch.empty((M, Nout), dtype=x2d.dtype, device=dev)
        ws_bytes = int(L.cb_w8a16_workspace_bytes(M, Nout, K))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev) if ws_bytes else None
        N.check(L.cb_w8a16_linear(
            x2d.data_ptr(), M, K, x2d.stride(0), int8_weights.data_ptr(), Nout,
            scales.data_ptr(), N.dtype_code(scales.dtype),
            N.ptr(bias), N.dtype_code(bias.dtype) if bias is not None else 0,
            N.ptr(x_outlier) if KO else None, x_outlier.stride(0) if KO else 0,
            N.ptr(w_outlier) if KO else None, KO,
            y.data_ptr(), y.stride(0), N.dtype_code(x2d.dtype),
            N.ptr(ws), ws_bytes, int(path), N.stream_ptr(x2d)))
    return y
