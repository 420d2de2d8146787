"""CPU oracle (PyTorch, IEEE fp32, no fast-math) for the cuBlade quantization hot path.

TEST INFRASTRUCTURE -- never imported by the shipped package.

Every function restates, operation for operation, what the reference's CUDA kernels and
Python layer compute; the file:line each one follows is given in its docstring (paths are
inside the emre570/cublade tree).  This is the "PyTorch formulation runnable on CPU" that
the bit-exact gate is defined against.

Pinning status: the reference ships no tests or golden vectors for this path (its ``/tests``
folder is git-ignored).  The oracle is pinned instead by (1) the independent plain-C
restatement in ``oracle_c.c`` (software E4M3 / bf16 / fp16 conversions), which must agree
bit for bit, and (2) the outputs of the reference's own CUDA kernels, compiled unmodified
into ``oracle/_ref`` and run on a B200, recorded in ``tests/golden/ref_gpu_*.npz``.
The W8A16 GEMM numerics of the reference live in Triton 3.5.1 (``tl.dot``); no reference
artefact pins them, so W8A16 parity is tolerance-based ("parity unpinned" for that op).

Known, deliberate facts encoded here:
  * the emitted scale is ``1 / (qmax / max(amax, eps))``, not ``amax / qmax``;
  * codes come from ``round(x_f32 * inv)``, a multiply by the reciprocal;
  * divisions are IEEE fp32 (the reference's fp64-then-narrow route is identical);
  * ``eps`` is ``float32(1e-12)``.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

E4M3_MAX = 448.0
INT8_MAX = 127.0


def _f32(v: float) -> torch.Tensor:
    return torch.tensor(v, dtype=torch.float32)


# ---------------------------------------------------------------------------------------
# FP8 E4M3 per tensor
# ---------------------------------------------------------------------------------------
def fp8_quantize(x: torch.Tensor, eps: float = 1e-12):
    """cublade/kernels/cuda/quantization/quantize_per_tensor_fp8.cu:38-86 (amax) and :99-131 (cast).

    amax = max|x| in fp32; inv = 448f / fmaxf(amax, eps); q = cvt.rn.satfinite.e4m3(x_f32 * inv);
    scale = 1f / inv.  torch's float32 -> float8_e4m3fn conversion is round-to-nearest-even and
    agrees with the saturating hardware convert everywhere below 464, which x * inv never exceeds.
    Returns (q as float8_e4m3fn, scale as 0-d float32).
    """
    x32 = x.detach().to("cpu").float().reshape(-1)
    amax = x32.abs().max() if x32.numel() else _f32(0.0)
    a = torch.maximum(amax, _f32(eps))
    inv = _f32(E4M3_MAX) / a
    q = (x32 * inv).to(torch.float8_e4m3fn).reshape(x.shape)
    scale = _f32(1.0) / inv
    return q, scale


def fp8_dequantize(q: torch.Tensor, scale: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16):
    """cublade/kernels/cuda/quantization/dequantize_per_tensor_fp8.cu:32-65: y = T_rn(float(q) * scale)."""
    return (q.detach().to("cpu").float() * scale.detach().to("cpu").float()).to(out_dtype)


# ---------------------------------------------------------------------------------------
# INT8 symmetric: one routine over "segments" (tensor = 1 segment, channel = rows, group = rows)
# ---------------------------------------------------------------------------------------
def int8_quantize_rows(x2d: torch.Tensor, eps: float = 1e-12):
    """Rows of ``x2d [S, L]`` quantized independently.

    cublade/kernels/cuda/quantization/quantize_int8.cu:120-165 (tensor), :245-296 (channel),
    :358-370 (group) and int8_pack.cuh:51-56:
      a = fmaxf(amax, eps); inv = float(127.0 / double(a)); scale = float(1.0 / double(inv));
      q = clamp(__float2int_rn(x_f32 * inv), -127, 127).
    Returns (q int8 [S, L], scale float32 [S]).
    """
    x32 = x2d.detach().to("cpu").float()
    if x32.numel() == 0:
        return torch.empty(x32.shape, dtype=torch.int8), torch.empty(x32.shape[0], dtype=torch.float32)
    amax = x32.abs().amax(dim=1)
    a = torch.maximum(amax, _f32(eps))
    inv = (127.0 / a.double()).float()
    scale = (1.0 / inv.double()).float()
    q = torch.round(x32 * inv[:, None]).clamp_(-127, 127).to(torch.int8)
    return q, scale


def int8_quantize_tensor(x: torch.Tensor, eps: float = 1e-12):
    """Per tensor: (q like x, scale 0-d).  quantize_int8.cu:470-484."""
    q, s = int8_quantize_rows(x.reshape(1, -1), eps)
    return q.reshape(x.shape), s.reshape(())


def int8_quantize_channel(x: torch.Tensor, eps: float = 1e-12):
    """Per channel along axis 0: (q like x, scale [C]).  quantize_int8.cu:487-509."""
    q, s = int8_quantize_rows(x.reshape(x.shape[0], -1), eps)
    return q.reshape(x.shape), s


def int8_quantize_axis(x: torch.Tensor, axis: int, eps: float = 1e-12):
    """Per channel along any axis: the axis-0 quantizer (quantize_int8.cu:487-509) applied to the tensor with
    ``axis`` moved to the front, codes moved back.  Returns (q like x, scale [x.shape[axis]])."""
    moved = x.detach().to("cpu").movedim(axis, 0).contiguous()
    q, s = int8_quantize_channel(moved, eps)
    return q.movedim(0, axis).contiguous(), s


def int8_dequantize_axis(q: torch.Tensor, scale: torch.Tensor, axis: int, out_dtype: torch.dtype = torch.bfloat16):
    """y = T_rn(float(q) * scale[index along axis]) (dequantize_int8.cu:81-108 with the axis in place)."""
    shape = [1] * q.dim()
    shape[axis] = -1
    return (q.detach().to("cpu").float() * scale.detach().to("cpu").float().view(shape)).to(out_dtype)


def int8_quantize_group(x_grouped: torch.Tensor, group_size: int, eps: float = 1e-12):
    """Per group on a [num_groups, group_size] view: (q same, scale [num_groups]).  quantize_int8.cu:514-536."""
    assert x_grouped.dim() == 2 and x_grouped.shape[1] == group_size
    return int8_quantize_rows(x_grouped, eps)


def int8_dequantize_rows(q2d: torch.Tensor, scale: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16):
    """cublade/kernels/cuda/quantization/dequantize_int8.cu:39-63, :81-108, :129-133: y = T_rn(float(q) * s_row)."""
    s = scale.detach().to("cpu").float().reshape(-1, 1)
    return (q2d.detach().to("cpu").float() * s).to(out_dtype)


# ---------------------------------------------------------------------------------------
# RMSNorm -> per-row quantize (the fused op the reference announces in README.md:20; the second
# half is int8_quantize_rows / the FP8 cast above applied per row)
# ---------------------------------------------------------------------------------------
def rmsnorm_rows(x2d: torch.Tensor, gamma: Optional[torch.Tensor] = None, rms_eps: float = 1e-6,
                 rstd: Optional[torch.Tensor] = None):
    """RMSNorm of the rows of ``x2d [R, H]`` (fp16 / bf16) with the roundings of an unfused layer:
    ``n = T(x * r)``, ``y = T(float(n) * float(gamma))``.  ``r = 1 / sqrt(mean(x^2) + rms_eps)`` in float32
    from a float64 sum of squares (the exact value a float32 summation approximates), unless ``rstd``
    supplies it.  Returns (y in x's dtype, r float32 [R])."""
    x32 = x2d.detach().to("cpu").float()
    if rstd is None:
        mean = (x32.double().pow(2).sum(dim=1) / x32.shape[1]).float()
        r = (1.0 / torch.sqrt((mean + _f32(rms_eps)).double())).float()
    else:
        r = rstd.detach().to("cpu").float()
    y = (x32 * r[:, None]).to(x2d.dtype)
    if gamma is not None:
        y = (y.float() * gamma.detach().to("cpu").float()[None, :]).to(x2d.dtype)
    return y, r


def rmsnorm_quantize(x2d: torch.Tensor, gamma: Optional[torch.Tensor] = None, rms_eps: float = 1e-6,
                     code: torch.dtype = torch.int8, eps: float = 1e-12, rstd: Optional[torch.Tensor] = None):
    """RMSNorm rows, then quantize every row on its own.  Returns (q, scale [R], y, r)."""
    y, r = rmsnorm_rows(x2d, gamma, rms_eps, rstd)
    if code == torch.int8:
        q, s = int8_quantize_rows(y, eps)
    else:
        y32 = y.float()
        a = torch.maximum(y32.abs().amax(dim=1), _f32(eps))
        inv = _f32(E4M3_MAX) / a
        q = (y32 * inv[:, None]).to(torch.float8_e4m3fn)
        s = _f32(1.0) / inv
    return q, s, y, r


# ---------------------------------------------------------------------------------------
# The Python layer: quantize_tensor / dequantize_tensor on CPU tensors
# ---------------------------------------------------------------------------------------
def quantize_tensor(x: torch.Tensor, dtype=torch.int8, mode: str = "tensor", group_size: int = 32, ch_axis: int = 0,
                    eps: float = 1e-12) -> dict:
    """cublade/quantization/quantizers.py:101-139 on a CPU tensor.  Returns a dict with the
    QuantizedTensor fields (data, scale, zero_point, mode, axis, group_size, dtype, original_dtype)."""
    if dtype == torch.float8_e4m3fn:
        assert mode == "tensor"
        q, scale = fp8_quantize(x, eps)
    elif mode == "tensor":
        q, scale = int8_quantize_tensor(x, eps)
    elif mode == "channel":
        assert ch_axis == 0
        q, scale = int8_quantize_channel(x, eps)
    elif mode == "group":
        moved = x.movedim(ch_axis, -1).contiguous()
        lead, length = moved.shape[:-1], moved.shape[-1]
        assert length % group_size == 0
        qg, scale = int8_quantize_group(moved.reshape(-1, group_size), group_size, eps)
        q = qg.reshape(*lead, length).movedim(-1, ch_axis).contiguous()
    else:
        raise ValueError(mode)
    return dict(data=q, scale=scale, zero_point=torch.zeros((), dtype=torch.float32), mode=mode, axis=ch_axis,
                group_size=group_size, dtype=dtype, original_dtype=x.dtype)


def dequantize_tensor(qt: dict) -> torch.Tensor:
    """cublade/quantization/dequantizers.py:38-75 on the dict produced above."""
    q, scale, out = qt["data"], qt["scale"], qt["original_dtype"]
    if qt["dtype"] == torch.float8_e4m3fn:
        return fp8_dequantize(q, scale, out)
    if qt["mode"] == "tensor":
        return int8_dequantize_rows(q.reshape(1, -1), scale.reshape(1), out).reshape(q.shape)
    if qt["mode"] == "channel":
        return int8_dequantize_rows(q.reshape(q.shape[0], -1), scale, out).reshape(q.shape)
    G = qt["group_size"]
    moved = q.movedim(qt["axis"], -1).contiguous()
    lead, length = moved.shape[:-1], moved.shape[-1]
    y = int8_dequantize_rows(moved.reshape(-1, G), scale, out)
    return y.reshape(*lead, length).movedim(-1, qt["axis"]).contiguous()


# ---------------------------------------------------------------------------------------
# W8A16 linear
# ---------------------------------------------------------------------------------------
def detect_outlier_columns(weight: torch.Tensor, threshold: float = 6.0):
    """cublade/quantization/outlier_utils.py:33-35."""
    return ((weight.abs().max(dim=0).values > threshold).nonzero(as_tuple=True)[0]).tolist()


def w8a16_quantize(weight: torch.Tensor, layer_dtype: torch.dtype, outlier_cols: Optional[Sequence[int]] = None):
    """cublade/quantization/linear.py:35-81.  Returns dict(int8_weights, scales (layer dtype),
    scales_f32, normal_cols, outlier_cols, outlier_weights)."""
    w = weight.detach().to("cpu")
    if outlier_cols is not None and len(outlier_cols) > 0:
        oc = list(outlier_cols)
        nc = sorted(set(range(w.shape[1])) - set(oc))  # outlier_utils.py:70-71
        w_normal, w_out = w[:, nc].contiguous(), w[:, oc]
    else:
        oc, nc, w_normal, w_out = [], list(range(w.shape[1])), w.contiguous(), None
    q, s = int8_quantize_channel(w_normal)
    return dict(int8_weights=q, scales=s.to(layer_dtype), scales_f32=s, normal_cols=nc, outlier_cols=oc,
                outlier_weights=w_out)


def w8a16_forward(x: torch.Tensor, layer: dict, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The reference forward, cublade/quantization/linear.py:93-137, in its GPU rounding order:
    y = T(fp32acc(x . T(q)^T)); y = T(y * scales_T); (+ T(x_out . W_out^T)); y = T(y + bias).
    fp32 accumulation is done as an fp32 matmul on the widened operands (exact products)."""
    T = x.dtype
    x2d = x.detach().to("cpu").reshape(-1, x.shape[-1])
    q = layer["int8_weights"]
    oc = layer["outlier_cols"]
    if oc:
        xn = x2d[:, layer["normal_cols"]]
        y = (xn.float() @ q.float().t()).to(T)
        y = (y * layer["scales"].to(T)).to(T)
        wo = layer["outlier_weights"].to(T)
        y = y + (x2d[:, oc].float() @ wo.float().t()).to(T)
    else:
        y = (x2d.float() @ q.float().t()).to(T)
        y = (y * layer["scales"].to(T)).to(T)
    if bias is not None:
        y = y + bias.to(T)
    return y.reshape(*x.shape[:-1], q.shape[0])


def w8a8_forward(x: torch.Tensor, layer: dict, bias: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None, xq: Optional[torch.Tensor] = None,
                 xs: Optional[torch.Tensor] = None) -> torch.Tensor:
    """W8A8 linear: per-token INT8 quantization of x (int8_quantize_rows on the [tokens, in] view, i.e.
    quantize_int8.cu:487-509 with axis 0 = token), exact integer dot products, then
    ``T((float(acc) * x_scale[m]) * w_scale[n] + bias[n])`` -- each step one float32 operation.
    ``layer`` as returned by ``w8a16_quantize`` (int8 weights [N, K], scales in the layer dtype)."""
    x2d = x.detach().to("cpu").reshape(-1, x.shape[-1])
    if xq is None:
        xq, xs = int8_quantize_rows(x2d)
    acc = (xq.detach().to("cpu").double() @ layer["int8_weights"].double().t()).to(torch.int32)  # exact: |acc| < 2^53
    y = acc.float() * xs.detach().to("cpu").float()[:, None]
    y = y * layer["scales"].float()[None, :]
    if bias is not None:
        y = y + bias.detach().to("cpu").float()[None, :]
    y = y.to(out_dtype or x.dtype)
    return y.reshape(*x.shape[:-1], layer["int8_weights"].shape[0])


def w8a16_forward_fp64(x: torch.Tensor, layer: dict, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Same contraction in float64 with the (layer-dtype) scales applied unrounded: the
    mathematically exact value both the reference and the fused kernel approximate."""
    x2d = x.detach().to("cpu").reshape(-1, x.shape[-1]).double()
    q = layer["int8_weights"].double()
    oc = layer["outlier_cols"]
    if oc:
        y = (x2d[:, layer["normal_cols"]] @ q.t()) * layer["scales"].double()
        y = y + x2d[:, oc] @ layer["outlier_weights"].to(x.dtype).double().t()
    else:
        y = (x2d @ q.t()) * layer["scales"].double()
    if bias is not None:
        y = y + bias.double()
    return y.reshape(*x.shape[:-1], q.shape[0])


# ------------------------------------------------------------------------------------------------
# W4A16 (layer type reserved by the reference's registry comment, cublade/quantization/quantizers.py:169-171,
# without an implementation): the reference's symmetric per-channel arithmetic at qmax = 7.
# ------------------------------------------------------------------------------------------------
def int4_quantize_rows(x2d: torch.Tensor, eps: float = 1e-12):
    """Rows of ``x2d [S, L]``: the INT8 row quantizer above (quantize_int8.cu:245-296, int8_pack.cuh:51-56) with
    qmax = 7.  Returns (codes int8 [S, L] in [-7, 7], scale float32 [S])."""
    x32 = x2d.detach().to("cpu").float()
    amax = x32.abs().amax(dim=1) if x32.shape[1] else torch.zeros(x32.shape[0])
    a = torch.maximum(amax, _f32(eps))
    inv = (7.0 / a.double()).float()
    scale = (1.0 / inv.double()).float()
    q = torch.round(x32 * inv[:, None]).clamp_(-7, 7).to(torch.int8)
    return q, scale


def int4_pack(codes: torch.Tensor) -> torch.Tensor:
    """int8 codes ``[N, K]`` (K % 8 == 0, values in [-8, 7]) -> uint8 ``[N, K // 2]``: byte ``4i + j`` of a row is
    ``code[8i + j] & 15 | (code[8i + 4 + j] & 15) << 4``."""
    n, k = codes.shape
    c = (codes.to(torch.int16) & 15).view(n, k // 8, 2, 4)
    return (c[:, :, 0, :] | (c[:, :, 1, :] << 4)).to(torch.uint8).reshape(n, k // 2)


def int4_unpack(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of ``int4_pack``."""
    n, half = packed.shape
    b = packed.to(torch.int16).view(n, half // 4, 4)
    lo, hi = b & 15, (b >> 4) & 15
    c = torch.stack([lo, hi], dim=2).reshape(n, half * 2)
    return torch.where(c >= 8, c - 16, c).to(torch.int8)


def w4a16_quantize(weight: torch.Tensor, layer_dtype: torch.dtype):
    """A layer dict for ``w8a16_forward`` (the forward is the W8A16 one on 4-bit codes) plus ``int4_weights``."""
    q, s = int4_quantize_rows(weight.detach().to("cpu").contiguous())
    return dict(int8_weights=q, int4_weights=int4_pack(q), scales=s.to(layer_dtype), scales_f32=s,
                normal_cols=list(range(weight.shape[1])), outlier_cols=[], outlier_weights=None)
