"""``cuBladeW8A8LinearLayer``: int8 weights (one scale per output feature) and int8 activations
(one scale per token, computed on the fly), multiplied on the integer tensor cores.

The reference reserves ``"w8a8"`` in its layer registry (cublade/quantization/quantizers.py:169-171) without a
layer; this one follows ``cuBladeW8A16LinearLayer`` (cublade/quantization/linear.py:8-81) for the constructor,
the buffers (``int8_weights [out, in]``, ``scales [out]``) and ``quantize``.  Forward: per-token symmetric INT8
quantization of the activations (the per-channel quantizer on the ``[tokens, in]`` view), then
``y = T((float(xq . wq) * x_scale[token]) * scales[out] + bias)`` with exact int32 accumulation.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..bindings.cuda.quantize_int8 import quantize_per_axis_int8, quantize_per_channel_int8
from ..bindings.w8a8 import w8a8_linear
from ._devcache import DeviceBufferCache
from .quantizers import quantize_tensor
from .tensor import QuantizedTensor


class cuBladeW8A8LinearLayer(DeviceBufferCache, nn.Module):
    def __init__(self, in_features, out_features, bias=True, dtype=torch.bfloat16):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.register_buffer("int8_weights", torch.empty(out_features, in_features, dtype=torch.int8))
        self.register_buffer("scales", torch.ones(out_features, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype)) if bias else None
        self._dev_cache = {}

    @torch.no_grad()
    def quantize(self, weight_fp: torch.Tensor):
        """Quantize ``weight_fp [out, in]`` per output feature (INT8, symmetric) into the buffers."""
        qt = quantize_tensor(weight_fp.cuda().contiguous(), scheme="symmetric", dtype=torch.int8, mode="channel", ch_axis=0)
        self.int8_weights.copy_(qt.data)
        self.scales.copy_(qt.scale.reshape(-1).to(self.scales.dtype))

    def forward(self, x, out_dtype: Optional[torch.dtype] = None):
        """``x``: a 16-bit CUDA tensor ``[..., in]`` (quantized per token here), or a per-token ``QuantizedTensor``
        over the ``[tokens, in]`` view (e.g. from ``rmsnorm_quantize_tensor``), which skips that pass."""
        if isinstance(x, QuantizedTensor):
            if x.dtype != torch.int8 or x.mode != "channel" or x.axis != 0 or x.data.dim() != 2:
                raise ValueError("cuBladeW8A8LinearLayer.forward: a QuantizedTensor input must be INT8, per channel along axis 0 "
                                 "of a [tokens, in] tensor")
            xq, xs, lead, dtype = x.data, x.scale, x.data.shape[:-1], out_dtype or x.original_dtype
        else:
            if not x.is_cuda:
                raise ValueError(f"cuBladeW8A8LinearLayer.forward: input must be on CUDA, got device={x.device} "
                                 "(this build has no CPU path)")
            if x.dtype not in (torch.float16, torch.bfloat16):
                raise NotImplementedError(f"cuBladeW8A8LinearLayer.forward: activations must be float16 or bfloat16, got {x.dtype}")
            lead, dtype = x.shape[:-1], out_dtype or x.dtype
            x2d = x.reshape(-1, self.in_features).contiguous()
            # the one-pass row kernel wants rows of a multiple of 16 bytes; any other width goes the per-axis way
            if (self.in_features * x2d.element_size()) % 16 == 0:
                xq, xs = quantize_per_channel_int8(x2d)
            else:
                xq, xs = quantize_per_axis_int8(x2d, 0)
        if xq.shape[-1] != self.in_features:
            raise ValueError(f"cuBladeW8A8LinearLayer.forward: expected {self.in_features} input features, got {xq.shape[-1]}")
        dev = xq.device
        wq, ws = self._on("int8_weights", dev), self._on("scales", dev)  # cached device copies, no upload per call
        bias = None
        if self.bias is not None:
            bias = self.bias.detach()
            bias = (bias if bias.device == dev else bias.to(dev)).contiguous()
        y2d = w8a8_linear(xq, xs, wq, ws, bias, out_dtype=dtype)
        return y2d.view(*lead, self.out_features)
