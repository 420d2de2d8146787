"""``cuBladeW4A16LinearLayer``: 4-bit weights (one scale per output feature), 16-bit activations.

The reference reserves ``"w4a16"`` in its layer registry (cublade/quantization/quantizers.py:169-171) without a
layer; this one follows ``cuBladeW8A16LinearLayer`` (cublade/quantization/linear.py:8-81) for the constructor,
``quantize`` and ``forward``.  Buffers: ``int4_weights [out, in // 2]`` uint8 (eight codes per 32-bit word, byte
``j`` = ``code[8i + j] | code[8i + 4 + j] << 4``), ``scales [out]`` in the layer dtype.  ``in_features`` must be a
multiple of 8.  No outlier split.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..bindings.w4a16 import w4_quantize_rows, w4a16_linear
from ._devcache import DeviceBufferCache


class cuBladeW4A16LinearLayer(DeviceBufferCache, nn.Module):
    def __init__(self, in_features, out_features, bias=True, dtype=torch.bfloat16):
        super().__init__()
        if in_features % 8 != 0:
            raise ValueError(f"cuBladeW4A16LinearLayer: in_features must be a multiple of 8, got {in_features}")
        self.in_features = in_features
        self.out_features = out_features
        self.register_buffer("int4_weights", torch.zeros(out_features, in_features // 2, dtype=torch.uint8))
        self.register_buffer("scales", torch.ones(out_features, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype)) if bias else None
        self._dev_cache = {}

    @torch.no_grad()
    def quantize(self, weight_fp: torch.Tensor):
        """Quantize ``weight_fp [out, in]`` per output feature (4 bits, symmetric, codes in [-7, 7]) into the buffers."""
        packed, scale = w4_quantize_rows(weight_fp.cuda().contiguous())
        self.int4_weights.copy_(packed)
        self.scales.copy_(scale.to(self.scales.dtype))

    def forward(self, x):
        if not x.is_cuda:
            raise ValueError(f"cuBladeW4A16LinearLayer.forward: input must be on CUDA, got device={x.device} "
                             "(this build has no CPU path)")
        if x.dtype not in (torch.float16, torch.bfloat16):
            raise NotImplementedError(f"cuBladeW4A16LinearLayer.forward: activations must be float16 or bfloat16, got {x.dtype}")
        if x.shape[-1] != self.in_features:
            raise ValueError(f"cuBladeW4A16LinearLayer.forward: expected {self.in_features} input features, got {x.shape[-1]}")
        dev = x.device
        wq, ws = self._on("int4_weights", dev), self._on("scales", dev)  # cached device copies, no upload per call
        bias = None
        if self.bias is not None:
            bias = self.bias.detach()
            bias = (bias if bias.device == dev else bias.to(dev)).contiguous()
        x2d = x.reshape(-1, self.in_features)
        if x2d.stride(-1) != 1:
            x2d = x2d.contiguous()
        y2d = w4a16_linear(x2d, wq, ws, bias)
        return y2d.view(*x.shape[:-1], self.out_features)
