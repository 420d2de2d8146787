"""``cuBladeW8A16LinearLayer``: int8 weights with one scale per output feature, 16-bit activations.

Buffer names, dtypes and shapes (``int8_weights [out, in]``, ``scales [out]``, ``outlier_weights``,
``normal_cols``, ``outlier_cols``) and the constructor / ``quantize`` / ``forward`` contract follow
cublade/quantization/linear.py:8-137, so ``state_dict()`` is interchangeable.  The forward pass
is one fused kernel (see ``bindings/w8a16.py``) whose epilogue rounds in the same places as the
reference's chain of kernels, so outputs agree with the reference's bit for bit up to the order of
the fp32 accumulation.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..bindings.w8a16 import gather_columns, w8a16_linear
from ._devcache import DeviceBufferCache
from .outlier_utils import separate_outliers
from .quantizers import quantize_tensor


class cuBladeW8A16LinearLayer(DeviceBufferCache, nn.Module):
    def __init__(self, in_features, out_features, bias=True, dtype=torch.bfloat16, handle_outliers=False,
                 outlier_threshold=6.0):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.handle_outliers = handle_outliers
        self.outlier_threshold = outlier_threshold

        self.register_buffer("int8_weights", torch.empty(out_features, in_features, dtype=torch.int8))
        self.register_buffer("scales", torch.ones(out_features, dtype=dtype))
        # only populated by quantize() when handle_outliers=True
        self.register_buffer("outlier_weights", None)
        self.register_buffer("normal_cols", None)
        self.register_buffer("outlier_cols", None)
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype)) if bias else None
        self._dev_cache = {}

    @torch.no_grad()
    def quantize(self, weight_fp: torch.Tensor):
        """Quantize ``weight_fp [out, in]`` per output feature (INT8, symmetric) into the buffers.

        With ``handle_outliers`` the columns whose peak magnitude exceeds ``outlier_threshold`` are
        kept aside in their original dtype (``outlier_weights``), only the remaining columns are
        quantized, and ``int8_weights`` becomes ``[out, in - n_outliers]``.  The weight is moved
        to the GPU for the kernel; its row length in bytes must be a multiple of 16.
        """
        self._dev_cache = {}
        if self.handle_outliers:
            w_normal, w_outlier, normal_cols, outlier_cols = separate_outliers(weight_fp, threshold=self.outlier_threshold)
            self.outlier_weights = w_outlier
            self.normal_cols = torch.tensor(normal_cols, dtype=torch.long)
            self.outlier_cols = torch.tensor(outlier_cols, dtype=torch.long)
            qt = quantize_tensor(w_normal.cuda().contiguous(), scheme="symmetric", dtype=torch.int8, mode="channel",
                                 ch_axis=0)
            self.int8_weights = qt.data
        else:
            qt = quantize_tensor(weight_fp.cuda().contiguous(), scheme="symmetric", dtype=torch.int8, mode="channel",
                                 ch_axis=0)
            self.int8_weights.copy_(qt.data)

        assert torch.allclose(qt.zero_point, torch.zeros_like(qt.zero_point)), "Expect symmetric zp=0"
        scale_1d = qt.scale.squeeze()
        assert scale_1d.ndim == 1 and scale_1d.numel() == self.out_features
        self.scales.copy_(scale_1d.to(self.scales.dtype))

    def _padded_weights(self, dev: torch.device, width: int) -> torch.Tensor:
        """``int8_weights`` on ``dev`` with zero columns appended up to ``width``.

        The tensor-core kernels fetch the int8 rows with TMA, whose row stride must be a multiple of 16
        bytes.  ``state_dict()`` keeps the stored shape -- the padded copy lives only in this cache."""
        src = self.int8_weights

        def build():
            padded = torch.zeros((src.shape[0], width), dtype=torch.int8, device=dev)
            padded[:, : src.shape[1]].copy_(src)
            return padded

        return self._cached(("int8_weights_padded", dev, width), (src,), build)

    def _full_k_weights(self, dev: torch.device) -> torch.Tensor:
        """The int8 codes spread back over all ``in_features`` columns, the outlier columns zero.

        With it the GEMM runs on the activations as they are: a zero code adds nothing to the fp32 sum, so
        ``x @ full.T`` equals ``x[:, normal_cols] @ int8_weights.T`` exactly, and the ``[M, in - n_outliers]``
        re-packing of the activations (a pass over all of x per call) is not needed -- only the few outlier
        columns are gathered.  Rows are ``in_features`` bytes, normally a multiple of 16 where
        ``in_features - n_outliers`` is not.  ``state_dict()`` keeps the reference's compact
        ``[out, in - n_outliers]`` buffer; this copy lives only in the cache."""
        src, cols = self.int8_weights, self.normal_cols

        def build():
            full = torch.zeros((src.shape[0], self.in_features), dtype=torch.int8, device=dev)
            full.index_copy_(1, cols.to(dev), src.to(dev))
            return full

        return self._cached(("int8_weights_full_k", dev), (src, cols), build)

    def _padded_outlier_weights(self, dev: torch.device, dtype: torch.dtype, width: int) -> torch.Tensor:
        """``outlier_weights`` in the activation dtype with zero columns up to ``width`` (a multiple of 8, so that
        rows are whole 16-byte chunks for the side product)."""
        src = self.outlier_weights

        def build():
            padded = torch.zeros((src.shape[0], width), dtype=dtype, device=dev)
            padded[:, : src.shape[1]].copy_(src)
            return padded

        return self._cached(("outlier_weights_padded", dev, dtype, width), (src,), build)

    def forward(self, x: torch.Tensor):
        """``y = x @ dequant(W).T (+ outlier columns in 16-bit) (+ bias)`` on the GPU, shape ``[..., out]``.

        The result is rounded to the activation dtype where the reference's forward materialises a
        tensor -- after the GEMM, after the scales, after adding the outlier product, after the bias
        (cublade/quantization/linear.py:97-135) -- inside the one fused kernel."""
        if not x.is_cuda:
            raise ValueError(
                f"cuBladeW8A16LinearLayer.forward: input must be on CUDA, got device={x.device} "
                "(this build has no CPU path)"
            )
        lead = x.shape[:-1]
        x2d = x.reshape(-1, self.in_features)
        if x2d.stride(-1) != 1:
            x2d = x2d.contiguous()
        dev = x2d.device
        scales = self._on("scales", dev)
        bias = None
        if self.bias is not None:
            bias = self.bias.detach()
            if bias.device != dev:
                bias = bias.to(dev)
            bias = bias.contiguous()

        if self.handle_outliers and self.outlier_cols is not None and len(self.outlier_cols) > 0:
            outlier_idx = self._on("outlier_cols", dev)
            ko = (len(self.outlier_cols) + 7) // 8 * 8
            x_out = gather_columns(x2d, outlier_idx, pad_to=ko)
            y2d = w8a16_linear(x2d, self._full_k_weights(dev), scales, bias, x_out,
                               self._padded_outlier_weights(dev, x2d.dtype, ko))
        elif self.in_features % 16 and x2d.shape[0] > 16:
            width = (self.in_features + 15) // 16 * 16
            every = self._dev_cache.get(("arange", dev))
            if every is None:
                every = self._dev_cache[("arange", dev)] = torch.arange(self.in_features, device=dev)
            y2d = w8a16_linear(gather_columns(x2d, every, pad_to=width), self._padded_weights(dev, width), scales, bias)
        else:
            y2d = w8a16_linear(x2d, self._on("int8_weights", dev), scales, bias)
        return y2d.view(*lead, self.out_features)


# lower-case-b spelling of the same class, used by some callers
cubladeW8A16LinearLayer = cuBladeW8A16LinearLayer
