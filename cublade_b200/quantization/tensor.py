"""Container returned by ``quantize_tensor`` (mirrors cublade/quantization/tensor.py:5-14)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class QuantizedTensor:
    """Quantized codes plus everything ``dequantize_tensor`` needs.

    ``group_size`` is recorded for every mode (it is simply the argument that was
    passed, default 32), and ``zero_point`` is a 0-d float32 zero because only the
    symmetric scheme exists.
    """

    data: torch.Tensor
    scale: torch.Tensor
    zero_point: torch.Tensor
    mode: str
    axis: int
    group_size: Optional[int]
    dtype: torch.dtype
    original_dtype: torch.dtype
