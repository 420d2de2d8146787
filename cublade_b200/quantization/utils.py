"""Module surgery used by ``quantize_model`` (mirrors cublade/quantization/utils.py:8-68)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Type

import torch
import torch.nn as nn

__all__ = ["replace_linear_layers"]


def replace_linear_layers(
    module: nn.Module,
    target_class: Type[nn.Module],
    target_modules: Optional[List[str]] = None,
    exclude_modules: Optional[List[str]] = None,
    quant_kwargs: Optional[Dict[str, Any]] = None,
    _parent_name: str = "",
):
    """Walk ``module`` depth-first and swap each selected ``nn.Linear`` for ``target_class``.

    Selection is by substring of the dotted module path: a layer is skipped when any entry
    of ``exclude_modules`` occurs in its path, or when ``target_modules`` is given and none
    of its entries occurs.  The replacement is constructed as
    ``target_class(in_features, out_features, bias=<had bias>, dtype=<weight dtype>, **quant_kwargs)``
    on the device of the layer it replaces, attached first, then asked to ``quantize(old_weight)``; the original bias ``Parameter``
    object is re-attached afterwards.
    """
    quant_kwargs = quant_kwargs or {}
    exclude_modules = exclude_modules or []

    for name, child in list(module.named_children()):
        path = f"{_parent_name}.{name}" if _parent_name else name
        if not isinstance(child, nn.Linear):
            replace_linear_layers(child, target_class, target_modules, exclude_modules, quant_kwargs,
                                  _parent_name=path)
            continue
        if any(pat in path for pat in exclude_modules):
            continue
        if target_modules is not None and not any(pat in path for pat in target_modules):
            continue
        weight, bias = child.weight, child.bias
        # the replacement's buffers are created where the weight lives, so the codes of a GPU-resident model
        # stay on the GPU (created on the CPU, as the reference does, every layer's codes would cross PCIe
        # twice: back to the host here and up again on the first forward)
        with torch.device(weight.device):
            replacement = target_class(child.in_features, child.out_features, bias=bias is not None,
                                       dtype=weight.dtype, **quant_kwargs)
        setattr(module, name, replacement)
        getattr(module, name).quantize(weight)
        if bias is not None:
            getattr(module, name).bias = bias
