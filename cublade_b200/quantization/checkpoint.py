"""Saving and restoring quantized models.

The reference has no checkpoint feature: a quantized layer's state simply is its registered buffers
(``int8_weights [out, in] int8``, ``scales [out]``, ``outlier_weights``, ``normal_cols``, ``outlier_cols``) and
``bias`` (cublade/quantization/linear.py:25-33), so ``model.state_dict()`` is the on-disk format and stays
interchangeable with the reference's.  Two quirks of that layout make a plain ``load_state_dict`` into a freshly
built model fail, and are handled here:

* buffers that are ``None`` are absent from ``state_dict()`` -- a new layer has no ``outlier_*`` entries, the
  checkpoint of an outlier-aware layer has them (unexpected keys);
* in outlier mode ``int8_weights`` is re-bound to a narrower ``[out, in - n_outliers]`` tensor
  (linear.py:66), which does not match the ``[out, in]`` buffer of a new layer (size mismatch).

``load_quantized_state_dict`` re-binds the buffers of every quantized layer to what the checkpoint holds before
loading; with ``rank`` / ``world_size`` it keeps only that rank's block of output features (the column-parallel
layout of ``cublade_b200.sharding``).  Nothing here touches a GPU.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn

FORMAT_VERSION = 1
_ROW_SHARDED = ("int8_weights", "int4_weights", "scales", "outlier_weights", "bias")
_REPLICATED = ("normal_cols", "outlier_cols")


def _quantized_layers(model: nn.Module):
    from .linear import cuBladeW8A16LinearLayer
    from .linear_w4a16 import cuBladeW4A16LinearLayer
    from .linear_w8a8 import cuBladeW8A8LinearLayer

    for name, module in model.named_modules():
        if isinstance(module, (cuBladeW8A16LinearLayer, cuBladeW8A8LinearLayer, cuBladeW4A16LinearLayer)):
            yield name, module


def quantized_layer_manifest(model: nn.Module) -> Dict[str, Dict[str, Any]]:
    """What is needed to rebuild the quantized layers of ``model`` without the original weights."""
    from .linear_w4a16 import cuBladeW4A16LinearLayer
    from .linear_w8a8 import cuBladeW8A8LinearLayer

    out = {}
    for name, m in _quantized_layers(model):
        out[name] = {
            "quant_type": ("w8a8" if isinstance(m, cuBladeW8A8LinearLayer) else
                           "w4a16" if isinstance(m, cuBladeW4A16LinearLayer) else "w8a16"),
            "in_features": m.in_features, "out_features": m.out_features, "bias": m.bias is not None,
            "dtype": str(m.scales.dtype).replace("torch.", ""),
            "handle_outliers": bool(getattr(m, "handle_outliers", False)),
            "outlier_threshold": float(getattr(m, "outlier_threshold", 6.0)),
        }
    return out


def save_quantized_model(model: nn.Module, path) -> None:
    """``torch.save`` of ``{"format_version", "layers": manifest, "state_dict": model.state_dict()}``; the
    ``state_dict`` part alone is what the reference's layers would save."""
    torch.save({"format_version": FORMAT_VERSION, "layers": quantized_layer_manifest(model),
                "state_dict": {k: v.detach().cpu() for k, v in model.state_dict().items()}}, path)


def build_quantized_skeleton(model: nn.Module, manifest: Dict[str, Dict[str, Any]]) -> nn.Module:
    """Swap the ``nn.Linear`` modules named in ``manifest`` for empty quantized layers (no quantization is run)."""
    from .quantizers import QUANT_LAYER_REGISTRY, _init_registry

    _init_registry()
    for name, meta in manifest.items():
        parent_name, _, leaf = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        old = getattr(parent, leaf)
        if not isinstance(old, nn.Linear):
            continue  # already a quantized layer
        kwargs = {}
        if meta["quant_type"] == "w8a16":
            kwargs = {"handle_outliers": meta["handle_outliers"], "outlier_threshold": meta["outlier_threshold"]}
        layer = QUANT_LAYER_REGISTRY[meta["quant_type"]](meta["in_features"], meta["out_features"], bias=meta["bias"],
                                                          dtype=getattr(torch, meta["dtype"]), **kwargs)
        setattr(parent, leaf, layer)
    return model


def load_quantized_state_dict(model: nn.Module, state_dict: Dict[str, torch.Tensor], rank: int = 0,
                              world_size: int = 1, strict: bool = True):
    """``model.load_state_dict`` that copes with the two layout quirks described in the module docstring.

    With ``world_size > 1`` every quantized layer keeps rows ``shard_range(out_features, rank, world_size)`` of
    ``int8_weights`` / ``scales`` / ``outlier_weights`` / ``bias`` (column index buffers are replicated) and its
    ``out_features`` shrinks accordingly; other modules load unsharded.  Returns what ``load_state_dict`` returns.
    """
    from ..sharding import shard_range

    if not 0 <= rank < world_size:
        raise ValueError(f"load_quantized_state_dict: rank {rank} outside world of {world_size}")
    sd = dict(state_dict)
    for name, layer in _quantized_layers(model):
        prefix = f"{name}." if name else ""
        rows = None
        if world_size > 1:
            full_out = sd[prefix + "int8_weights"].shape[0] if prefix + "int8_weights" in sd else layer.out_features
            rows = shard_range(full_out, rank, world_size)
        for key in _ROW_SHARDED + _REPLICATED:
            full = prefix + key
            if full not in sd:
                if key.startswith("outlier") or key == "normal_cols":
                    if hasattr(layer, key) and key in layer._buffers:
                        layer._buffers[key] = None  # the checkpoint's layer had no outliers
                continue
            t = sd[full]
            if rows is not None and key in _ROW_SHARDED:
                t = t[rows[0]:rows[1]].contiguous()
                sd[full] = t
            if key == "bias":
                if layer.bias is None or layer.bias.shape != t.shape:
                    layer.bias = nn.Parameter(torch.empty_like(t), requires_grad=False)
            elif key in layer._buffers:
                cur = layer._buffers[key]
                if cur is None or cur.shape != t.shape or cur.dtype != t.dtype:
                    layer._buffers[key] = torch.empty_like(t)  # narrower int8_weights, outlier buffers, a shard ...
            else:
                raise KeyError(f"load_quantized_state_dict: layer '{name}' has no buffer '{key}'")
        if rows is not None:
            layer.out_features = rows[1] - rows[0]
            layer.shard = (rank, world_size, rows[0], rows[1])
        if hasattr(layer, "_dev_cache"):
            layer._dev_cache = {}
    return model.load_state_dict(sd, strict=strict)


def load_quantized_model(model: nn.Module, path, rank: int = 0, world_size: int = 1, map_location="cpu") -> nn.Module:
    """Rebuild a quantized model from ``save_quantized_model``'s file: ``model`` is the unquantized architecture
    (its Linear weights are discarded), the quantized layers are created empty from the manifest and filled from the
    file; ``rank`` / ``world_size`` as in ``load_quantized_state_dict``."""
    blob = torch.load(path, map_location=map_location, weights_only=True)
    if blob.get("format_version") != FORMAT_VERSION:
        raise ValueError(f"load_quantized_model: unknown format_version {blob.get('format_version')!r}")
    build_quantized_skeleton(model, blob["layers"])
    load_quantized_state_dict(model, blob["state_dict"], rank=rank, world_size=world_size)
    return model
