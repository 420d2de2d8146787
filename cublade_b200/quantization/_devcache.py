"""Per-layer cache of device copies of a quantized layer's buffers.

``quantize_model`` on a CPU-resident model leaves the quantized buffers on the CPU (as the reference does,
cublade/quantization/linear.py:26-33); a forward on a GPU must not upload them on every call.  A copy is kept per
(buffer, device, dtype) and dropped when the buffer object is replaced or written in place.
"""
from __future__ import annotations

import torch


class DeviceBufferCache:
    """Mixin for ``nn.Module`` layers; the module sets ``self._dev_cache = {}`` in ``__init__``."""

    def _on(self, name: str, dev: torch.device, dtype=None) -> torch.Tensor:
        """Buffer ``name`` on ``dev`` (and cast to ``dtype``), cached while the buffer object is unchanged."""
        src = getattr(self, name)
        if src.device == dev and (dtype is None or src.dtype == dtype) and src.is_contiguous():
            return src
        return self._cached((name, dev, dtype), (src,),
                            lambda: src.to(device=dev, dtype=dtype if dtype is not None else src.dtype).contiguous())

    def _cached(self, key, sources, build):
        """Derived device tensor ``key``, rebuilt when one of the ``sources`` buffers was replaced or written."""
        stamp = tuple((id(t), t._version) for t in sources)
        hit = self._dev_cache.get(key)
        if hit is not None and hit[0] == stamp and all(a is b for a, b in zip(hit[1], sources)):
            return hit[2]
        made = build()
        self._dev_cache[key] = (stamp, tuple(sources), made)
        return made
