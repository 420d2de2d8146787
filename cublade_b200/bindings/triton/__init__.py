"""Counterpart of ``cublade.bindings.triton`` for the one wrapper on the quantization path: ``matmul``."""
from .matmul import matmul

__all__ = ["matmul"]
