"""``matmul(A, B, activation="", override_config=None, use_autotune=True)``: the generic GEMM wrapper the W8A16 layer of
the reference calls (cublade/bindings/triton/matmul.py:17-132, kernel cublade/kernels/triton/matmul_kernel.py:9-105),
served by this library's tcgen05 GEMM (``cb_matmul``) instead of a Triton kernel.

Same contract for the dtypes served: ``C = A @ B`` with ``C`` in the input dtype for float16 / bfloat16 (float32
accumulation, optional ``leaky_relu`` on the accumulator, one rounding) and int32 for int8 (the activation is ignored,
as there).  ``override_config`` and ``use_autotune`` select Triton tile shapes in the reference; they are accepted and
have no meaning here.  float32 and float8_e5m2 inputs, which the reference's table also lists, raise ``ValueError``.
"""
from __future__ import annotations

import torch

from ... import _native as N

_IN_KIND = {torch.float16: 0, torch.bfloat16: 1, torch.int8: 2}
_OUT_DTYPE = {torch.float16: torch.float16, torch.bfloat16: torch.bfloat16, torch.int8: torch.int32}


def matmul(A: torch.Tensor, B: torch.Tensor, activation: str = "", override_config=None, use_autotune=True) -> torch.Tensor:
    assert A.shape[1] == B.shape[0], "Incompatible dimensions"
    A = A.contiguous()
    B = B.contiguous()
    if A.device.type != "cuda" or B.device.type != "cuda":
        raise ValueError(f"Triton matmul requires CUDA tensors. Got A on {A.device}, B on {B.device}.")
    if A.device != B.device:
        raise ValueError(f"A and B must be on the same device. Got A on {A.device}, B on {B.device}.")
    if A.dtype != B.dtype or A.dtype not in _IN_KIND:
        raise ValueError(f"Unsupported dtype combination: A={A.dtype}, B={B.dtype}")
    if activation not in ("", "leaky_relu"):
        raise ValueError(f"Unsupported activation '{activation}'; expected '' or 'leaky_relu'")
    M, K = A.shape
    Nn = B.shape[1]
    with N.device_guard(A):
        C = torch.empty((M, Nn), dtype=_OUT_DTYPE[A.dtype], device=A.device)
        if M == 0 or Nn == 0:
            return C
        L = N.lib()
        ws_bytes = int(L.cb_gemm_workspace_bytes(Nn, K, _IN_KIND[A.dtype]))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=A.device)
        N.check(L.cb_matmul(A.data_ptr(), B.data_ptr(), M, Nn, K, _IN_KIND[A.dtype], C.data_ptr(), C.stride(0),
                            1 if activation == "leaky_relu" else 0, ws.data_ptr(), ws_bytes, N.stream_ptr(A)))
    return C
