"""``wmma_gemm``: dense GEMM with the reference's name and contract (cublade/bindings/cuda/wmma.py:16-47), served by
a tcgen05 / TMEM kernel instead of 16x16x16 WMMA fragments.

| input dtype | accumulator / output dtype |
|-------------|----------------------------|
| float16     | float32 (default), float16 |
| bfloat16    | float32                    |
| int8, uint8 | int32                      |
"""
from __future__ import annotations

from typing import Optional

import torch

from ... import _native as N
from ._common import require

_IN_KIND = {torch.float16: 0, torch.bfloat16: 1, torch.int8: 2, torch.uint8: 3}
_OUT_KIND = {torch.float32: 0, torch.float16: 1, torch.int32: 2}


def wmma_gemm(A: torch.Tensor, B: torch.Tensor, acc_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``C = A @ B`` for ``A [M, K]`` and ``B [K, N]`` of one dtype; ``C [M, N]`` has the accumulator dtype.

    Errors follow the reference's checks (cublade/kernels/cuda/wmma.cu:188-259): ``RuntimeError`` for CPU tensors,
    non-2-D inputs, mismatched shapes or dtypes, an unsupported dtype or accumulator pairing.  The reference's
    "multiples of 16" restriction is lifted."""
    require(isinstance(A, torch.Tensor) and isinstance(B, torch.Tensor) and A.is_cuda and B.is_cuda,
            "Inputs must be CUDA tensors")
    require(A.dim() == 2 and B.dim() == 2, "Inputs must be 2D matrices")
    require(A.size(1) == B.size(0), "Matrix dimensions incompatible for GEMM")
    require(A.dtype == B.dtype, "A and B must have the same dtype")
    require(A.dtype in _IN_KIND, "Unsupported dtype. Expected: float16, bfloat16, int8, or uint8")
    require(A.device == B.device, "A and B must be on the same device")
    if A.dtype == torch.float16:
        acc = acc_dtype or torch.float32
        require(acc in (torch.float32, torch.float16), "float16 inputs support float32 or float16 accumulator")
    elif A.dtype == torch.bfloat16:
        acc = acc_dtype or torch.float32
        require(acc == torch.float32, "bfloat16 inputs only support float32 accumulator")
    else:
        acc = acc_dtype or torch.int32
        require(acc == torch.int32, "int8 / uint8 inputs only support int32 accumulator")
    A, B = A.contiguous(), B.contiguous()
    M, K = A.shape
    Nn = B.shape[1]
    with N.device_guard(A):
        C = torch.empty((M, Nn), dtype=acc, device=A.device)
        if M == 0 or Nn == 0:
            return C
        require(K > 0, "K must be positive")
        L = N.lib()
        ws_bytes = int(L.cb_gemm_workspace_bytes(Nn, K, _IN_KIND[A.dtype]))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=A.device)
        N.check(L.cb_gemm(A.data_ptr(), B.data_ptr(), M, Nn, K, _IN_KIND[A.dtype], C.data_ptr(), C.stride(0),
                          _OUT_KIND[acc], ws.data_ptr(), ws_bytes, N.stream_ptr(A)))
    return C
