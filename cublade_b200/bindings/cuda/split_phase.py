"""The two phases of per-tensor quantization as separate calls, for tensors sharded over GPUs.

``amax_abs`` is the first kernel of the reference's per-tensor quantizers and ``cast_per_tensor`` the
second (cublade/kernels/cuda/quantization/quantize_per_tensor_fp8.cu:140-159,
quantize_int8.cu:394-410); between them a caller max-reduces the fp32 amax across ranks -- with a collective of its
own, or with ``amax_peer_exchange`` (peer-memory stores over NVLink, one small kernel per rank).
"""
from __future__ import annotations

import torch

from ... import _native as N
from ._common import check_quant_input

_CODE = {torch.int8: N.CODE_INT8, torch.float8_e4m3fn: N.CODE_E4M3}


def amax_abs(x: torch.Tensor) -> torch.Tensor:
    """``max |x|`` of a contiguous CUDA tensor as a 1-element float32 tensor (NaNs are ignored)."""
    check_quant_input(x, (torch.float16, torch.bfloat16, torch.float32), "torch.float16, torch.bfloat16, or torch.float32")
    with N.device_guard(x):
        amax = torch.zeros(1, dtype=torch.float32, device=x.device)
        N.check(N.lib().cb_amax_abs(x.data_ptr(), N.dtype_code(x.dtype), x.numel(), amax.data_ptr(), N.stream_ptr(x)))
    return amax


def cast_per_tensor(x: torch.Tensor, amax: torch.Tensor, dtype: torch.dtype, eps: float = 1e-12):
    """Quantize ``x`` with a given (global) amax: returns ``(q, scale)`` like the one-call quantizers."""
    if dtype not in _CODE:
        raise ValueError(f"cast_per_tensor: dtype must be torch.int8 or torch.float8_e4m3fn, got {dtype}")
    allowed = (torch.float16, torch.bfloat16) if dtype == torch.float8_e4m3fn else (torch.float16, torch.bfloat16, torch.float32)
    check_quant_input(x, allowed, " or ".join(str(a) for a in allowed))
    if amax.dtype != torch.float32 or amax.numel() != 1 or amax.device != x.device:
        raise ValueError("cast_per_tensor: amax must be a 1-element float32 tensor on x's device")
    with N.device_guard(x):
        q = torch.empty(x.shape, dtype=dtype, device=x.device)
        scale = torch.empty((), dtype=torch.float32, device=x.device)
        N.check(N.lib().cb_cast_per_tensor(x.data_ptr(), N.dtype_code(x.dtype), x.numel(), amax.data_ptr(), float(eps),
                                           _CODE[dtype], q.data_ptr(), scale.data_ptr(), N.stream_ptr(x)))
    return q, scale


def amax_peer_exchange(local_amax: torch.Tensor, peer_state_ptrs, rank: int) -> torch.Tensor:
    """Maximum of the ranks' ``local_amax`` through peer memory: ``peer_state_ptrs[r]`` is the address, in THIS process,
    of rank ``r``'s state array (``peer_exchange_state_bytes()`` bytes, zeroed once before the first exchange).  Every
    rank must call it once per exchange; the kernels wait for one another with a bounded wait (NaN and the device
    error flag when a peer does not arrive)."""
    import ctypes

    if local_amax.dtype != torch.float32 or local_amax.numel() != 1 or not local_amax.is_cuda:
        raise ValueError("amax_peer_exchange: local_amax must be a 1-element float32 CUDA tensor")
    world = len(peer_state_ptrs)
    ptrs = (ctypes.c_void_p * world)(*[int(p) for p in peer_state_ptrs])
    with N.device_guard(local_amax):
        out = torch.empty(1, dtype=torch.float32, device=local_amax.device)
        N.check(N.lib().cb_amax_peer_exchange(local_amax.data_ptr(), ptrs, int(rank), world, out.data_ptr(),
                                              N.stream_ptr(local_amax)))
    return out


def peer_exchange_state_bytes() -> int:
    return int(N.lib().cb_peer_exchange_state_bytes())
