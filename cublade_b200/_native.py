"""ctypes loader for ``libcublade_b200.so`` (the C ABI declared in ``include/cublade_b200.h``).

There is no CPU or PyTorch fallback: if the shared library is missing or does
not export a declared symbol, importing an op raises ``RuntimeError``.  PyTorch
is used only for device memory, streams and the current-device guard.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_char_p, c_float, c_int32, c_int64, c_size_t, c_void_p
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "libcublade_b200.so"

CB_F16, CB_BF16, CB_F32 = 0, 1, 2
CODE_INT8, CODE_E4M3 = 0, 1

_DTYPE_CODE = {torch.float16: CB_F16, torch.bfloat16: CB_BF16, torch.float32: CB_F32}

# status code -> exception type raised on the Python side.  Alignment / range /
# CUDA failures surface as RuntimeError like the reference's TORCH_CHECKs.
_STATUS_EXC = {1: ValueError, 2: ValueError, 3: RuntimeError, 4: RuntimeError, 5: RuntimeError, 6: RuntimeError,
               7: NotImplementedError}

# name -> (restype, argtypes); one entry per declaration in include/cublade_b200.h
SIGNATURES = {
    "cb_version": (c_int32, []),
    "cb_last_error": (c_char_p, []),
    "cb_launch_count": (c_int64, []),
    "cb_per_tensor_scratch_floats": (c_int32, []),
    "cb_quantize_per_tensor_fp8": (c_int32, [c_void_p, c_int32, c_int64, c_float, c_void_p, c_void_p, c_void_p, c_void_p]),
    "cb_dequantize_per_tensor_fp8": (c_int32, [c_void_p, c_void_p, c_int64, c_int32, c_void_p, c_void_p]),
    "cb_quantize_per_tensor_int8": (c_int32, [c_void_p, c_int32, c_int64, c_float, c_void_p, c_void_p, c_void_p, c_void_p]),
    "cb_quantize_per_channel_int8": (c_int32, [c_void_p, c_int32, c_int64, c_int64, c_float, c_void_p, c_void_p, c_void_p]),
    "cb_quantize_per_group_int8": (c_int32, [c_void_p, c_int32, c_int64, c_int64, c_float, c_void_p, c_void_p, c_void_p]),
    "cb_dequantize_per_tensor_int8": (c_int32, [c_void_p, c_void_p, c_int64, c_int32, c_void_p, c_void_p]),
    "cb_dequantize_per_channel_int8": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int32, c_void_p, c_void_p]),
    "cb_dequantize_per_group_int8": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int32, c_void_p, c_void_p]),
    "cb_amax_abs": (c_int32, [c_void_p, c_int32, c_int64, c_void_p, c_void_p]),
    "cb_cast_per_tensor": (c_int32, [c_void_p, c_int32, c_int64, c_void_p, c_float, c_int32, c_void_p, c_void_p, c_void_p]),
    "cb_peer_exchange_state_bytes": (c_int32, []),
    "cb_peer_exchange_max_ranks": (c_int32, []),
    "cb_amax_peer_exchange": (c_int32, [c_void_p, c_void_p, c_int32, c_int32, c_void_p, c_void_p]),
    "cb_w8a16_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "cb_w8a16_linear": (c_int32, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int32, c_void_p,
                                   c_int32, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int32, c_void_p,
                                   c_size_t, c_int32, c_void_p]),
    "cb_device_error_state": (c_int32, [c_void_p, c_void_p]),
    "cb_static_scratch_bytes": (c_size_t, []),
    "cb_static_last_error": (c_char_p, []),
    "cb_w8a16_linear_outlier_static": (c_int32, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int64,
                                                  c_void_p, c_int64, c_void_p, c_int32, c_void_p, c_int32, c_void_p,
                                                  c_void_p, c_int64, c_int32, c_void_p]),
    "cb_gemm_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int32]),
    "cb_gemm": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int32, c_void_p, c_int64, c_int32, c_void_p,
                          c_size_t, c_void_p]),
    "cb_matmul": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int32, c_void_p, c_int64, c_int32, c_void_p,
                            c_size_t, c_void_p]),
    "cb_w4_quantize_rows": (c_int32, [c_void_p, c_int32, c_int64, c_int64, c_float, c_void_p, c_void_p, c_void_p]),
    "cb_w4_unpack": (c_int32, [c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "cb_w4a16_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "cb_w4a16_linear": (c_int32, [c_void_p, c_int32, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int32, c_void_p,
                                  c_int32, c_void_p, c_int64, c_void_p, c_size_t, c_void_p]),
    "cb_w8a8_linear": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int32, c_void_p,
                                 c_int32, c_void_p, c_int64, c_int32, c_void_p]),
    "cb_quantize_per_axis_int8": (c_int32, [c_void_p, c_int32, c_int64, c_int64, c_int64, c_float, c_void_p, c_void_p,
                                            c_void_p, c_void_p]),
    "cb_dequantize_per_axis_int8": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int32, c_void_p, c_void_p]),
    "cb_quantize_per_group_axis_int8": (c_int32, [c_void_p, c_int32, c_int64, c_int64, c_int64, c_int64, c_float, c_void_p,
                                                  c_void_p, c_void_p]),
    "cb_dequantize_per_group_axis_int8": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int32,
                                                    c_void_p, c_void_p]),
    "cb_rmsnorm_quantize": (c_int32, [c_void_p, c_int32, c_int64, c_int64, c_void_p, c_float, c_float, c_int32, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p]),
    "cb_gather_columns": (c_int32, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int32, c_void_p]),
    "cb_gather_columns_padded": (c_int32, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64,
                                           c_int32, c_void_p]),
}

_lib = None
_lock = threading.Lock()


def lib() -> ctypes.CDLL:
    """The loaded library; raises RuntimeError (never falls back) when it cannot be loaded."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH.name} is not built; run `python -m cublade_b200.build` (needs nvcc). "
                "cublade_b200 has no CPU or PyTorch fallback."
            )
        try:
            handle = ctypes.CDLL(str(LIB_PATH))
        except OSError as exc:  # pragma: no cover - depends on the machine
            raise RuntimeError(f"cannot load {LIB_PATH}: {exc}") from exc
        for name, (res, args) in SIGNATURES.items():
            try:
                fn = getattr(handle, name)
            except AttributeError as exc:
                raise RuntimeError(f"{LIB_PATH.name} does not export {name}; rebuild it") from exc
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


_scratch_floats = None


def per_tensor_scratch_floats() -> int:
    """Floats of device scratch the one-call per-tensor quantizers need."""
    global _scratch_floats
    if _scratch_floats is None:
        _scratch_floats = int(lib().cb_per_tensor_scratch_floats())
    return _scratch_floats


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise ValueError(f"unsupported dtype {dt}") from None


def check(status: int) -> None:
    """Turn a non-zero cb_status into the matching Python exception."""
    if status == 0:
        return
    msg = lib().cb_last_error().decode("utf-8", "replace")
    raise _STATUS_EXC.get(status, RuntimeError)(msg)


def stream_ptr(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def launch_count() -> int:
    return int(lib().cb_launch_count())


def device_error_state(device=None) -> int:
    """Synchronise the current stream and return the device's bounded-wait flag (0 = healthy)."""
    flag = ctypes.c_uint32(0)
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        check(lib().cb_device_error_state(ctypes.byref(flag), torch.cuda.current_stream(dev).cuda_stream))
    return int(flag.value)


def ptr(t):
    return None if t is None else t.data_ptr()


class _NoGuard:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def device_guard(t: torch.Tensor):
    """Context manager that makes ``t``'s device current; free when it already is."""
    idx = t.device.index
    if idx is None or idx == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(idx)
