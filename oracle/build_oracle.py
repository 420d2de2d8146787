"""Compile ``oracle_c.c`` into ``oracle/_build/liboracle_c.so`` with gcc (test infrastructure)."""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "oracle_c.c"
OUT = HERE / "_build" / "liboracle_c.so"


def build(force: bool = False) -> Path:
    if OUT.exists() and not force and OUT.stat().st_mtime >= SRC.stat().st_mtime:
        return OUT
    OUT.parent.mkdir(exist_ok=True)
    cmd = ["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC", str(SRC), "-o",
           str(OUT), "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


def load() -> ctypes.CDLL:
    """Build if needed and load with argument types set."""
    from ctypes import POINTER, c_double, c_float, c_int, c_int64, c_uint8, c_uint16, c_void_p

    lib = ctypes.CDLL(str(build()))
    lib.oc_fp8_quantize.argtypes = [c_void_p, c_int, c_int64, c_float, c_void_p, c_void_p]
    lib.oc_fp8_dequantize.argtypes = [c_void_p, c_void_p, c_int64, c_int, c_void_p]
    lib.oc_int8_quantize_segments.argtypes = [c_void_p, c_int, c_int64, c_int64, c_float, c_void_p, c_void_p]
    lib.oc_int8_quantize_tensor.argtypes = [c_void_p, c_int, c_int64, c_float, c_void_p, c_void_p]
    lib.oc_int8_dequantize.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]
    lib.oc_w8a16_forward.argtypes = [c_void_p, c_int, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_int64, c_void_p]
    lib.oc_probe_e4m3.argtypes = [c_float]
    lib.oc_probe_e4m3.restype = c_uint8
    lib.oc_probe_e4m3_decode.argtypes = [c_uint8]
    lib.oc_probe_e4m3_decode.restype = c_float
    lib.oc_probe_bf16.argtypes = [c_float]
    lib.oc_probe_bf16.restype = c_uint16
    lib.oc_probe_f16.argtypes = [c_float]
    lib.oc_probe_f16.restype = c_uint16
    lib.oc_probe_f16_decode.argtypes = [c_uint16]
    lib.oc_probe_f16_decode.restype = c_float
    _ = (POINTER, c_double)
    return lib


if __name__ == "__main__":
    print(build(force=True))
