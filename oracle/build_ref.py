"""Build recipe for the reference's own quantization CUDA extensions (test infrastructure).

Compiles the four reference translation units *where they lie* in a read-only
checkout of emre570/cublade (``cublade/kernels/cuda/quantization/*.cu``) into
``oracle/_ref/`` as importable torch extensions.  Nothing is copied: nvcc reads
the sources in place and only the built ``.so`` files land in ``oracle/_ref``.

Flags follow the reference's own loader (``cublade/_loader.py:96-103``): ``-O3
-std=c++17 -arch=sm_100 --expt-relaxed-constexpr``; the FP8 modules add
``--use_fast_math`` because their bindings take the loader default
(``bindings/cuda/quantize_fp8.py:11-12``, ``dequantize_fp8.py:11-12``) while the
INT8 bindings switch it off (``bindings/cuda/quantize_int8.py:11-15``).

The products are GPU-only (the reference has no CPU path for these ops) and are
used exclusively by ``tests/`` as a second, device-side checker and by
``tests/golden/make_ref_gpu_golden.py`` to record the reference's real outputs.
The shipped package never imports them.

Usage:  python oracle/build_ref.py [--reference /path/to/cublade]
"""
from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"

# module name -> (source file relative to the reference root, fast-math flag)
MODULES = {
    "cublade_quantize_per_tensor_fp8": ("cublade/kernels/cuda/quantization/quantize_per_tensor_fp8.cu", True),
    "cublade_dequantize_per_tensor_fp8": ("cublade/kernels/cuda/quantization/dequantize_per_tensor_fp8.cu", True),
    "cublade_quantize_int8": ("cublade/kernels/cuda/quantization/quantize_int8.cu", False),
    "cublade_dequantize_int8": ("cublade/kernels/cuda/quantization/dequantize_int8.cu", False),
}


def built(name: str) -> bool:
    return (OUT / name / f"{name}.so").exists()


def build_all(reference: Path, verbose: bool = False) -> None:
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ.setdefault("MAX_JOBS", "8")
    from torch.utils.cpp_extension import load

    inc = reference / "cublade/kernels/cuda"
    for name, (rel, fast) in MODULES.items():
        if built(name):
            continue
        bdir = OUT / name
        bdir.mkdir(parents=True, exist_ok=True)
        flags = ["-O3", "-std=c++17", "-arch=sm_100", "--expt-relaxed-constexpr"]
        if fast:
            flags.insert(3, "--use_fast_math")
        load(
            name=name,
            sources=[str(reference / rel)],
            extra_cuda_cflags=flags,
            extra_include_paths=[str(inc)],
            build_directory=str(bdir),
            verbose=verbose,
            is_python_module=True,
        )
        print(f"[oracle/_ref] built {name}", flush=True)


def load_ref(name: str):
    """Import a prebuilt reference extension from ``oracle/_ref`` (never rebuilds)."""
    import importlib.util

    import torch  # libtorch must be loaded before the extension

    # Loading these extensions before the CUDA context exists crashed the first CUDA call on
    # the GPU box, so bring the context up first.
    if torch.cuda.is_available():
        torch.cuda.init()
        torch.zeros(1, device="cuda")

    so = OUT / name / f"{name}.so"
    if not so.exists():
        raise FileNotFoundError(f"{so} not built; run oracle/build_ref.py where the reference checkout exists")
    spec = importlib.util.spec_from_file_location(name, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("CUBLADE_REFERENCE", str(HERE.parents[1] / "reference")))
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    ref = Path(a.reference)
    if not ref.exists():
        print(f"reference checkout {ref} not found; nothing built", file=sys.stderr)
        sys.exit(0)
    build_all(ref, a.verbose)
