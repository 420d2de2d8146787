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

For the W8A16 layer the reference's arithmetic is Python + Triton
(``cublade/quantization/linear.py``, ``cublade/bindings/triton/matmul.py``), so there is nothing
to compile ahead of time: ``install_package`` pip-installs the unmodified reference into
``oracle/_ref/site`` (a build product, like the ``.so`` files beside it) so that a GPU box
without the checkout can ``import cublade`` and run the reference's own
``cuBladeW8A16LinearLayer`` -- which ``tests/golden/make_ref_w8a16_golden.py`` does to record the
layer's real outputs.  ``prebuild_jit`` warms the reference loader's JIT cache for the one CUDA
module that layer's ``quantize()`` needs, with the loader's own name, flags and source path, so
the box does not spend minutes compiling it.

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
    install_package(reference)
    prebuild_jit(verbose)


SITE = OUT / "site"          # pip --target directory holding the installed reference package
JIT_CACHE = OUT / "torch_ext"  # TORCH_EXTENSIONS_DIR for the reference's own JIT loader


def install_package(reference: Path) -> Path:
    """``pip install --no-deps --target oracle/_ref/site`` of the unmodified reference.

    The checkout is read-only and setuptools writes ``build/`` and ``*.egg-info`` beside
    ``pyproject.toml``, so the wheel is built from a temporary copy."""
    import shutil
    import subprocess
    import tempfile

    if (SITE / "cublade" / "quantization" / "linear.py").exists():
        return SITE
    with tempfile.TemporaryDirectory() as tmp:
        copy = Path(tmp) / "cublade_src"
        shutil.copytree(reference, copy, ignore=shutil.ignore_patterns(".git"))
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
               "--find-links", "/opt/wheelhouse", "--target", str(SITE), str(copy)]
        subprocess.run(cmd, check=True, capture_output=True)
    print(f"[oracle/_ref] installed the reference package into {SITE}", flush=True)
    return SITE


def reference_env() -> dict:
    """Environment under which the installed reference is imported (here and on a GPU box): its
    import-time warm-up off, its JIT cache inside ``oracle/_ref``, and a fixed arch list so that
    the compile command -- and with it ninja's up-to-date check -- is the same on both machines."""
    return {"CUBLADE_SKIP_WARMUP": "1", "TORCH_EXTENSIONS_DIR": str(JIT_CACHE), "TORCH_CUDA_ARCH_LIST": "10.0",
            "MAX_JOBS": "8"}


def prebuild_jit(verbose: bool = False) -> None:
    """Compile ``cublade_quantize_int8`` into the JIT cache exactly as ``cublade/_loader.py:92-111``
    would on a B200 (``-arch=sm_100``, no fast-math for the INT8 module)."""
    if not SITE.exists():
        return
    os.environ.update(reference_env())
    from torch.utils.cpp_extension import load

    csrc = SITE / "cublade" / "kernels" / "cuda"
    name = "cublade_quantize_int8"
    if (JIT_CACHE / name / f"{name}.so").exists():
        return
    load(name=name, sources=[str(csrc / "quantization" / "quantize_int8.cu")],
         extra_cuda_cflags=["-O3", "-std=c++17", "-arch=sm_100", "--expt-relaxed-constexpr"],
         extra_include_paths=[str(csrc)], extra_ldflags=None, verbose=verbose)
    print(f"[oracle/_ref] JIT cache warmed for {name}", flush=True)


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
