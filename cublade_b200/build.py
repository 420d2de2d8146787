"""Ahead-of-time build of ``libcublade_b200.so`` for sm_100a.

``python -m cublade_b200.build`` compiles every ``csrc/*.cu`` with nvcc
(``-gencode arch=compute_100a,code=sm_100a``, no fast-math, no FMA contraction
in the quantizers) and links one shared library next to the package.  nvcc
cross-compiles, so no GPU is needed to build.  The library has no torch or
Python dependency; the CUDA runtime is linked statically.
"""
from __future__ import annotations

import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "_build"
LIB = PKG / "libcublade_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-fmad=false",  # the bit-exact quantizers must never contract mul+add
]
# translation units where FMA contraction is wanted (fp32 accumulate GEMMs)
FMAD_OK = {"w8a16_stream.cu", "w8a16_tc.cu"}


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; cannot build libcublade_b200.so")
    return cand


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build(verbose: bool = False, force: bool = False) -> Path:
    nvcc = _nvcc()
    OBJ.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((PKG.parent / "include").glob("*.h"))
    sources = sorted(CSRC.glob("*.cu"))
    jobs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        flags = [f for f in NVCC_FLAGS if not (src.name in FMAD_OK and f == "-fmad=false")]
        # an object built with other flags is stale too: the flags it was built with sit beside it
        stamp = obj.with_suffix(".flags")
        same_flags = stamp.exists() and stamp.read_text() == " ".join(flags)
        if force or verbose or not same_flags or _stale(obj, [src, *headers]):
            cmd = [nvcc, *flags, "-Xptxas", "-v" if verbose else "-O3", "-c", str(src), "-o", str(obj)]
            jobs.append((src, cmd, stamp, " ".join(flags)))

    def run(job):
        src, cmd, stamp, flag_text = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode == 0:
            stamp.write_text(flag_text)
        return src, r

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for src, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(f"--- {src.name}\n{r.stdout}{r.stderr}\n")
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}")
    objs = [OBJ / (s.stem + ".o") for s in sources]
    if force or jobs or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
               "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link of libcublade_b200.so failed")
    return LIB


if __name__ == "__main__":
    lib = build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(lib)
